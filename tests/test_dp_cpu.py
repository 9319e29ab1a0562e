"""Data-parallel gradient exchange on CPU: two gloo ranks, bucketed all-reduce in place."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from evt_ae_b200.dp import GradAllReducer
    g = torch.Generator().manual_seed(100 + rank)
    grads = {"w1": torch.randn(300, 17, generator=g), "b1": torch.randn(17, generator=g),
             "w2": torch.randn(1000, generator=g).to(torch.bfloat16), "emb": torch.randn(64, 8, generator=g)}
    mine = {k: v.clone() for k, v in grads.items()}
    red = GradAllReducer(grads, bucket_bytes=4096)       # forces several buckets
    assert len(red.buckets) >= 3
    for flat, entries in red.buckets:      # every tensor starts on a 256-byte boundary of its bucket
        assert (flat.numel() * flat.element_size()) % 256 == 0
        for _, off, _ in entries:
            assert (off * flat.element_size()) % 256 == 0
    red.allreduce(grads)
    # expected: mean over ranks, rebuilt from the seeds
    ok = True
    for k in grads:
        exp = torch.zeros_like(mine[k], dtype=torch.float32)
        for r in range(world):
            gr = torch.Generator().manual_seed(100 + r)
            all_r = {"w1": torch.randn(300, 17, generator=gr), "b1": torch.randn(17, generator=gr),
                     "w2": torch.randn(1000, generator=gr).to(torch.bfloat16), "emb": torch.randn(64, 8, generator=gr)}
            exp += all_r[k].float()
        exp /= world
        tol = 2e-2 if grads[k].dtype == torch.bfloat16 else 1e-6
        ok = ok and torch.allclose(grads[k].float(), exp, atol=tol, rtol=tol)
    q.put((rank, ok))
    dist.destroy_process_group()


def test_bucketed_allreduce_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]


def test_single_process_is_a_no_op():
    from evt_ae_b200.dp import GradAllReducer
    grads = {"a": torch.ones(5)}
    red = GradAllReducer(grads)
    red.allreduce(grads)
    assert torch.equal(grads["a"], torch.ones(5))
