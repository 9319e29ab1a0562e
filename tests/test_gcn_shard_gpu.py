"""The row-partitioned GCN step on two GPUs (child processes, NCCL) against the fp32 autograd
oracle of the whole graph.  Skipped where fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    try:
        _worker_body(rank, world, port, q)
    except Exception:
        import traceback
        q.put((rank, "error", traceback.format_exc()))


def _worker_body(rank, world, port, q):
    import numpy as np
    import torch.distributed as dist
    import partitions as P
    from evt_ae_b200.workloads import gcn as wg
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    n, edges, F, H, C = 3000, 14000, 128, 256, 40
    cfg = wg.GcnConfig(nodes=n, in_feats=F, hidden=H, classes=C)
    r, c = P.chung_lu_graph(n, edges)
    crow, col = P.csr_reference(r, c, n)
    dinv = ((crow[1:] - crow[:-1]).to(torch.float32) + 1.0) ** -0.5
    x = P.seeded((n, F), 301, 1.0, torch.float32)
    labels = torch.from_numpy(np.random.default_rng(302).integers(0, C, size=n))
    params = wg.init_params(cfg, dtype=torch.bfloat16)
    shard = wg.partition_rows(crow, col, dinv, world)[rank]
    sh = wg.GcnShard(cfg, shard, world, dev)
    p = {k: v.to(dev) for k, v in params.items()}
    loss, grads = sh.step(p, x[sh.r0:sh.r1].to(dev), labels[sh.r0:sh.r1].to(dev))
    torch.cuda.synchronize()
    sh.check_status()
    q.put((rank, float(loss), {k: v.float().cpu().numpy() for k, v in grads.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_row_partitioned_step_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import numpy as np
    import partitions as P
    from evt_ae_b200.workloads import gcn as wg
    from oracle import gcn_ref
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in procs], key=lambda t: t[0])
    assert all(r[1] != "error" for r in res), [r[2] for r in res if r[1] == "error"]
    for p in procs:
        p.join(timeout=60)
    n, edges, F, H, C = 3000, 14000, 128, 256, 40
    cfg = wg.GcnConfig(nodes=n, in_feats=F, hidden=H, classes=C)
    r, c = P.chung_lu_graph(n, edges)
    crow, col = P.csr_reference(r, c, n)
    dinv = ((crow[1:] - crow[:-1]).to(torch.float32) + 1.0) ** -0.5
    x = P.seeded((n, F), 301, 1.0, torch.float32)
    labels = torch.from_numpy(np.random.default_rng(302).integers(0, C, size=n))
    ref_loss, ref_grads = gcn_ref.loss_and_grads(wg.init_params(cfg, dtype=torch.bfloat16), crow, col, dinv, x, labels)
    for rank, loss, grads in res:            # every rank holds the reduced loss and gradients
        assert abs(loss - ref_loss.item()) <= 2e-2 * abs(ref_loss.item()), (rank, loss, ref_loss.item())
        for k, rg in ref_grads.items():
            g = torch.from_numpy(grads[k]).reshape(rg.shape)
            assert (g - rg).norm() / (rg.norm() + 1e-12) <= 5e-2, (rank, k)
