"""Row partition of the GCN graph and the operand gather, two gloo ranks on CPU.

The fused SpMM has no CPU path, so this test checks what is host logic: the partition (blocks
cover the rows once, balanced work, local CSR consistent with the global one) and that a rank
which gathers the operand through `GcnShard.gather` and multiplies its row block (torch.sparse
here, the fused kernel on a GPU) gets exactly its rows of the unpartitioned product."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import partitions as P
from evt_ae_b200.workloads import gcn as wg


def _graph(n=3000, edges=14000):
    r, c = P.chung_lu_graph(n, edges)
    crow, col = P.csr_reference(r, c, n)
    deg = (crow[1:] - crow[:-1]).to(torch.float32)
    return crow, col, (deg + 1.0) ** -0.5


def test_partition_covers_rows_and_balances_work():
    crow, col, dinv = _graph()
    n = crow.shape[0] - 1
    for world in (1, 2, 4, 8):
        shards = wg.partition_rows(crow, col, dinv, world)
        assert shards[0]["r0"] == 0 and shards[-1]["r1"] == n
        work = []
        for a, b in zip(shards[:-1], shards[1:]):
            assert a["r1"] == b["r0"]
        for s in shards:
            rows = s["r1"] - s["r0"]
            assert s["crow"].shape[0] == rows + 1 and int(s["crow"][0]) == 0
            assert int(s["crow"][-1]) == s["col"].shape[0] == s["val"].shape[0]
            p0 = int(crow[s["r0"]])
            assert torch.equal(s["col"], col[p0:p0 + s["col"].shape[0]])
            work.append(s["col"].shape[0] + 8 * rows)
        assert max(work) <= 1.0 * sum(work) / world + (int((crow[1:] - crow[:-1]).max()) + 8), work


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    crow, col, dinv = _graph()
    n = crow.shape[0] - 1
    cfg = wg.GcnConfig(nodes=n, in_feats=32, hidden=64, classes=8)
    x = P.seeded((n, 32), 301, 1.0, torch.float32)
    shard = wg.partition_rows(crow, col, dinv, world)[rank]
    sh = wg.GcnShard(cfg, shard, world, "cpu", build_step=False)
    full, exchange = sh.gather(x[sh.r0:sh.r1].clone())
    exchange()
    ok = torch.equal(full, x)
    a_loc = torch.sparse_csr_tensor(sh.crow.to(torch.int64), sh.col.to(torch.int64), sh.val, size=(sh.rows, n))
    y_loc = torch.matmul(a_loc, full) + x[sh.r0:sh.r1]
    from oracle import gcn_ref
    y_ref = torch.matmul(gcn_ref.normalised_adjacency(crow, col, dinv), x) + x
    ok = ok and torch.allclose(y_loc, y_ref[sh.r0:sh.r1], rtol=1e-6, atol=1e-6)
    # loss / gradient reduction: sums over ranks
    flat, run, unpack = sh.reduce(torch.tensor(float(rank + 1)), {"w": torch.full((3, 2), float(rank + 1))})
    run()
    loss, grads = unpack()
    tot = world * (world + 1) / 2
    ok = ok and float(loss) == tot and bool((grads["w"] == tot).all())
    q.put((rank, bool(ok)))
    dist.destroy_process_group()


def test_gather_and_row_block_product_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]
