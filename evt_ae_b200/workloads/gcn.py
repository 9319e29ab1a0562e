"""Two-layer GCN training step on fused nodes (BASELINE configuration 4).

Model (python/model_zoo/gcn/gcn_modeling.py:120-160 of the reference, `GraphConv`): a layer
whose output is wider than its input aggregates first, `h = A_hat x + x`, then applies the
linear map; a layer whose output is narrower applies the linear map first and aggregates
after; ReLU between the layers; cross-entropy over all nodes.  A_hat = D^-1/2 A D^-1/2 with
the normalisation fused into the SpMM (the reference materialises the products as edge values
on the host, python/model_zoo/gcn/gcn.py:57-62).  The graph is symmetric, so the backward
aggregation uses the same CSR (the reference keeps a CSC copy for the general case).

Fused nodes: SpMM (+ self term, + cast), linear + bias + ReLU, linear + bias, softmax - one-hot
(loss gradient), data gradient with the ReLU mask, two split-K weight gradients; the bias
gradients are column sums.  Features enter in fp32 (the configuration's dtype) and the first
aggregation runs in fp32; the dense maps and the 40-wide second aggregation run on bf16 storage
with fp32 accumulation.

The step has no edge gradients: the normalised adjacency is a constant of the graph, not a
parameter, so nothing is differentiated with respect to edge values (an SDDMM would compute
exactly those; `ops.sddmm` is provided and tested for models with learnable edge weights).

Multi-GPU (`GcnShard`): 1-D partition of the destination rows into contiguous blocks balanced by
nonzeros (hub rows sit at the front of a power-law graph); every rank owns its rows of A, of the
features and of every activation.  Before each aggregation the ranks all-gather the operand into
a local buffer of all rows (every rank broadcasts its block into its slice), so the SpMM only
ever reads local memory and column indices stay global.  Weight and bias gradients and the loss
are all-reduced.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..fused_ops import ReductionArena
from ..fuser import fuse_module
from ..ops import colsum, one_hot, spmm, spmm_sym

aten = torch.ops.aten
torch.fx.wrap("spmm_sym")
torch.fx.wrap("spmm")
torch.fx.wrap("one_hot")


@dataclass
class GcnConfig:
    nodes: int = 169343
    in_feats: int = 128
    hidden: int = 256
    classes: int = 40


def init_params(cfg: GcnConfig, seed: int = 1238, dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)

    def xavier(out_f, in_f):
        std = (2.0 / (in_f + out_f)) ** 0.5
        return (torch.randn(out_f, in_f, generator=g) * std).to(dtype).to(device)
    return {"w1": xavier(cfg.hidden, cfg.in_feats), "b1": (torch.randn(cfg.hidden, generator=g) * 0.01).to(dtype).to(device),
            "w2": xavier(cfg.classes, cfg.hidden), "b2": (torch.randn(cfg.classes, generator=g) * 0.01).to(dtype).to(device)}


def _meta(shape, dtype):
    return torch.empty(tuple(shape), dtype=dtype, device="meta")


class GcnStep:
    """`step(params, crow, col, w, x, labels)` -> (loss, grads).  `nnz` fixes the SpMM plans.

    One GPU: `w` is the per-node vector d^-1/2 and the normalisation is fused into the SpMM.
    A shard of a row partition (`rows` = rows it owns, `operand_rows` = rows of the gathered
    operand buffers) passes per-edge values instead (the products d_i^-1/2 d_j^-1/2 of its own
    edges, formed once when the graph is partitioned: the kernel's fused form indexes the vector
    with the local row number); `gather` is called on every aggregation operand (own rows -> all
    rows) and `reduce` on the loss and the parameter gradients."""

    def __init__(self, cfg: GcnConfig, nnz: int, dtype=torch.bfloat16, rows: int = None, operand_rows: int = None,
                 gather=None, reduce=None):
        self.cfg, self.nnz, self.dtype = cfg, nnz, dtype
        n = rows if rows is not None else cfg.nodes
        xr = operand_rows if operand_rows is not None else n
        self.rows, self.operand_rows = n, xr
        self.sharded = sharded = rows is not None
        self.gather = gather or (lambda t: t)
        self.reduce = reduce
        F, H, C = cfg.in_feats, cfg.hidden, cfg.classes
        dt, f32, i32 = dtype, torch.float32, torch.int32
        self.ops = {}
        self.specs = {}

        def make(name, module, *metas):
            gm, op = fuse_module(module, list(metas))
            self.ops[name] = op
            self.specs[name] = (module, list(metas))
            return gm
        csr = (_meta((n + 1,), i32), _meta((nnz,), i32), _meta((nnz,) if sharded else (n,), f32))

        class AggIn(torch.nn.Module):            # a1 = bf16(A_hat x + x), x in fp32
            def forward(self, crow, col, dinv, x):
                return aten._to_copy(aten.add(spmm_sym(crow, col, dinv, x), x), dtype=dt)

        class AggInShard(torch.nn.Module):       # a row block: gathered x as the operand, own rows as the self term
            def forward(self, crow, col, val, x, x_own):
                return aten._to_copy(aten.add(spmm(crow, col, val, x), x_own), dtype=dt)
        if not sharded:
            self.agg_in = make("agg_in", AggIn(), *csr, _meta((n, F), f32))
        else:
            self.agg_in = make("agg_in", AggInShard(), *csr, _meta((xr, F), f32), _meta((n, F), f32))

        class LinRelu(torch.nn.Module):          # h1 = relu(a1 W1^T + b1)
            def forward(self, a, w, b):
                return aten.relu(aten.add(aten.mm(a, aten.permute(w, [1, 0])), b))
        self.lin1 = make("lin1", LinRelu(), _meta((n, F), dt), _meta((H, F), dt), _meta((H,), dt))

        class Lin(torch.nn.Module):              # z = h1 W2^T + b2
            def forward(self, h, w, b):
                return aten.add(aten.mm(h, aten.permute(w, [1, 0])), b)
        self.lin2 = make("lin2", Lin(), _meta((n, H), dt), _meta((C, H), dt), _meta((C,), dt))

        class AggOut(torch.nn.Module):           # logits = A_hat z + z
            def forward(self, crow, col, dinv, z):
                return aten.add(spmm_sym(crow, col, dinv, z), z)

        class AggOutShard(torch.nn.Module):
            def forward(self, crow, col, val, z, z_own):
                return aten.add(spmm(crow, col, val, z), z_own)
        if not sharded:
            self.agg_out = make("agg_out", AggOut(), *csr, _meta((n, C), dt))
        else:
            self.agg_out = make("agg_out", AggOutShard(), *csr, _meta((xr, C), dt), _meta((n, C), dt))

        inv_n = 1.0 / cfg.nodes                  # the loss is the mean over ALL nodes, also on a shard

        class LossGrad(torch.nn.Module):         # (softmax(logits) - one_hot(labels)) / nodes
            def forward(self, logits, labels):
                p = aten._softmax(logits, -1, False)
                return aten.mul(aten.sub(p, one_hot(labels, C)), inv_n)
        self.loss_grad = make("loss_grad", LossGrad(), _meta((n, C), dt), _meta((n,), torch.int64))

        class DgradRelu(torch.nn.Module):        # dh1 = (dz W2) * (h1 > 0)
            def forward(self, dz, w, h):
                return aten.mul(aten.mm(dz, w), aten.gt(h, 0.0))
        self.dgrad2 = make("dgrad2", DgradRelu(), _meta((n, C), dt), _meta((C, H), dt), _meta((n, H), dt))

        class Wgrad(torch.nn.Module):            # dW = dy^T x
            def forward(self, dy, x):
                return aten.mm(aten.permute(dy, [1, 0]), x)
        self.wgrad2 = make("wgrad2", Wgrad(), _meta((n, C), dt), _meta((n, H), dt))
        self.wgrad1 = make("wgrad1", Wgrad(), _meta((n, H), dt), _meta((n, F), dt))
        self._arena = None

    def check_status(self):
        for op in self.ops.values():
            op.check_status()

    def step(self, p: Dict[str, torch.Tensor], crow, col, w, x, labels):
        """`x`, `labels`: the rows this step owns (all rows on one GPU)."""
        gen = self.step_parts(p, crow, col, w, x, labels)
        item = next(gen)
        while item[0] != "done":
            item[2]()                      # the exchange this part ends with, right away
            item = next(gen)
        return item[1], item[2]

    def step_parts(self, p: Dict[str, torch.Tensor], crow, col, w, x, labels):
        """The step as a generator that stops wherever ranks exchange data: it yields
        ("exchange", tensor, run) with everything before the exchange already enqueued -- the caller
        runs `run()` (the collective) and resumes -- and finally ("done", loss, grads).  A caller may
        capture the parts between the stops in CUDA graphs and replay graph, collective, graph, ...
        On one GPU there is no stop."""
        if self._arena is None or self._arena.buf.device != x.device:
            self._arena = ReductionArena(x.device, 1 << 16)
        self._arena.reset()
        with self._arena:
            if self.sharded:
                full, run = self.gather(x)
                yield ("exchange", full, run)
                a1 = self.agg_in(crow, col, w, full, x)
            else:
                a1 = self.agg_in(crow, col, w, x)
            h1 = self.lin1(a1, p["w1"], p["b1"])
            z = self.lin2(h1, p["w2"], p["b2"])
            if self.sharded:
                full, run = self.gather(z)
                yield ("exchange", full, run)
                logits = self.agg_out(crow, col, w, full, z)
            else:
                logits = self.agg_out(crow, col, w, z)
            lf = logits.to(torch.float32)
            loss = (torch.logsumexp(lf, -1) - lf.gather(1, labels.view(-1, 1)).view(-1)).sum() / self.cfg.nodes
            dlogits = self.loss_grad(logits, labels)
            if self.sharded:                                   # A_hat is symmetric: the same row block
                full, run = self.gather(dlogits, slot=1)
                yield ("exchange", full, run)
                dz = self.agg_out(crow, col, w, full, dlogits)
            else:
                dz = self.agg_out(crow, col, w, dlogits)
            grads = {"w2": self.wgrad2(dz, h1), "b2": colsum(dz, torch.float32)}
            dh1 = self.dgrad2(dz, p["w2"], h1)
            grads["w1"] = self.wgrad1(dh1, a1)
            grads["b1"] = colsum(dh1, torch.float32)
        if self.reduce is not None:
            flat, run, unpack = self.reduce(loss, grads)
            yield ("exchange", flat, run)
            loss, grads = unpack()
        yield ("done", loss, grads)


# ---------------------------------------------------------------------------------------------
# row partition
# ---------------------------------------------------------------------------------------------

def partition_rows(crow: torch.Tensor, col: torch.Tensor, dinv: torch.Tensor, world: int, row_cost: int = 8):
    """Cuts the rows of a CSR matrix into `world` contiguous blocks of about equal work, work =
    nonzeros + row_cost x rows: the nonzeros are the aggregation's gathers, the rows carry the dense
    maps and the epilogues (by row count alone the rank with the hub rows of a power-law graph
    would get most of the nonzeros; by nonzeros alone the last rank would get most of the rows).
    Host-side, once per graph.

    Returns a list of dicts, one per rank: row range [r0, r1), local `crow` (int32, starts at 0),
    `col` (int32, global node ids) and `val` (fp32, d_i^-1/2 d_j^-1/2 per edge)."""
    crow64 = crow.to(torch.int64)
    n = crow.shape[0] - 1
    weight = crow64 + row_cost * torch.arange(n + 1)
    bounds = [0]
    for r in range(1, world):
        target = (int(weight[-1]) * r) // world
        bounds.append(min(n, max(bounds[-1], int(torch.searchsorted(weight, target)))))
    bounds.append(n)
    row_of = torch.repeat_interleave(torch.arange(n), crow64[1:] - crow64[:-1])
    val_all = (dinv[row_of] * dinv[col.to(torch.int64)]).to(torch.float32)
    shards = []
    for r in range(world):
        r0, r1 = bounds[r], bounds[r + 1]
        p0, p1 = int(crow64[r0]), int(crow64[r1])
        shards.append(dict(rank=r, r0=r0, r1=r1, bounds=list(bounds),
                           crow=(crow64[r0:r1 + 1] - p0).to(torch.int32),
                           col=col[p0:p1].to(torch.int32).contiguous(),
                           val=val_all[p0:p1].contiguous()))
    return shards


class GcnShard:
    """One rank's part of the row-partitioned step.  `shard` = this rank's entry of
    `partition_rows`; collectives go through `torch.distributed` (NCCL on GPUs, gloo in the CPU
    test of the bookkeeping)."""

    def __init__(self, cfg: GcnConfig, shard: dict, world: int, device, dtype=torch.bfloat16, group=None, build_step=True):
        import torch.distributed as dist
        self.dist, self.group, self.world = dist, group, world
        self.cfg, self.shard, self.device = cfg, shard, device
        self.r0, self.r1, self.bounds = shard["r0"], shard["r1"], shard["bounds"]
        self.rows = self.r1 - self.r0
        self.crow = shard["crow"].to(device)
        self.col = shard["col"].to(device)
        self.val = shard["val"].to(device)
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self.bytes_gathered = 0
        self.step_impl = None
        if build_step:
            self.step_impl = GcnStep(cfg, int(self.col.shape[0]), dtype, rows=self.rows, operand_rows=cfg.nodes,
                                     gather=self.gather, reduce=self.reduce)

    def gather(self, own: torch.Tensor, slot: int = 0):
        """own rows [rows, F] -> (buffer of all nodes' rows [nodes, F] with this rank's slice filled
        in, the function that completes it: every rank broadcasts its block into its slice).
        `slot` keeps two operands of one shape apart (both stay in use)."""
        key = (own.shape[1], own.dtype, slot)
        if key not in self._bufs:
            self._bufs[key] = torch.zeros(self.cfg.nodes, own.shape[1], dtype=own.dtype, device=own.device)
        full = self._bufs[key]
        full[self.r0:self.r1].copy_(own)

        views = [full[self.bounds[k]:self.bounds[k + 1]] for k in range(self.world)]

        def run():
            if self.dist.get_backend(self.group) == "nccl":
                # blocks of unequal length: one coalesced launch of per-rank broadcasts, in place
                self.dist.all_gather(views, views[self.shard["rank"]], group=self.group)
            else:
                for k, v in enumerate(views):
                    if v.numel():
                        self.dist.broadcast(v, src=self._global_rank(k), group=self.group)
            self.bytes_gathered += full.numel() * full.element_size()
        return full, run

    def _global_rank(self, k: int) -> int:
        return k if self.group is None else self.dist.get_global_rank(self.group, k)

    def reduce(self, loss, grads):
        """(flat fp32 buffer of loss + gradients, the all-reduce, the function that unpacks it)"""
        flat = torch.cat([loss.reshape(1).to(torch.float32)] + [g.reshape(-1).to(torch.float32) for g in grads.values()])

        def run():
            self.dist.all_reduce(flat, group=self.group)

        def unpack():
            out, o = {}, 1
            for k, g in grads.items():
                out[k] = flat[o:o + g.numel()].view(g.shape)
                o += g.numel()
            return flat[0], out
        return flat, run, unpack

    def step(self, p, x_own, labels_own):
        self.bytes_gathered = 0
        return self.step_impl.step(p, self.crow, self.col, self.val, x_own, labels_own)

    def step_parts(self, p, x_own, labels_own):
        return self.step_impl.step_parts(p, self.crow, self.col, self.val, x_own, labels_own)

    def check_status(self):
        self.step_impl.check_status()
