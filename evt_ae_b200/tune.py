"""Tile tuner for the fused GEMM / batched-GEMM nodes of a workload.

    python -m evt_ae_b200.tune --workload bert --compile-only     # any box with nvcc
    python -m evt_ae_b200.tune --workload bert --out tuned.json   # on the GPU

For every GEMM node the candidates are the closed-form choice of `fused_ops.pick_gemm_tile`
and its neighbours (8 or 16 epilogue warps, a narrower tile, other K splits); each is timed
alone with CUDA events on random operands of the node's shapes and the fastest is written to
the table `tuning.lookup()` reads.  The reference's counterpart is the profile-guided tuner
of python/gtl/compiler/autotuner/gemm_tuner.py:126-153 with its SQLite cache.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from typing import Dict, List, Tuple

import torch

from . import jit, tuning
from .codegen import GemmTileConfig
from .fused_ops import _FusedMatmulBase, pick_gemm_tile
from .fuser import fuse_module


def candidates(op: _FusedMatmulBase) -> List[GemmTileConfig]:
    base = pick_gemm_tile(op.M, op.N, op.K, op.L, op.b_major)
    out: List[GemmTileConfig] = []

    def add(bn, ew, sk, pair=False):
        if op.b_major == "MN" and bn % 64:
            return
        if bn // 2 >= op.N and bn > 32:
            return
        if pair and (bn not in (128, 256) or op.M <= 128):
            return
        c = GemmTileConfig(bn=bn, stages=8, epi_warps=ew, split_k=sk, cta_pair=pair)   # ring depth is fitted later
        key = lambda t: (t.bn, t.epi_warps, t.split_k, t.cta_pair)
        if all(key(c) != key(o) for o in out):
            out.append(c)

    add(base.bn, base.epi_warps, base.split_k, base.cta_pair)
    for pair in (False, True):
        for ew in (8, 16):
            add(base.bn, ew, base.split_k, pair)
    if base.bn == 256:
        add(128, 8, base.split_k)
        add(128, 8, base.split_k, True)      # 256 x 128 pair tiles: twice the tiles, fuller last wave
        add(128, 16, base.split_k, True)
    tiles = ((op.M + 127) // 128) * ((op.N + base.bn - 1) // base.bn) * op.L
    num_k = (op.K + 63) // 64
    if tiles < 148 and num_k >= 32:
        for sk in (1, 2, 4, 8):
            if sk <= num_k // 8:
                for bn in (256, 128):
                    add(bn, 8, sk)
                add(256, 8, sk, True)
        # cuts that fill whole rounds of the grid: units = tiles x cuts just below 1, 2 or 3 times the
        # number of CTAs (148) or CTA pairs (74) -- 16 pair tiles cut 9 ways are 144 units on 74 pairs
        # (1.95 rounds), cut 8 ways 128 units (1.73 rounds, the second one three quarters full)
        pair_tiles = ((op.M + 255) // 256) * ((op.N + base.bn - 1) // base.bn) * op.L
        for rounds in (1, 2, 3):
            for sk, pair in ((rounds * 148 // max(tiles, 1), False), (rounds * 74 // max(pair_tiles, 1), True)):
                if 1 <= sk <= min(num_k // 8, 16):
                    add(base.bn, 8, sk, pair)
    return out


def row_candidates(op) -> List:
    """threads per row x CTA size around the closed-form choice (the row must fit the registers:
    at most 8 vectors of 8 elements per thread)."""
    from .codegen import RowKernelConfig
    base = op.cfg
    vectors = (op.cols + 7) // 8
    out = [base]
    for tpr in (base.tpr // 2, base.tpr, base.tpr * 2):
        if tpr < 8 or tpr > 1024:
            continue
        vpt = (vectors + tpr - 1) // tpr
        if vpt > 2 * op.max_vpt or vpt < 1:
            continue
        for threads in (128, 256, 512):
            threads = max(threads, tpr)
            c = RowKernelConfig(tpr=tpr, vpt=vpt, threads=threads, vec=base.vec)
            if all((c.tpr, c.threads) != (o.tpr, o.threads) for o in out):
                out.append(c)
    return out


def conv_candidates(op) -> List:
    from .codegen import ConvTileConfig
    nt = op.geom["C"] if op.dgrad else op.geom["K"]
    out = [op.tile]
    for bn in (64, 128, 256):
        if bn > nt:
            continue
        for stages, ew in ((6, 8), (4, 8), (6, 16)):
            c = ConvTileConfig(bn=bn, stages=stages, epi_warps=ew)
            if all((c.bn, c.stages, c.epi_warps) != (o.bn, o.stages, o.epi_warps) for o in out):
                out.append(c)
    return out


def spmm_candidates(op) -> List:
    import copy
    out = [op.cfg]
    for t_long, task_len, u_short, min_ctas in [(64, 1024, 4, 4), (128, 1024, 4, 4), (256, 1024, 4, 4), (128, 512, 4, 4),
                                               (128, 1024, 2, 4), (128, 1024, 4, 3)]:
        c = copy.copy(op.cfg)
        c.t_long, c.task_len, c.u_short, c.min_ctas = t_long, task_len, u_short, min_ctas
        if all((c.t_long, c.task_len, c.u_short, c.min_ctas) != (o.t_long, o.task_len, o.u_short, o.min_ctas) for o in out):
            out.append(c)
    return out


def wgrad_candidates(op) -> List:
    """channel-tile width x number of cuts of the N*P*Q reduction around the closed-form choice"""
    import copy
    base = op.tile
    out = [base]
    for bn in (64, 128, 256):
        if op.geom["C"] % bn:
            continue
        tiles = ((op.geom["K"] + 127) // 128) * (op.geom["R"] * op.geom["S"] * op.geom["C"] // bn)
        boxes = max(1, op.geom["N"] * op.geom["P"] * op.geom["Q"] // 64)
        full = max(1, min(148 // max(tiles, 1), boxes // 8, 64))
        for split in sorted({max(1, full // 2), full, min(64, full * 2)}):
            c = GemmTileConfig(bn=bn, stages=6, epi_warps=8, split_k=split)
            if all((c.bn, c.split_k) != (o.bn, o.split_k) for o in out):
                out.append(c)
    return out


def node_candidates(op):
    """(keyword of fuse_module, candidate list, fields stored in the table) for any fused node."""
    from . import fused_ops as F
    if isinstance(op, _FusedMatmulBase):
        return "tile", candidates(op), ("bn", "stages", "epi_warps", "split_k", "cta_pair")
    if isinstance(op, F._FusedRowBase):
        return "row_config", row_candidates(op), ("tpr", "vpt", "threads")
    if isinstance(op, F._FusedConvBase):
        return "conv_tile", conv_candidates(op), ("bn", "stages", "epi_warps")
    if isinstance(op, F.FusedConvWgrad):
        return "tile", wgrad_candidates(op), ("bn", "stages", "epi_warps", "split_k")
    if isinstance(op, F.FusedSpmm):
        return "spmm_config", spmm_candidates(op), ("t_long", "task_len", "u_short", "u_long", "min_ctas")
    raise TypeError(type(op))


def random_like(meta: torch.Tensor, device) -> torch.Tensor:
    if meta.dtype.is_floating_point:
        return (torch.randn(meta.shape, device=device, dtype=torch.float32) * 0.1).to(meta.dtype)
    if meta.dtype == torch.bool:
        return torch.rand(meta.shape, device=device) < 0.5
    return torch.zeros(meta.shape, device=device, dtype=meta.dtype)


def fused_args(gm, op, inputs):
    """The tensors the fused node of `gm` is called with, given the module's inputs."""
    ph = [n for n in gm.graph.nodes if n.op == "placeholder"]
    call = [n for n in gm.graph.nodes if n.op == "call_function" and n.target is op][0]
    by_name = {n.name: t for n, t in zip(ph, inputs)}
    return [by_name[a.name] for a in call.args]


def workload_specs(name: str) -> Dict[str, Tuple[torch.nn.Module, list]]:
    if name == "bert":
        from .workloads import bert as wb
        step = wb.BertStep(wb.BERT_LARGE, 32, 512, dtype=torch.bfloat16)
        # row-resident nodes (softmax fused into the GEMM) have one configuration and are not tuned
        return {k: v for k, v in step.n.specs.items()
                if not (isinstance(step.n.ops[k], _FusedMatmulBase) and step.n.ops[k].tile.row_resident)}
    if name == "vit":
        from .workloads import vit as wv
        step = wv.VitStep(wv.VIT_BASE_16, 128, dtype=torch.bfloat16)
        return {k: v for k, v in step.n.specs.items()
                if not (isinstance(step.n.ops[k], _FusedMatmulBase) and step.n.ops[k].tile.row_resident)}
    if name == "resnet_convs":
        # forward convolutions with batch-norm statistics and strided data gradients at ResNet-50 shapes, batch 128
        from .workloads import cases as P
        out = {}
        for (h, c, k, r, s) in [(56, 64, 64, 3, 1), (56, 64, 256, 1, 1), (28, 128, 128, 3, 1), (14, 256, 256, 3, 1), (7, 512, 512, 3, 1)]:
            case = P.conv_fprop_bn_stat(128, h, h, c, k, r, s)
            out[f"fprop_{h}_{c}_{k}_{r}"] = (case.module, [torch.empty(t.shape, dtype=t.dtype, device="meta") for t in case.inputs])
        case = P.conv_dgrad_strided(128, 28, 28, 128, 256, 3, 2)
        out["dgrad_28_128_256_s2"] = (case.module, [torch.empty(t.shape, dtype=t.dtype, device="meta") for t in case.inputs])
        for (h, c, k, r, s) in [(56, 64, 64, 3, 1), (56, 64, 256, 1, 1), (28, 128, 128, 3, 1), (14, 256, 256, 3, 1), (7, 512, 512, 3, 1),
                                (28, 128, 256, 3, 2)]:
            case = P.conv_wgrad_plain(128, h, h, c, k, r, s)
            out[f"wgrad_{h}_{c}_{k}_{r}_s{s}"] = (case.module, [torch.empty(t.shape, dtype=t.dtype, device="meta") for t in case.inputs])
        return out
    if name == "resnet50":
        # every fused convolution of the ResNet-50 step at batch 128: forward with batch-norm
        # statistics, data gradient, weight gradient of each of the 22 geometries
        from .workloads import resnet as wr
        out = {}
        for geo in wr.geometries(wr.RESNET50, 128):
            for kind, spec in wr.conv_modules(geo).items():
                out[kind + "_" + "x".join(map(str, geo))] = spec
        return out
    if name == "gcn":
        from .workloads import cases as P
        case = P.spmm_case(169343, 585000, 128, "sym")
        return {"agg_sym_128": (case.module, list(case.inputs))}
    if name == "config0":
        aten = torch.ops.aten

        class Config0(torch.nn.Module):     # D = GELU(A@B + bias) + C, colsum(D), rowmax(D)
            def forward(self, a, b, bias, c):
                d = aten.add(aten.gelu(aten.add(aten.mm(a, b), bias)), c)
                return d, aten.sum(d, [0]), aten.amax(d, [1])
        M, N, K, dt = 16384, 4096, 1024, torch.float16
        m = lambda *s: torch.empty(s, dtype=dt, device="meta")
        return {"config0": (Config0(), [m(M, K), m(K, N), m(N), m(M, N)])}
    raise SystemExit(f"unknown workload {name!r}")


def tune_bn_stats(out_path: str, iters: int, min_gain: float):
    """For every convolution geometry of the ResNet-50 step: the forward convolution with the batch-norm
    statistics in its epilogue against the plain-store convolution followed by a statistics pass over its
    output.  Writes {"separate": 1} entries (workloads/resnet.py:stats_key) where the second form wins."""
    from . import ops
    from .workloads import resnet as wr
    dev, dt = torch.device("cuda:0"), torch.float16
    entries = {}
    for geo in wr.geometries(wr.RESNET50, 128):
        mods = wr.conv_modules(geo, dt)
        gm_f, op_f = fuse_module(*mods["fprop"])
        gm_p, op_p = fuse_module(*mods["fprop_plain"])
        inputs = [random_like(m, dev) for m in mods["fprop"][1]]
        fused_us = statistics.median(op_f.time_kernel(fused_args(gm_f, op_f, inputs), iters=iters)) * 1e3
        plain_us = statistics.median(op_p.time_kernel(fused_args(gm_p, op_p, inputs), iters=iters)) * 1e3
        y = gm_p(*inputs)
        rf = 1.0 / (y.shape[0] * y.shape[1] * y.shape[2])
        g = torch.cuda.CUDAGraph()
        ops.batch_norm_stat(y, rf)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            for _ in range(iters):
                ops.batch_norm_stat(y, rf)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g.replay()
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        stat_us = e0.elapsed_time(e1) / iters * 1e3
        separate = plain_us + stat_us < min_gain * fused_us
        if separate:
            entries[wr.stats_key(geo, dt)] = dict(separate=1, fused_us=round(fused_us, 1), plain_us=round(plain_us, 1),
                                                  stat_us=round(stat_us, 1))
        print(json.dumps(dict(geometry=list(geo), fused_us=round(fused_us, 1), plain_us=round(plain_us, 1),
                              stat_us=round(stat_us, 1), separate=int(separate))))
        sys.stdout.flush()
    tuning.save(entries, out_path)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="bert")
    ap.add_argument("--compile-only", action="store_true")
    ap.add_argument("--only", default="", help="comma-separated node names of the workload (default: all)")
    ap.add_argument("--out", default=tuning.TABLE_PATH)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--min-gain", type=float, default=0.96,
                    help="a candidate replaces the closed-form choice only below this fraction of its time")
    a = ap.parse_args(argv)
    if a.workload == "resnet50_stats":
        if a.compile_only:
            from .workloads import resnet as wr
            with jit.deferred() as d:
                for geo in wr.geometries(wr.RESNET50, 128):
                    mods = wr.conv_modules(geo, torch.float16)
                    fuse_module(*mods["fprop"])
                    fuse_module(*mods["fprop_plain"])
            print("compiled", d.flush(), "kernel variants")
            return
        tune_bn_stats(a.out, a.iters, a.min_gain)
        return
    specs = workload_specs(a.workload)
    if a.only:
        specs = {k: v for k, v in specs.items() if k in a.only.split(",")}
    def as_meta(ts):
        return [torch.empty(t.shape, dtype=t.dtype, device="meta") if t.device.type != "meta" else t for t in ts]
    if a.compile_only:
        with jit.deferred() as d:
            for name, (module, metas) in specs.items():
                _, op0 = fuse_module(module, as_meta(metas))
                kw, cands, _ = node_candidates(op0)
                for c in cands:
                    fuse_module(module, as_meta(metas), **{kw: c})
        print("compiled", d.flush(), "kernel variants")
        return
    if not torch.cuda.is_available():
        raise SystemExit("tuning needs a GPU (use --compile-only to build the candidates)")
    # Candidate lists start with the node's current choice, which is the shipped table's entry where
    # there is one; a candidate is written only if it beats that by the margin, so entries of the
    # shipped table stay valid unless this run's output replaces them (merge, do not drop).
    dev = torch.device("cuda:0")
    entries = {}
    for name, (module, metas) in specs.items():
        _, op0 = fuse_module(module, as_meta(metas))
        kw, cands, fields = node_candidates(op0)
        # real tensors where the spec carries them (a CSR structure cannot be random), else random
        inputs = [m.to(dev) if m.device.type != "meta" else random_like(m, dev) for m in metas]
        rows = []
        for c in cands:
            gm, op = fuse_module(module, as_meta(metas), **{kw: c})
            us = statistics.median(op.time_kernel(fused_args(gm, op, inputs), iters=a.iters)) * 1e3
            op.check_status()
            used = op.tile if kw in ("tile", "conv_tile") else op.cfg
            rows.append((us, used))
        default_us, default_cfg = rows[0]           # the candidate lists start with the closed-form choice
        rows.sort(key=lambda r: r[0])
        us, t = rows[0]
        if us > a.min_gain * default_us:
            us, t = default_us, default_cfg            # within noise of the default: keep the default
        desc = lambda c: [int(getattr(c, f)) for f in fields]
        if t is not default_cfg:        # the table only lists departures from the closed-form choice
            entries[op0.tune_key] = dict({f: int(getattr(t, f)) for f in fields}, node=name, us=round(us, 1),
                                         default_us=round(default_us, 1))
        rate = {"tflops": round(op0.flops / us / 1e6, 1)} if getattr(op0, "flops", 0) else \
               ({"gbs": round(op0.bytes_moved / us / 1e3, 1)} if hasattr(op0, "bytes_moved") else {})
        print(json.dumps(dict(node=name, fields=list(fields), best=desc(t), us=round(us, 1), **rate,
                              all=[desc(r[1]) + [round(r[0], 1)] for r in rows])))
        sys.stdout.flush()
    tuning.save(entries, a.out)


if __name__ == "__main__":
    main()
