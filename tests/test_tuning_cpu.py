"""Tile-tuner table: keys, lookup, the deferred compile mode (no GPU needed)."""
import json
import os

import torch

from evt_ae_b200 import tuning
from evt_ae_b200.codegen import GemmTileConfig
from evt_ae_b200.fuser import fuse_module
from evt_ae_b200.tune import candidates, workload_specs

import partitions as P


def _meta(case):
    return [torch.empty(t.shape, dtype=t.dtype, device="meta") for t in case.inputs]


def test_key_separates_shapes_dtypes_and_epilogues():
    a = P.mm_bias_gelu(256, 512, 128, 16, 16, torch.float16)
    b = P.mm_bias_gelu(256, 512, 256, 16, 16, torch.float16)
    c = P.mm_bias_tanh(256, 512, 128, torch.float16)
    d = P.mm_bias_gelu(256, 512, 128, 16, 16, torch.bfloat16)
    keys = [fuse_module(x.module, _meta(x))[1].tune_key for x in (a, b, c, d)]
    assert len(set(keys)) == 4
    again = fuse_module(a.module, _meta(a))[1].tune_key
    assert again == keys[0]


def test_table_round_trip_and_lookup(tmp_path, monkeypatch):
    path = str(tmp_path / "t.json")
    tuning.save({"k1": dict(bn=128, stages=5, epi_warps=16, split_k=2, node="x", us=1.0)}, path)
    tuning.save({"k2": dict(bn=256, stages=4, epi_warps=8, split_k=1, node="y", us=2.0)}, path)
    assert set(json.load(open(path))) == {"k1", "k2"}
    monkeypatch.setattr(tuning, "TABLE_PATH", path)
    monkeypatch.setattr(tuning, "_table", None)
    t = tuning.lookup("k1")
    assert (t.bn, t.stages, t.epi_warps, t.split_k) == (128, 5, 16, 2)
    assert tuning.lookup("absent") is None
    monkeypatch.setattr(tuning, "_table", None)


def test_shipped_table_is_well_formed_and_explicit_tile_wins(tmp_path, monkeypatch):
    shipped = json.load(open(tuning.TABLE_PATH))
    for key, e in shipped.items():
        kind = key.split("|")[0]
        if kind == "bn_stats":       # where a convolution's batch-norm statistics are taken (workloads/resnet.py)
            assert key.count("|") == 2 and e["separate"] in (0, 1) and e["plain_us"] + e["stat_us"] < e["fused_us"], key
            continue
        assert key.count("|") == 3
        if kind == "row":
            assert e["tpr"] in (8, 16, 32, 64, 128, 256, 512, 1024) and e["threads"] % 32 == 0 and 1 <= e["vpt"] <= 8, key
        elif kind == "spmm":
            assert e["t_long"] > 0 and e["task_len"] >= 32 and e["u_short"] in (1, 2, 4, 8), key
        elif kind.startswith("conv"):
            assert e["bn"] in (64, 128, 256) and e["epi_warps"] in (8, 16) and 2 <= e["stages"] <= 8, key
        else:
            assert e["bn"] in (32, 64, 128, 256) and e["epi_warps"] in (4, 8, 12, 16) and 2 <= e["stages"] <= 8
            assert e.get("cta_pair", 0) in (0, 1) and e["split_k"] >= 1, key
    mod, metas = workload_specs("config0")["config0"]
    _, op = fuse_module(mod, metas)
    path = str(tmp_path / "t.json")
    tuning.save({op.tune_key: dict(bn=128, stages=5, epi_warps=16, split_k=1, cta_pair=0, node="c0", us=1.0)}, path)
    monkeypatch.setattr(tuning, "TABLE_PATH", path)
    monkeypatch.setattr(tuning, "_table", None)
    _, op1 = fuse_module(mod, metas)
    assert (op1.tile.bn, op1.tile.epi_warps, op1.tile.cta_pair) == (128, 16, False)
    _, op2 = fuse_module(mod, metas, tile=GemmTileConfig(bn=256, stages=4))
    assert op2.tile.bn == 256 and op2.tile.epi_warps == 8
    monkeypatch.setattr(tuning, "_table", None)


def test_candidates_start_with_the_closed_form_choice_and_are_unique():
    case = P.mm_wgrad(1024, 1024, 16384, torch.bfloat16)
    _, op = fuse_module(case.module, _meta(case))
    from evt_ae_b200.fused_ops import pick_gemm_tile
    base = pick_gemm_tile(op.M, op.N, op.K, op.L, op.b_major)
    cands = candidates(op)
    assert (cands[0].bn, cands[0].split_k, cands[0].epi_warps, cands[0].cta_pair) == (base.bn, base.split_k, 8, base.cta_pair)
    sig = [(c.bn, c.epi_warps, c.split_k, c.cta_pair) for c in cands]
    assert len(sig) == len(set(sig)) and any(c.split_k == 1 for c in cands)


def test_every_node_kind_has_candidates_and_a_table_entry_is_applied(tmp_path, monkeypatch):
    """Row kernels, convolutions and SpMM go through the same table as the GEMMs."""
    from evt_ae_b200.tune import node_candidates
    from evt_ae_b200 import codegen
    row = P.softmax_plain(256, 512, torch.float16)
    conv = P.conv_fprop_bn_stat(4, 28, 28, 128, 256, 3, 1)
    sp = P.spmm_case(2000, 9000, 128, "sym")
    entries = {}
    for case, kw_expected in ((row, "row_config"), (conv, "conv_tile"), (sp, "spmm_config")):
        _, op = fuse_module(case.module, _meta(case))
        kw, cands, fields = node_candidates(op)
        assert kw == kw_expected and len(cands) >= 3
        pick = cands[-1]
        entries[op.tune_key] = {f: int(getattr(pick, f)) for f in fields}
    path = str(tmp_path / "t.json")
    tuning.save(entries, path)
    monkeypatch.setattr(tuning, "TABLE_PATH", path)
    monkeypatch.setattr(tuning, "_table", None)
    for case in (row, conv, sp):
        _, op = fuse_module(case.module, _meta(case))
        e = entries[op.tune_key]
        cfg = op.tile if hasattr(op, "geom") else op.cfg
        for f, v in e.items():
            if f == "stages":       # the ring is shortened when the staging tiles need the shared memory
                assert int(getattr(cfg, f)) <= v, (case.name, f)
            else:
                assert int(getattr(cfg, f)) == v, (case.name, f)
    monkeypatch.setattr(tuning, "_table", None)


def test_ffn1_profile_note_describes_the_kernel_the_benchmark_times():
    """bench.py reports the FFN1 GEMM's DRAM traffic from a profiler capture summarised under profiles/;
    the figure is only valid for the tile the capture ran with.  The note names that tile and the traffic:
    both must agree with what the code uses now."""
    import os
    import re
    import torch
    from evt_ae_b200.workloads import bert as wb
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    note = open(os.path.join(root, "profiles", "bert_ffn1_gemm_ncu_metrics.md")).read()
    m = re.search(r"(\d+) x (\d+)\s+pair tiles, (\d+)-stage ring, (\d+) epilogue warps", note)
    assert m, "the note no longer names the tile"
    step = wb.BertStep(wb.BERT_LARGE, 32, 512, dtype=torch.bfloat16)
    tile = step.n.ops["lin_hf_gelu"].tile
    assert tile.cta_pair and (256, tile.bn, tile.stages, tile.epi_warps) == tuple(int(v) for v in m.groups())
    traffic = float(re.search(r"-> traffic ([0-9.]+) MB per launch", note).group(1)) * 1e6
    src = open(os.path.join(root, "bench.py")).read()
    assert abs(float(re.search(r"FFN1_DRAM_TRAFFIC_BYTES = ([0-9.e]+)", src).group(1)) - traffic) < 1e5
