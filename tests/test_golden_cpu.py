"""Pins the oracle: this repository's restated modules (tests/partitions.py), run unfused in
fp32 on CPU, against outputs of the REFERENCE's own fused-node test modules on the same seeded
inputs (tests/golden/golden.npz, produced by tests/golden/make_golden.py from
unittest/evt_fuser/*.py).  The inputs are rebuilt here from seeds; their construction was
verified bit for bit against the reference's when the fixture was generated."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import cases as G  # noqa: E402
from oracle import run_unfused_fp32

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))


def golden_outputs(name):
    n = int(GOLD[f"{name}/n_out"])
    return [dict(shape=tuple(GOLD[f"{name}/{j}/shape"]), sample=GOLD[f"{name}/{j}/sample"],
                 sum=float(GOLD[f"{name}/{j}/sum"]), abs_sum=float(GOLD[f"{name}/{j}/abs_sum"])) for j in range(n)]


def check_against_golden(name, outs, rtol, atol, checksum_rtol=None, full_numel=None, skip=()):
    """|got - want| <= rtol |want| + floor per sampled element.  With `full_numel` (the number of
    elements of an elementwise result of the node) the floor follows the golden output's own RMS:
    atol x max(1, RMS) for elementwise results, rtol x RMS for reduction results (fewer elements);
    without it the floor is `atol`."""
    gold = golden_outputs(name)
    if name in G.LEADING_OUTPUTS:
        gold = gold[:G.LEADING_OUTPUTS[name]]
    assert len(outs) == len(gold), (name, len(outs), len(gold))
    for j, (o, g) in enumerate(zip(outs, gold)):
        if j in skip:
            continue
        assert int(np.prod(o.shape)) == int(np.prod(g["shape"])), (name, j, tuple(o.shape), g["shape"])
        flat = o.detach().cpu().to(torch.float64).reshape(-1).numpy()
        idx = G.sample_index(flat.size)
        got, want = flat[idx], g["sample"].astype(np.float64)
        floor = atol
        if full_numel is not None:
            rms = float(np.sqrt(np.mean(want ** 2)))
            floor = max(atol, rtol * rms) if flat.size < full_numel else atol * max(1.0, rms)
        bad = np.abs(got - want) > rtol * np.abs(want) + floor
        assert not bad.any(), (name, j, float(np.abs(got - want).max()), int(bad.sum()))
        if checksum_rtol is not None:
            assert abs(np.abs(flat).sum() - g["abs_sum"]) <= checksum_rtol * g["abs_sum"] + 1e-3, (name, j)


@pytest.mark.parametrize("name", list(G.CASES), ids=list(G.CASES))
def test_oracle_matches_reference_modules(name):
    case = G.CASES[name][3]()
    inputs = G.golden_inputs(name)
    case.inputs = inputs
    outs = run_unfused_fp32(case.module, inputs)
    # both sides are fp32 eager evaluations of the same graph: agreement to rounding
    check_against_golden(name, outs, rtol=G.ORACLE_RTOL.get(name, 1e-5), atol=1e-5, checksum_rtol=1e-6)


@pytest.mark.parametrize("leaf", G.LEAVES)
def test_leaves_match_the_reference_leaves(leaf):
    """evt_ae_b200/ops.py's wrapped leaf functions against the reference's functions of the same
    names (python/gtl/compiler/passes/pass_decomposition.py:61-189) on the same seeded tensors.
    fp32 evaluations of the same expression: agreement to rounding; the batch-norm leaves keep
    their half-precision outputs (1e-3 relative)."""
    from evt_ae_b200 import ops
    with torch.no_grad():
        outs = G.leaf_call(ops, leaf, G.leaf_inputs(leaf))
    if leaf == "batch_norm":
        check_against_golden(f"leaf/{leaf}", list(outs), rtol=2e-3, atol=2e-3)
    else:
        check_against_golden(f"leaf/{leaf}", list(outs), rtol=1e-5, atol=1e-4, checksum_rtol=1e-5)


def test_dropout_formula_with_the_reference_mask():
    """unittest/evt_fuser/dropout.py:33-75: with the keep mask the reference module drew, the
    restated module's arithmetic (scale by 1 / (1 - p), then the residual) gives its output."""
    keep = torch.from_numpy(np.unpackbits(GOLD["dropout/keep_bits"])[: 512 * 2 * 1024].astype(bool)).view(512, 2, 1024)
    out = G.dropout_formula(G.dropout_inputs(), keep)
    check_against_golden("dropout", [out], rtol=1e-5, atol=1e-4, checksum_rtol=1e-6)
