"""The CUDA path at the reference's full test shapes against the golden outputs of the
reference's own test modules (see test_golden_cpu.py).  Tolerance per sampled element for
half-precision results (fp32 accumulate): 1e-2 relative + an absolute term tied to the golden
output's own RMS -- 1e-3 x max(1, RMS) for elementwise results, 1e-2 x RMS for reductions."""
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import cases as G  # noqa: E402
from test_golden_cpu import check_against_golden
from evt_ae_b200.fuser import fuse_module

pytestmark = pytest.mark.gpu


SINGLE_NODE = [n for n in G.CASES if n not in G.MULTI_NODE]


@pytest.mark.parametrize("name", SINGLE_NODE, ids=SINGLE_NODE)
def test_cuda_path_matches_reference_modules(name, cuda_device):
    case = G.CASES[name][3]()
    inputs = [t.to(cuda_device) for t in G.golden_inputs(name)]
    gm, fused = fuse_module(case.module, inputs)
    outs = gm(*inputs)
    torch.cuda.synchronize()
    fused.check_status()
    if isinstance(outs, torch.Tensor):
        outs = (outs,)
    # a fused dropout mask comes from the kernel's own generator: with keep probability 1 - 1e-19 it
    # must be all ones like the reference's, the other outputs then agree as usual
    for j in G.RANDOM_MASK_OUTPUTS.get(name, []):
        assert bool(outs[j].all()), (name, j)
    bool_outs = [j for j, o in enumerate(outs) if o.dtype == torch.bool and j not in G.RANDOM_MASK_OUTPUTS.get(name, [])]
    check_against_golden(name, list(outs), rtol=1e-2, atol=1e-3, full_numel=fused.ir.M * fused.ir.N * fused.ir.L,
                         skip=tuple(bool_outs))
    for j in bool_outs:
        # comparisons with zero flip where the fp32 sums of the two sides round differently: a handful of
        # the 4096 sampled elements at most
        import numpy as np
        from test_golden_cpu import golden_outputs
        flat = outs[j].detach().cpu().to(torch.float64).reshape(-1).numpy()
        want = golden_outputs(name)[j]["sample"]
        assert (flat[G.sample_index(flat.size)] != want).mean() < 2e-3, (name, j)


def _fused_on_gpu(case, device):
    inputs = [t.to(device) for t in case.inputs]
    gm, fused = fuse_module(case.module, inputs)
    outs = gm(*inputs)
    torch.cuda.synchronize()
    fused.check_status()
    return [outs] if isinstance(outs, torch.Tensor) else list(outs)


def test_fused_spmm_matches_the_reference_leaf(cuda_device):
    """python/gtl/compiler/passes/pass_decomposition.py:61-64 (`spmm`) on the seeded CSR of
    cases.leaf_inputs: fp32, 1e-5 relative + 1e-5 of the output's RMS."""
    import partitions as P
    case = P.spmm_case(G.SPMM["n"], G.SPMM["edges"], G.SPMM["F"], "plain")
    check_against_golden("leaf/spmm", _fused_on_gpu(case, cuda_device), rtol=1e-5, atol=1e-5, full_numel=0)


@pytest.mark.parametrize("leaf,geo", [("conv_fprop", G.CONV), ("conv_fprop_s2", G.CONV_S2), ("conv_dgrad", G.CONV),
                                      ("conv_dgrad_s2", G.CONV_S2), ("conv_wgrad", G.CONV), ("conv_wgrad_s2", G.CONV_S2)])
def test_fused_convolutions_match_the_reference_leaves(leaf, geo, cuda_device):
    """pass_decomposition.py:66-107 (channels-last forward, data-gradient and weight-gradient leaves)
    through the implicit-GEMM kernels, half-precision storage."""
    import partitions as P
    t = G.leaf_inputs(leaf)
    if leaf.startswith("conv_fprop"):
        case = P.conv_fprop_plain(geo["N"], geo["H"], geo["W"], geo["C"], geo["K"], geo["R"], geo["stride"][0])
        case.inputs = [t["x"], t["w"]]
    elif leaf.startswith("conv_wgrad"):
        case = P.conv_wgrad_plain(geo["N"], geo["H"], geo["W"], geo["C"], geo["K"], geo["R"], geo["stride"][0])
        case.inputs = [t["dy"], t["x"], t["w"]]
    else:
        case = P.conv_dgrad_strided(geo["N"], geo["H"], geo["W"], geo["C"], geo["K"], geo["R"], geo["stride"][0])
        case.inputs = [t["dy"], t["x"], t["w"]]
    outs = _fused_on_gpu(case, cuda_device)
    check_against_golden(f"leaf/{leaf}", outs[:1], rtol=1e-2, atol=1e-3, full_numel=outs[0].numel())


def test_batch_norm_leaves_on_gpu(cuda_device):
    """pass_decomposition.py:135-189: the four split batch-norm leaves chained, run on the GPU."""
    from evt_ae_b200 import ops
    t = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in G.leaf_inputs("batch_norm").items()}
    with torch.no_grad():
        outs = G.leaf_call(ops, "batch_norm", t)
    check_against_golden("leaf/batch_norm", list(outs), rtol=2e-3, atol=2e-3)


def test_fused_dropout_by_mask_reuse(cuda_device):
    """unittest/evt_fuser/dropout.py:33-75: x W^T + b, dropout with p = 0.7, residual.  The kernel
    draws its own mask; as in the reference's test the result is checked with that mask and the
    kept fraction must be 0.3 (1 M elements: three sigma = 1.4e-3; the bar is 2e-3)."""
    import partitions as P
    case = P.mm_bias_dropout_residual(1024, 1024, 1024, 512, 2, G.DROPOUT_P)
    case.inputs = G.dropout_inputs()
    out, keep = _fused_on_gpu(case, cuda_device)
    assert keep.dtype == torch.bool
    assert abs(keep.float().mean().item() - (1 - G.DROPOUT_P)) < 2e-3
    ref = G.dropout_formula(case.inputs, keep.cpu())
    from oracle import compare
    assert compare(out.cpu(), ref.reshape(out.shape), "half")["bad_frac"] == 0.0


def test_stem_convolution_and_batch_norm_match_the_reference_module(cuda_device):
    """unittest/evt_fuser/conv.py:33-49 at its full shape (128 x 4 x 224 x 224 -> 64 channels, 7x7 / 2,
    then training-mode batch norm): the fused forward convolution with the statistics in its epilogue on
    the window view of the image, then the normalising kernel."""
    from evt_ae_b200 import ops
    from evt_ae_b200.workloads import resnet as wr
    name = "conv_fprop_partition1"
    x, w, gamma, beta = [t.to(cuda_device) for t in G.golden_inputs(name)]
    xl, wl = x.permute(0, 2, 3, 1), w.permute(0, 2, 3, 1)
    win = ops.StemWindow(xl.shape, wl.shape, [2, 2], [3, 3])
    gm, fused = fuse_module(*wr.stem_modules(win, x.dtype)["fprop"])
    y, mean, msq = gm(win.image(xl), win.filter(wl))
    out, m, rstd = ops.bn_apply(y, mean, msq, gamma, beta, 1e-5)
    torch.cuda.synchronize()
    fused.check_status()
    check_against_golden(name, [out.permute(0, 3, 1, 2), m, rstd], rtol=1e-2, atol=1e-3, full_numel=out.numel())
