"""Fused softmax / LayerNorm nodes (forward and backward) on the GPU, through the C-ABI,
against the fp32 unfused graph.  Tolerance as in test_gemm_gpu.py: |out - ref| <=
1e-2 |ref| + 1e-3 for half-precision outputs; per-row statistics (fp32) likewise;
boolean outputs exact."""
import pytest
import torch

import partitions as P
from evt_ae_b200.fuser import fuse_module
from oracle import compare, run_unfused_fp32

pytestmark = pytest.mark.gpu


def run_case(case, device):
    inputs = [t.to(device) for t in case.inputs]
    gm, fused = fuse_module(case.module, inputs)
    out = gm(*inputs)
    torch.cuda.synchronize()
    fused.check_status()
    if isinstance(out, torch.Tensor):
        out = (out,)
    ref = run_unfused_fp32(case.module, case.inputs)
    assert len(out) == len(ref)
    for o, r in zip(out, ref):
        # a reduction that consumes a fused output (computed outside the node, in the storage
        # dtype) carries the rounding of every row it adds up
        reduced = r.dtype.is_floating_point and r.numel() * 2 <= fused.ir.M * fused.ir.N and r.shape[-1] == fused.ir.N
        st = compare(o.reshape(r.shape), r, "half", reduction=reduced)
        assert st["bad_frac"] == 0.0, (case.name, tuple(r.shape), st)
    return fused


@pytest.mark.parametrize("case", P.small_row_cases(torch.float16), ids=lambda c: c.name)
def test_row_kernels_fp16(case, cuda_device):
    run_case(case, cuda_device)


@pytest.mark.parametrize("case", [c for c in P.small_row_cases(torch.bfloat16) if "float32" not in c.name][:14:2],
                         ids=lambda c: c.name)
def test_row_kernels_bf16(case, cuda_device):
    run_case(case, cuda_device)


def test_softmax_dropout_mask_reuse(cuda_device):
    """Fused dropout: the mask is an output; check density and that out == softmax * mask /
    (1 - p) with the produced mask (the reference's method, unittest/evt_fuser/dropout.py:63-75)."""
    p = 0.1
    case = P.softmax_dropout(2, 4, 128, p)
    inputs = [t.to(cuda_device) for t in case.inputs]
    gm, fused = fuse_module(case.module, inputs)
    s, mask, out = gm(*inputs)
    torch.cuda.synchronize()
    fused.check_status()
    assert mask.dtype == torch.bool
    density = mask.float().mean().item()
    assert abs(density - (1 - p)) < 2e-2, density
    ref_s = torch.softmax(case.inputs[0].float(), -1)
    assert compare(s, ref_s, "half")["bad_frac"] == 0.0
    ref_out = (ref_s * mask.cpu().float() / (1 - p)).reshape(out.shape)
    assert compare(out, ref_out, "half")["bad_frac"] == 0.0
    # a second call draws a different mask
    _, mask2, _ = gm(*inputs)
    assert (mask2 != mask).any().item()
