"""The unfused graph in fp32 eager PyTorch on CPU, and the comparison rule.

Follows python/gtl/helper/test_helper.py:78-104 (`UnitTestBase.util_test`: run the same
module unfused and compare with `torch.allclose`) and the in-situ check at
python/gtl/compiler/passes/evt_fuser.py:85-96, 126-141 (rtol 1e-2, atol 1e-3).
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

# per-element |out - ref| <= rtol * |ref| + atol
TOL = {
    "half": dict(rtol=1e-2, atol=1e-3),     # fp16 / bf16 storage, fp32 accumulate
    "fp32": dict(rtol=1e-5, atol=1e-6),     # fp32 SpMM / SDDMM
}


def _up(t):
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu()
        if t.dtype in (torch.float16, torch.bfloat16):
            t = t.to(torch.float32)
    return t


def run_unfused_fp32(module: torch.nn.Module, inputs: Sequence[torch.Tensor]):
    """Run `module` unfused, on CPU, with every half-precision input upcast to fp32."""
    # a module that names a storage dtype in an aten call keeps it in `.dt`
    saved = getattr(module, "dt", None)
    if saved is not None:
        module.dt = torch.float32
    try:
        with torch.no_grad():
            out = module(*[_up(x) for x in inputs])
    finally:
        if saved is not None:
            module.dt = saved
    if isinstance(out, torch.Tensor):
        out = (out,)
    return tuple(out)


def compare(out: torch.Tensor, ref: torch.Tensor, kind: str = "half", scale_atol: float = 1.0,
            reduction: bool = False) -> Dict[str, float]:
    """Returns max abs / max rel error and the fraction of elements outside the tolerance
    |out - ref| <= rtol |ref| + floor.  The absolute floor is tied to the magnitude of the
    reference itself: atol x max(1, RMS(ref)) for an elementwise result (the resolution of 16-bit
    storage at that magnitude), rtol x RMS(ref) for a reduction result (sums of terms of both
    signs land near zero, where a relative bound per element means nothing).  Integer and boolean
    tensors must match exactly."""
    out = out.detach().cpu()
    ref = ref.detach().cpu()
    assert out.shape == ref.shape, (out.shape, ref.shape)
    if not out.dtype.is_floating_point or not ref.dtype.is_floating_point:
        mism = (out.to(torch.int64) != ref.to(torch.int64)).double().mean().item()
        return dict(max_abs=float(mism > 0), max_rel=float(mism > 0), bad_frac=mism)
    o = out.to(torch.float64)
    r = ref.to(torch.float64)
    tol = TOL[kind]
    err = (o - r).abs()
    finite = r[torch.isfinite(r)]
    rms = float(finite.pow(2).mean().sqrt()) if finite.numel() else 0.0
    floor = max(tol["atol"], tol["rtol"] * rms) if reduction else tol["atol"] * max(1.0, rms)
    bad = err > (tol["rtol"] * r.abs() + floor * scale_atol)
    bad |= torch.isnan(o) != torch.isnan(r)
    rel = err / r.abs().clamp_min(1e-6)
    return dict(max_abs=err.max().item() if err.numel() else 0.0,
                max_rel=rel.max().item() if rel.numel() else 0.0,
                bad_frac=bad.double().mean().item() if bad.numel() else 0.0)
