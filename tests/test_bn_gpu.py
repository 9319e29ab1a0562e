"""The one-pass batch-norm kernels (evtb_bn_apply, evtb_bn_backward_reduce, evtb_bn_backward_apply)
against the formulas of the reference's leaves (python/gtl/compiler/passes/pass_decomposition.py:
143-189) evaluated in fp32 / fp64 by PyTorch, with and without the fused ReLU, residual addition, ReLU
mask and gradient addition; channel counts that do and do not divide the CTA size, more than 2048
channels (several column blocks), row counts that leave ragged chunks.

Tolerances: outputs are rounded once to fp16 / bf16 (4e-3 / 2e-2 of the largest value); the sums are
fp32 atomics over n rows (1e-3 * sqrt(n) absolute + 1e-4 relative); the masked / added gradient that
is stored must equal PyTorch's rounding bit for bit."""
import pytest
import torch

from evt_ae_b200 import ops

pytestmark = pytest.mark.gpu

SHAPES = [(8, 5, 7, 64), (3, 9, 9, 192), (16, 14, 14, 1024), (2, 7, 7, 2048), (4, 3, 3, 4096), (32, 28, 28, 128)]


def _setup(shape, dt, dev):
    g = torch.Generator().manual_seed(sum(shape))
    C = shape[-1]
    rnd = lambda *s: torch.randn(*s, generator=g)
    y = (rnd(shape) * 1.5 + 0.3).to(dt).to(dev)
    gamma, beta = (torch.rand(C, generator=g) + 0.5).to(dt).to(dev), rnd(C).to(dt).to(dev)
    yf = y.float()
    mean, msq = yf.mean((0, 1, 2)), (yf * yf).mean((0, 1, 2))
    extra = [rnd(shape).to(dt).to(dev) for _ in range(3)]
    return y, yf, gamma, beta, mean, msq, torch.rsqrt(msq - mean * mean + 1e-5), extra


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_bn_apply(shape, dt, cuda_device):
    y, yf, gamma, beta, mean, msq, rstd, (res, _, _) = _setup(shape, dt, cuda_device)
    tol = 2e-2 if dt == torch.bfloat16 else 4e-3
    for relu in (False, True):
        for r in (None, res):
            z, m, rs = ops.bn_apply(y, mean, msq, gamma, beta, 1e-5, residual=r, relu=relu)
            ref = (yf - mean) * (gamma.float() * rstd) + beta.float()
            ref = ref + r.float() if r is not None else ref
            ref = ref.relu() if relu else ref
            assert (z.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
            assert torch.allclose(m, mean) and torch.allclose(rs, rstd, rtol=1e-5)
    # the reference's leaf signature routes here on the GPU
    z, m, rs = ops.batch_norm_elemt(y, gamma, beta, mean, msq, 1e-5, shape[-1])
    ref = (yf - mean) * (gamma.float() * rstd) + beta.float()
    assert (z.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_bn_backward(shape, dt, cuda_device):
    y, yf, gamma, beta, mean, msq, rstd, (g, g2, act) = _setup(shape, dt, cuda_device)
    C = shape[-1]
    n = g.numel() // C
    xhat = ((yf - mean) * rstd).double()
    for a in (None, act):
        for b in (None, g2):
            gm, sums = ops.bn_backward_reduce(g, y, mean, rstd, act=a, grad2=b)
            gr = g.float() + (b.float() if b is not None else 0.0)
            gr = (gr * (a > 0) if a is not None else gr).to(dt)
            assert torch.equal(gm, gr)
            s0, s1 = gr.double().sum((0, 1, 2)), (gr.double() * xhat).sum((0, 1, 2))
            for got, want in ((sums[0], s0), (sums[1], s1)):
                assert (got.double() - want).abs().max().item() <= 1e-3 * n ** 0.5 + 1e-4 * want.abs().max().item()
    _, sums = ops.bn_backward_reduce(g, y, mean, rstd)
    s0, s1 = ops.batch_norm_backward_stat(g, y, mean, rstd, C)          # the reference's leaf signature
    assert torch.allclose(s0, sums[0], rtol=1e-4, atol=1e-3 * n ** 0.5) and torch.allclose(s1, sums[1], rtol=1e-4, atol=1e-3 * n ** 0.5)
    rf = 1.0 / n
    tol = 2e-2 if dt == torch.bfloat16 else 4e-3
    ref = (g.float() - sums[0] * rf - xhat.float() * sums[1] * rf) * (gamma.float() * rstd)
    for dy, dgm, dbt in (ops.bn_backward_apply(g, y, mean, rstd, gamma, sums, rf),
                         ops.batch_norm_backward_elemt(g, y, mean, rstd, C, sums[0], sums[1], rf, gamma)):
        assert (dy.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
        assert torch.allclose(dgm.float(), sums[1], rtol=1e-2, atol=1e-2) and torch.allclose(dbt.float(), sums[0], rtol=1e-2, atol=1e-2)


def test_bn_refusals(cuda_device):
    y = torch.zeros(4, 2, 2, 12, device=cuda_device, dtype=torch.float16)          # 12 channels: not a multiple of 8
    v = torch.zeros(12, device=cuda_device)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ops.bn_apply(y, v, v, v.half(), v.half(), 1e-5)
    y = torch.zeros(2, 1, 1, 4104, device=cuda_device, dtype=torch.float16)
    v = torch.zeros(4104, device=cuda_device)
    with pytest.raises(RuntimeError, match="4096"):
        ops.bn_apply(y, v, v, v.half(), v.half(), 1e-5)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.bn_apply(torch.zeros(2, 1, 1, 8), torch.zeros(8), torch.zeros(8), torch.zeros(8), torch.zeros(8), 1e-5)
