"""Max-pooling kernels (evtb_maxpool_forward / evtb_maxpool_backward) through the leaves of the same names
as the reference's (python/gtl/compiler/passes/pass_decomposition.py:109-132) against the library's
max_pool2d_with_indices on the same tensors: outputs equal bit for bit, the one-byte window places decode
to the library's int64 indices (inputs after a ReLU, so that windows of equal values are common: ties go
to the first maximum in scan order on both sides), gradients equal up to the order of at most four fp32
additions (1e-3 relative)."""
import pytest
import torch

from evt_ae_b200 import ops

pytestmark = pytest.mark.gpu

CASES = [(2, 16, 16, 64, 3, 2, 1), (3, 17, 23, 8, 3, 2, 1), (2, 12, 12, 16, 2, 2, 0), (1, 9, 14, 24, 3, 1, 1),
         (2, 15, 15, 8, 5, 3, 2), (8, 112, 112, 64, 3, 2, 1)]


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,H,W,C,k,s,p", CASES)
def test_maxpool_matches_library(N, H, W, C, k, s, p, dt, cuda_device):
    g = torch.Generator().manual_seed(N * 100 + H)
    x = torch.relu(torch.randn(N, H, W, C, generator=g)).to(dt).to(cuda_device)
    y, code = ops.max_pool2d_with_indices_channel_last(x, [k, k], [s, s], [p, p])
    assert code.dtype == torch.uint8
    ref_y, ref_idx = torch.ops.aten.max_pool2d_with_indices(x.permute(0, 3, 1, 2), [k, k], [s, s], [p, p])
    ref_y, ref_idx = ref_y.permute(0, 2, 3, 1), ref_idx.permute(0, 2, 3, 1)
    assert torch.equal(y, ref_y)
    P, Q = y.shape[1], y.shape[2]
    ph = torch.arange(P, device=cuda_device).view(1, P, 1, 1)
    pw = torch.arange(Q, device=cuda_device).view(1, 1, Q, 1)
    c = code.long()
    idx = (ph * s - p + c // k) * W + (pw * s - p + c % k)
    assert torch.equal(idx, ref_idx)
    dy = torch.randn(y.shape, generator=g).to(dt).to(cuda_device)
    dx = ops.max_pool2d_with_indices_backward_channel_last(dy, x, [k, k], [s, s], [p, p], [1, 1], False, code)
    ref_dx = torch.ops.aten.max_pool2d_with_indices_backward(dy.permute(0, 3, 1, 2), x.permute(0, 3, 1, 2), [k, k], [s, s], [p, p],
                                                             [1, 1], False, ref_idx.permute(0, 3, 1, 2)).permute(0, 2, 3, 1)
    assert dx.shape == x.shape
    assert torch.allclose(dx.float(), ref_dx.float(), rtol=1e-3, atol=1e-3 if dt == torch.float16 else 1e-2)


def test_maxpool_nan_and_refusals(cuda_device):
    x = torch.zeros(1, 4, 4, 8, device=cuda_device, dtype=torch.float16)
    x[0, 1, 1, 3] = float("nan")
    y, code = ops.max_pool2d_with_indices_channel_last(x, [3, 3], [2, 2], [1, 1])
    ref_y, _ = torch.ops.aten.max_pool2d_with_indices(x.permute(0, 3, 1, 2), [3, 3], [2, 2], [1, 1])
    assert torch.equal(torch.isnan(y), torch.isnan(ref_y.permute(0, 2, 3, 1)))
    with pytest.raises(NotImplementedError):
        ops.max_pool2d_with_indices_channel_last(x, [3, 2], [2, 2], [1, 1])
    # channel counts that are not multiples of 8 take the library path (int64 indices)
    x5 = torch.randn(1, 6, 6, 5, device=cuda_device).half()
    _, idx = ops.max_pool2d_with_indices_channel_last(x5, [3, 3], [2, 2], [1, 1])
    assert idx.dtype == torch.int64
