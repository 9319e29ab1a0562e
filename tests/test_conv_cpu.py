"""Convolution partitions: tracer + index maps vs the unfused module on CPU."""
import pytest

import partitions as P
from helpers import check_ir_against_module


@pytest.mark.parametrize("case", P.small_conv_cases(), ids=lambda c: c.name)
def test_conv_ir_matches_unfused_module(case):
    tr, stats = check_ir_against_module(case)
    assert tr.kind in ("conv_fprop", "conv_dgrad") and stats
    for st in stats:
        assert st["bad_frac"] == 0.0, st
    if "bn" in case.name:
        assert tr.ir.statistics()["row_red"] == 2      # two [channels] reductions ride in the epilogue


def test_stem_window_restates_the_convolution():
    """ops.StemWindow on the CPU: the R x 1 convolution over 64-wide windows of the zero-padded image,
    with the filter rows laid into the windows, is the original few-channel convolution (exactly, same
    fp32 arithmetic), window starts are 16-byte aligned, and the filter gradient folds back."""
    import torch
    from evt_ae_b200 import ops
    g = torch.Generator().manual_seed(3)
    for (N, H, W, C, K, R, s, pd) in [(2, 32, 32, 3, 16, 7, 2, 3), (2, 20, 28, 4, 8, 7, 2, 3), (1, 16, 16, 8, 8, 3, 1, 1),
                                      (2, 17, 19, 4, 8, 5, 2, 2)]:
        x, w = torch.randn(N, H, W, C, generator=g), torch.randn(K, R, R, C, generator=g)
        win = ops.StemWindow(x.shape, w.shape, [s, s], [pd, pd])
        xv, wv = win.image(x), win.filter(w)
        assert tuple(xv.shape) == win.view_shape and tuple(xv.stride()) == win.view_strides
        assert all(v % 8 == 0 for v in win.view_strides[:3]) and win.view_strides[3] == 1
        ref = ops.convolution_forward_channel_last(x, w, [s, s], [pd, pd], [1, 1], False, [0, 0], 1)
        got = ops.convolution_forward_channel_last(xv, wv, win.stride, win.padding, [1, 1], False, [0, 0], 1)
        assert got.shape == ref.shape == (N, win.P, win.Q, K) and torch.allclose(got, ref, rtol=1e-5, atol=1e-5)
        dy = torch.randn(ref.shape, generator=g)
        dref = ops.convolution_backward_weight_channel_last(dy, x, w, [s, s], [pd, pd], [1, 1], False, [0, 0], 1)
        dwin = ops.convolution_backward_weight_channel_last(dy, xv, wv, win.stride, win.padding, [1, 1], False, [0, 0], 1)
        assert torch.allclose(win.unfold(dwin), dref, rtol=1e-4, atol=1e-4)
    import pytest
    with pytest.raises(NotImplementedError):
        ops.StemWindow((1, 8, 8, 4), (8, 3, 3, 4), [1, 1], [1, 1])       # stride 1 x 4 channels: 8-byte window steps
    with pytest.raises(NotImplementedError):
        ops.StemWindow((1, 64, 64, 16), (8, 7, 7, 16), [2, 2], [3, 3])   # 7 taps do not fit 4 pixels of 16 channels
