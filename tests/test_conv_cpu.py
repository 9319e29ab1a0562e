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


def test_generated_epilogue_options():
    """What the code generator emits for the options that change an epilogue's structure (source level; the
    GPU tests run the kernels): column sums of a convolution are held back across a column strip for tiles
    of up to 128 columns and sent at once otherwise; the staged rows of a convolution take their output
    positions from the per-tile table; a second set of staging tiles alternates per chunk."""
    import torch
    import partitions as P
    from evt_ae_b200.codegen import ConvTileConfig, GemmTileConfig
    from evt_ae_b200.fuser import fuse_module
    case = P.conv_fprop_bn_stat(4, 28, 28, 128, 256, 3, 1)
    metas = [torch.empty(x.shape, dtype=x.dtype, device="meta") for x in case.inputs]
    _, narrow = fuse_module(case.module, metas, conv_tile=ConvTileConfig(bn=128))
    _, wide = fuse_module(case.module, metas, conv_tile=ConvTileConfig(bn=256))
    assert "flush_" in narrow.source and "dr_mask_" in narrow.source
    assert "flush_" not in wide.source and "red_add_f32(" in wide.source
    assert narrow.tile.stage_tiles == wide.tile.stage_tiles + 1          # the strip's partial sums
    for op in (narrow, wide):
        assert "(c).m_rows[" in op.source and "conv_row_to_m(*(c).conv" not in op.source
    g = P.mm_bias_gelu(512, 1024, 512, 128, 4, torch.bfloat16, "tanh")
    metas = [torch.empty(x.shape, dtype=x.dtype, device="meta") for x in g.inputs]
    _, one = fuse_module(g.module, metas, tile=GemmTileConfig(bn=128, stages=4))
    _, two = fuse_module(g.module, metas, tile=GemmTileConfig(bn=128, stages=4, double_buffer=True))
    assert "dbuf_" not in one.source and "tma_store_wait_read<0>" in one.source
    assert "dbuf_ ^= 1" in two.source and "tma_store_wait_read<1>" in two.source
    assert two.tile.stage_tiles == 2 * one.tile.stage_tiles
