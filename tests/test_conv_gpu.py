"""Fused implicit-GEMM convolutions (forward, data gradient, weight gradient; strides 1 and 2;
batch-norm statistics in the epilogue) on the GPU, through the C-ABI, against the fp32 unfused graph.
Tolerance as in test_gemm_gpu.py; reduction outputs scale with sqrt(positions reduced)."""
import pytest

import partitions as P
from test_gemm_gpu import run_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", P.small_conv_cases(), ids=lambda c: c.name)
def test_conv(case, cuda_device):
    fused = run_case(case, cuda_device)
    assert fused.plan.grid >= 1


def test_conv_narrow_and_wide_tiles(cuda_device):
    from evt_ae_b200.codegen import ConvTileConfig
    for bn in (64, 256):
        run_case(P.conv_fprop_bn_stat(4, 28, 28, 128, 256, 3, 1), cuda_device, conv_tile=ConvTileConfig(bn=bn))
        run_case(P.conv_dgrad_strided(4, 28, 28, 256, 128, 3, 2), cuda_device, conv_tile=ConvTileConfig(bn=bn))


@pytest.mark.parametrize("case", P.small_conv_wgrad_cases(), ids=lambda c: c.name)
def test_conv_weight_gradient(case, cuda_device):
    """dW as an implicit GEMM over boxes of output positions (the reference's cuDNN leaf,
    pass_decomposition.py:92-107): strides 1 and 2, 1x1 and 3x3, fewer output channels than a tile
    is tall, ragged boxes."""
    fused = run_case(case, cuda_device)
    assert fused.plan.grid >= 1


def test_conv_weight_gradient_split_and_tiles(cuda_device):
    """The reduction over N*P*Q cut into units whose fp32 partial tiles meet in the workspace, twice on
    one workspace; every channel-tile width."""
    from evt_ae_b200.codegen import GemmTileConfig
    for bn, split in [(64, 7), (128, 4), (256, 2), (64, 1)]:
        case = P.conv_wgrad_plain(8, 28, 28, 256, 128, 3, 1)
        fused = run_case(case, cuda_device, tile=GemmTileConfig(bn=bn, stages=4, split_k=split))
        assert fused.tile.split_k == split
    case = P.conv_wgrad_plain(16, 28, 28, 128, 128, 3, 1)
    fused = run_case(case, cuda_device)
    assert fused.tile.split_k > 1 and fused.plan.workspace_bytes > 0
    run_case(case, cuda_device)


@pytest.mark.parametrize("N,H,W,C,K,R,s,pad", [(4, 64, 64, 3, 64, 7, 2, 3), (2, 40, 56, 4, 64, 7, 2, 3), (2, 30, 30, 8, 64, 3, 1, 1),
                                               (3, 33, 47, 4, 128, 5, 2, 2)])
def test_few_channel_convolution_through_window_view(N, H, W, C, K, R, s, pad, cuda_device):
    """A stem convolution (few input channels) through the ordinary fused forward (+ batch-norm
    statistics) and weight-gradient kernels: the activation is an overlapping 64-wide window view of the
    zero-padded image (ops.StemWindow, strides passed to the plan), the filter rows are laid into the
    windows.  Compared with the fp32 convolution of the original tensors on the CPU: outputs to 1e-2
    relative + 1e-3 x RMS, statistics (means over N*P*Q positions) to 1e-3 x RMS of the output (its
    square for the second moment), filter gradient to 1e-2 relative + 1e-2 x RMS."""
    import torch
    from evt_ae_b200 import ops
    from evt_ae_b200.fuser import fuse_module
    from evt_ae_b200.workloads import resnet as wr
    dt = torch.float16
    g = torch.Generator().manual_seed(N * 1000 + H)
    x = torch.randn(N, H, W, C, generator=g).to(dt)
    w = (torch.randn(K, R, R, C, generator=g) * 0.2).to(dt)
    win = ops.StemWindow(x.shape, w.shape, [s, s], [pad, pad])
    dy = torch.randn(N, win.P, win.Q, K, generator=g).to(dt)
    mods = wr.stem_modules(win, dt)
    gm_f, op_f = fuse_module(*mods["fprop"])
    gm_w, op_w = fuse_module(*mods["wgrad"])
    assert op_f.view_strides == win.view_strides and op_w.view_strides == win.view_strides
    xv, wv = win.image(x.to(cuda_device)), win.filter(w.to(cuda_device))
    y, mean, msq = gm_f(xv, wv)
    dw = win.unfold(gm_w(dy.to(cuda_device), xv, wv))
    torch.cuda.synchronize()
    op_f.check_status()
    op_w.check_status()
    ref = ops.convolution_forward_channel_last(x.float(), w.float(), [s, s], [pad, pad], [1, 1], False, [0, 0], 1)
    rms = ref.pow(2).mean().sqrt().item()
    assert (y.float().cpu() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-3 * rms
    assert (mean.reshape(-1).cpu() - ref.mean((0, 1, 2))).abs().max().item() <= 1e-3 * rms
    assert (msq.reshape(-1).cpu() - (ref * ref).mean((0, 1, 2))).abs().max().item() <= 1e-3 * rms * rms
    dref = ops.convolution_backward_weight_channel_last(dy.float(), x.float(), w.float(), [s, s], [pad, pad], [1, 1], False, [0, 0], 1)
    drms = dref.pow(2).mean().sqrt().item()
    assert dw.shape == dref.shape
    assert (dw.float().cpu() - dref).abs().max().item() <= 1e-2 * dref.abs().max().item() + 1e-2 * drms
    # a dense tensor where the plan expects the view is refused, not misread
    with pytest.raises(RuntimeError, match="strides"):
        gm_f(xv.contiguous(), wv)
