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
