"""CTA-pair GEMM (cluster of two CTAs, tcgen05 cta_group::2) against the fp32 unfused graph:
every operand layout, ragged edges, batches, many tiles per pair (accumulator and ring reuse),
both tile widths, 8 and 16 epilogue warps.  Same tolerance as test_gemm_gpu.py."""
import pytest
import torch

import partitions as P
from evt_ae_b200.codegen import GemmTileConfig
from test_gemm_gpu import run_case

pytestmark = pytest.mark.gpu


def pair(bn=256, ew=8):
    return GemmTileConfig(bn=bn, stages=8, epi_warps=ew, cta_pair=True)


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pair_every_layout_ragged(a_t, b_t, dtype, cuda_device):
    run_case(P.mm_plain(556, 520, 200, a_t, b_t, dtype), cuda_device, tile=pair())


@pytest.mark.parametrize("bn,ew", [(128, 8), (256, 16), (128, 16)])
def test_pair_tile_widths_and_epilogue_warps(bn, ew, cuda_device):
    run_case(P.config0(640, 384, 256), cuda_device, tile=pair(bn, ew))


def test_pair_many_tiles_per_pair(cuda_device):
    """512 pair tiles: every pair walks several tiles, so both accumulator stages and every ring
    slot are reused with flipped phases."""
    fused = run_case(P.mm_bias_gelu(8192, 4096, 320, 64, 128, torch.bfloat16, "tanh"), cuda_device, tile=pair())
    assert fused.plan.grid % 2 == 0 and fused.plan.grid >= 64


def test_pair_batched(cuda_device):
    run_case(P.bmm_scores_mask(256, 2, 4, 64), cuda_device, tile=pair())


def test_pair_weight_gradient_long_k_twice(cuda_device):
    from evt_ae_b200.fuser import fuse_module
    from oracle import compare, run_unfused_fp32
    case = P.mm_wgrad(1024, 4096, 16384, torch.bfloat16)
    inputs = [t.to(cuda_device) for t in case.inputs]
    gm, fused = fuse_module(case.module, inputs, tile=pair())
    ref = run_unfused_fp32(case.module, case.inputs)[0]
    for _ in range(2):
        out = gm(*inputs)
        torch.cuda.synchronize()
        fused.check_status()
        st = compare(out, ref, "half")
        assert st["bad_frac"] == 0.0, st


@pytest.mark.parametrize("split,bn", [(2, 128), (3, 256), (5, 256)])
def test_pair_split_k(split, bn, cuda_device):
    """Split-K on CTA pairs: every CTA parks the partial of its own 128-row half; ragged M and N,
    a bias-gradient reduction in the epilogue of the last arriver."""
    case = P.mm_tanh_backward_sum(600, 200, 1024 + 64)
    run_case(case, cuda_device, tile=GemmTileConfig(bn=bn, stages=8, split_k=split, cta_pair=True))
