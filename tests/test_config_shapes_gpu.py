"""Parity at the shapes of the BASELINE configurations that are not the benchmark workload:
ViT-B/16 (197 tokens: pitches that are not multiples of 8 elements, so operands are materialised
padded and results leave through the per-lane store path) at a reduced batch, and ResNet-50
convolutions at the configuration's full batch of 128.  Same tolerances as the per-operator
tests; the oracle is the fp32 unfused module on CPU."""
import pytest
import torch

import partitions as P
from test_gemm_gpu import run_case as run_gemm_case
from test_rowkernels_gpu import run_case as run_row_case

pytestmark = pytest.mark.gpu

BF = torch.bfloat16
VIT_B, VIT_S, VIT_H, VIT_D, VIT_DIM, VIT_MLP = 8, 197, 12, 64, 768, 3072


@pytest.mark.parametrize("case", [
    P.bmm_scores_mask(VIT_S, VIT_B, VIT_H, VIT_D, BF),                      # 96 x (197 x 197 x 64)
    P.bmm_context_permuted_store(VIT_S, VIT_B, VIT_H, VIT_D, BF),           # 96 x (197 x 64 x 197)
    P.bmm_dgrad_sum(VIT_S, VIT_B, VIT_H, VIT_D, BF),
    P.mm_bias_gelu(VIT_B * VIT_S, VIT_MLP, VIT_DIM, VIT_S, VIT_B, BF, "tanh"),   # MLP up
    P.mm_residual_permute(VIT_B * VIT_S, VIT_DIM, VIT_MLP, VIT_S, VIT_B, BF),    # MLP down + residual
    P.mm_wgrad(VIT_DIM, VIT_MLP, VIT_B * VIT_S, BF),                        # weight gradient, K = 1576
], ids=lambda c: c.name)
def test_vit_gemm_shapes(case, cuda_device):
    run_gemm_case(case, cuda_device)


@pytest.mark.parametrize("case", [
    P.softmax_plain(VIT_B * VIT_H * VIT_S, VIT_S, BF, shape=(VIT_B, VIT_H, VIT_S, VIT_S)),
    P.softmax_backward_plain((VIT_B * VIT_H, VIT_S, VIT_S), BF),
    P.layernorm_affine(VIT_S, VIT_B, VIT_DIM, BF),
    P.layernorm_backward_mask(VIT_S, VIT_B, VIT_DIM, BF),
], ids=lambda c: c.name)
def test_vit_row_kernel_shapes(case, cuda_device):
    run_row_case(case, cuda_device)


@pytest.mark.parametrize("case", [
    P.conv_fprop_bn_stat(128, 56, 56, 64, 64, 3, 1),          # conv2_x 3x3 at the configuration's batch
    P.conv_dgrad_strided(128, 28, 28, 128, 256, 3, 2),        # unittest/evt_fuser/conv.py:80-97 at full size
    P.conv_wgrad_plain(128, 56, 56, 64, 64, 3, 1),            # weight gradient of conv2_x 3x3: 401,408 positions reduced
    P.conv_wgrad_plain(128, 14, 14, 256, 256, 3, 1),          # conv4_x 3x3
], ids=lambda c: c.name)
def test_resnet_conv_full_batch(case, cuda_device):
    run_gemm_case(case, cuda_device)
