"""The fused ViT step on the GPU (bf16, 13 + 1 tokens padded to 16 with masked tokens) against fp32
autograd of the UNPADDED model on CPU.  Bars as for the BERT step: loss to 1e-2 relative, every
parameter gradient to 3e-2 relative Frobenius error (plus a floor tied to the typical gradient
size for tensors that are zero by construction)."""
import pytest
import torch

from evt_ae_b200.workloads import vit as wv
from oracle import vit_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layers,dim,heads,mlp,image,patch,B", [(2, 128, 2, 256, 40, 8, 4), (1, 256, 4, 512, 48, 16, 8)])
def test_vit_step_gradients(layers, dim, heads, mlp, image, patch, B, cuda_device):
    cfg = wv.VitConfig(layers=layers, dim=dim, heads=heads, mlp=mlp, image=image, patch=patch, classes=10)
    assert cfg.tokens_padded > cfg.tokens          # the padding path is exercised
    dt, dev = torch.bfloat16, cuda_device
    params = {k: v.to(dt).to(torch.float32) for k, v in wv.init_params(cfg, seed=3, dtype=torch.float32).items()}
    images, labels = wv.synthetic_batch(cfg, B, seed=3)
    images = images.to(dt).to(torch.float32)
    ref_loss, ref_grads = vit_ref.loss_and_grads(params, cfg, images, labels)

    step = wv.VitStep(cfg, B, dtype=dt)
    p = {k: v.to(dt).to(dev) for k, v in params.items()}
    tok, pm = step.embed_tokens(p, images.to(dev))
    loss, grads, dtok = step.step(p, tok, labels.to(dev))
    grads.update(step.embed_backward(dtok, pm))
    torch.cuda.synchronize()
    step.check_status()
    assert abs(loss.item() - ref_loss.item()) <= 1e-2 * abs(ref_loss.item()), (loss.item(), ref_loss.item())
    assert set(grads) == set(ref_grads)
    # padded rows carry no gradient
    assert float(dtok[cfg.tokens:].float().abs().max()) == 0.0
    typical = sorted((r.norm().item() / r.numel() ** 0.5) for r in ref_grads.values())[len(ref_grads) // 2]
    for k, r in ref_grads.items():
        g = grads[k].float().cpu().reshape(r.shape)
        err = (g - r).norm().item()
        assert err <= 3e-2 * r.norm().item() + 2e-2 * typical * r.numel() ** 0.5, (k, err, r.norm().item())
