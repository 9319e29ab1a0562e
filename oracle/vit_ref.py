"""ViT in plain PyTorch (fp32, autograd) -- ORACLE ONLY.

Restates the reference's model (python/model_zoo/vit/vit_modeling.py:13-160: PreNorm attention and
MLP blocks in [S, B, H] token order, erf GELU, linear patch embedding, class token, learned
positions, LayerNorm + linear head on the class token) WITHOUT any token padding: the fused step
in evt_ae_b200/workloads/vit.py pads 197 tokens to 200 with masked tokens and must reproduce this
module's loss and gradients.  No reference-generated numbers pin it (the reference's own model
needs its CUTLASS fork to run)."""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn.functional as F


def patchify(cfg, images):
    B, C, H, W = images.shape
    p = cfg.patch
    x = images.reshape(B, C, H // p, p, W // p, p).permute(2, 4, 0, 1, 3, 5)
    return x.reshape(cfg.patches, B, C * p * p)


def loss_and_grads(params: Dict[str, torch.Tensor], cfg, images, labels, dtype=torch.float32, device="cpu", prepared=None):
    """`dtype` / `device` other than fp32 on the CPU give the same autograd model in reduced precision
    (the eager-PyTorch baseline of bench.py); `prepared` reuses a parameter dictionary made by an
    earlier call (returned as third value when given) instead of cloning the parameters again."""
    if prepared is None:
        p = {k: v.detach().clone().to(dtype).to(device).requires_grad_(True) for k, v in params.items()}
    else:
        p = prepared
        for v in p.values():
            v.grad = None
    images, labels = images.to(device), labels.to(device)
    B = images.shape[0]
    D, nh = cfg.dim, cfg.heads
    d = D // nh
    e = F.linear(patchify(cfg, images.to(dtype)), p["embed.w"], p["embed.b"])       # [patches, B, D]
    x = torch.cat([(p["cls"] + p["pos"][0]).expand(1, B, D), e + p["pos"][1:].unsqueeze(1)], 0)
    S = x.shape[0]
    for i in range(cfg.layers):
        pre = f"l{i}."
        n1 = F.layer_norm(x, (D,), p[pre + "ln1.g"], p[pre + "ln1.b"], cfg.eps)
        q = F.linear(n1, p[pre + "q.w"], p[pre + "q.b"]).view(S, B * nh, d).transpose(0, 1)
        k = F.linear(n1, p[pre + "k.w"], p[pre + "k.b"]).view(S, B * nh, d).permute(1, 2, 0)
        v = F.linear(n1, p[pre + "v.w"], p[pre + "v.b"]).view(S, B * nh, d).transpose(0, 1)
        pr = torch.softmax(torch.bmm(q, k) * (d ** -0.5), -1)
        ctx = torch.bmm(pr, v).transpose(0, 1).contiguous().view(S, B, D)
        x = F.linear(ctx, p[pre + "o.w"], p[pre + "o.b"]) + x
        n2 = F.layer_norm(x, (D,), p[pre + "ln2.g"], p[pre + "ln2.b"], cfg.eps)
        x = F.linear(F.gelu(F.linear(n2, p[pre + "ff1.w"], p[pre + "ff1.b"])), p[pre + "ff2.w"], p[pre + "ff2.b"]) + x
    z = F.linear(F.layer_norm(x[0], (D,), p["head.ln.g"], p["head.ln.b"], cfg.eps), p["head.w"], p["head.b"])
    loss = F.cross_entropy(z.float(), labels)
    loss.backward()
    if prepared is not None:
        return loss.detach(), {k: v.grad for k, v in p.items()}, p
    return loss.detach(), {k: v.grad for k, v in p.items()}
