"""ResNet-50 (v1.5 bottlenecks, batch norm on batch statistics, summed cross-entropy) in plain
PyTorch, fp32 autograd, NCHW -- ORACLE ONLY.

Restates python/model_zoo/resnet/resnet_modeling.py:37-260 of the reference (torchvision's topology
with `track_running_stats=False` and `CrossEntropyLoss(reduction="sum")`) on the parameter dictionary of
evt_ae_b200/workloads/resnet.py (filters in channels-last [K, R, S, C] layout).  No reference-generated
numbers pin it: the reference's model object needs its CUTLASS fork to be built."""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn.functional as F


def loss_and_grads(params: Dict[str, torch.Tensor], cfg, arch, images_nhwc, labels, dtype=torch.float32, device="cpu",
                   prepared=None):
    """`arch` = evt_ae_b200.workloads.resnet._arch(cfg).  Returns (loss, grads) with filter gradients in
    the [K, R, S, C] layout of the parameters.  `dtype` / `device` other than fp32 on the CPU give the
    same autograd model in reduced precision: the yardstick for how much of a difference to the fp32
    result is rounding that any half-precision run of this network shows."""
    if prepared is None:
        # filters stored channels-last in memory (as the reference runs the model): the NCHW view below
        # is then a channels_last tensor
        p = {k: v.detach().clone().to(dtype).to(device).requires_grad_(True) for k, v in params.items()}
    else:
        p = prepared                       # the dictionary of an earlier call: no clones (bench.py's eager leg)
        for v in p.values():
            v.grad = None
    images_nhwc, labels = images_nhwc.to(device), labels.to(device)

    def conv_bn(x, name, stride, r):
        w = p[name + ".w"].permute(0, 3, 1, 2)
        y = F.conv2d(x, w, None, stride, r // 2)
        return F.batch_norm(y, None, None, p[name + ".bn.g"], p[name + ".bn.b"], True, 0.0, cfg.eps)
    x = images_nhwc.to(dtype).permute(0, 3, 1, 2)
    x = F.max_pool2d(torch.relu(conv_bn(x, "stem", 2, 7)), 3, 2, 1)
    for pre, convs, down in arch:
        identity = x
        out = x
        for j, (name, c, k, r, s) in enumerate(convs):
            out = conv_bn(out, name, s, r)
            if j < 2:
                out = torch.relu(out)
        if down is not None:
            identity = conv_bn(x, down[0], down[4], down[3])
        x = torch.relu(out + identity)
    feat = x.mean(dim=(2, 3))
    loss = F.cross_entropy(F.linear(feat, p["fc.w"], p["fc.b"]).float(), labels, reduction="sum")
    loss.backward()
    if prepared is not None:
        return loss.detach(), {k: v.grad for k, v in p.items()}, p
    return loss.detach().cpu(), {k: v.grad.float().cpu() for k, v in p.items()}
