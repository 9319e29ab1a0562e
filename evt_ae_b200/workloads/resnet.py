"""ResNet-50 training step (forward + backward), channels-last fp16.

Topology: the reference's model (python/model_zoo/resnet/resnet_modeling.py: torchvision's v1.5
bottleneck ResNet, batch norm without running statistics, cross-entropy summed over the batch).
What the reference's decomposition pass makes of it (pass_decomposition.py:66-189) is what runs here:

  every convolution   -> fused implicit GEMM whose epilogue also emits the per-channel E[y], E[y^2]
                         of training-mode batch norm (`batch_norm_stat`, fused as in evt_fuser.py:1272-1284)
  batch-norm apply    -> `batch_norm_elemt` + residual addition + ReLU in one pass (ops.bn_apply; the
                         reference hands these partitions to TorchScript, nv_fuser.py:224-244)
  backward            -> gradient addition + ReLU mask + `batch_norm_backward_stat` in one pass
                         (ops.bn_backward_reduce), `batch_norm_backward_elemt` in one pass
                         (ops.bn_backward_apply), fused data-gradient and weight-gradient convolutions
  7x7 three-channel stem
                      -> the same fused forward (+ statistics) and weight-gradient kernels on a window
                         view of the zero-padded image: the 7 taps of a filter row times the channels
                         become the 64 "channels" the kernels move at a time (ops.StemWindow)
  max-pool            -> the reference's leaves (pass_decomposition.py:109-132) on this library's kernels
                         (ops.max_pool2d_with_indices_channel_last: one byte per output element
                         instead of an int64 index)
  average pool + classifier + loss
                      -> eager calls on [batch, 2048] tensors
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

from .. import ops, tuning
from ..fused_ops import ReductionArena
from ..fuser import fuse_module

aten = torch.ops.aten
for _name in ("convolution_forward_channel_last", "convolution_backward_data_channel_last",
              "convolution_backward_weight_channel_last"):
    globals()[_name] = getattr(ops, _name)
    torch.fx.wrap(_name)


@dataclass
class ResNetConfig:
    layers: Tuple[int, ...] = (3, 4, 6, 3)
    width: int = 64
    classes: int = 1000
    image: int = 224
    in_channels: int = 3
    eps: float = 1e-5


RESNET50 = ResNetConfig()


def _arch(cfg: ResNetConfig):
    """[(name, C_in, K_out, R, stride)] of every convolution after the stem, in forward order, grouped
    per bottleneck block: (conv1 1x1, conv2 3x3 (carries the stride), conv3 1x1, optional downsample 1x1)."""
    blocks = []
    inp = cfg.width
    for si, nblocks in enumerate(cfg.layers):
        planes = cfg.width * (2 ** si)
        for bi in range(nblocks):
            stride = 2 if (bi == 0 and si > 0) else 1
            pre = f"s{si}.b{bi}."
            convs = [(pre + "conv1", inp, planes, 1, 1), (pre + "conv2", planes, planes, 3, stride),
                     (pre + "conv3", planes, planes * 4, 1, 1)]
            down = (pre + "down", inp, planes * 4, 1, stride) if (stride != 1 or inp != planes * 4) else None
            blocks.append((pre, convs, down))
            inp = planes * 4
    return blocks


def init_params(cfg: ResNetConfig, seed: int = 1236, dtype=torch.float16, device="cpu") -> Dict[str, torch.Tensor]:
    """Kaiming-normal (fan-out) filters in channels-last [K, R, S, C] layout, unit gains, zero shifts."""
    g = torch.Generator().manual_seed(seed)

    def conv(k, r, c):
        std = (2.0 / (k * r * r)) ** 0.5
        return (torch.randn(k, r, r, c, generator=g) * std).to(dtype).to(device)
    p = {"stem.w": conv(cfg.width, 7, cfg.in_channels), "stem.bn.g": torch.ones(cfg.width), "stem.bn.b": torch.zeros(cfg.width)}
    for pre, convs, down in _arch(cfg):
        for name, c, k, r, _ in convs + ([down] if down else []):
            p[name + ".w"] = conv(k, r, c)
            p[name + ".bn.g"], p[name + ".bn.b"] = torch.ones(k), torch.zeros(k)
    feat = cfg.width * 8 * 4
    p["fc.w"] = (torch.randn(cfg.classes, feat, generator=g) * feat ** -0.5)
    p["fc.b"] = torch.zeros(cfg.classes)
    return {k: (v.to(dtype) if v.dim() != 4 else v).to(device) for k, v in p.items()}


def synthetic_batch(cfg: ResNetConfig, B: int, seed: int = 1236):
    g = torch.Generator().manual_seed(seed + 1)
    return torch.randn(B, cfg.image, cfg.image, cfg.in_channels, generator=g), torch.randint(0, cfg.classes, (B,), generator=g)



def conv_flops_per_sample(cfg: ResNetConfig) -> float:
    """Forward + data-gradient + weight-gradient FLOPs of the 1x1 / 3x3 convolutions for one image
    (3 x 2 x P x Q x K x R x S x C each; the stem is not counted)."""
    h = cfg.image // 4
    total = 0.0
    for _, convs, down in _arch(cfg):
        hin = h
        for _, c, k, r, s in convs:
            h = (h + 2 * (r // 2) - r) // s + 1
            total += 6.0 * h * h * k * r * r * c
        if down is not None:
            _, c, k, r, s = down
            po = (hin + 2 * (r // 2) - r) // s + 1
            total += 6.0 * po * po * k * r * r * c
    return total

def _meta(shape, dtype):
    return torch.empty(tuple(shape), dtype=dtype, device="meta")


def conv_modules(geo, dtype=torch.float16):
    """The three fused nodes of one convolution geometry (N, H, W, C, K, R, stride) as
    {"fprop" | "dgrad" | "wgrad": (module, meta inputs)}: forward with the batch-norm statistics in
    the epilogue, data gradient, weight gradient."""
    B, H, W, C, K, R, s = geo
    pad = R // 2
    P = (H + 2 * pad - R) // s + 1
    rf = 1.0 / (B * P * P)

    class Fprop(torch.nn.Module):            # y = conv(x, w); E[y], E[y^2] per channel in the epilogue
        def forward(self, x, w):
            y = convolution_forward_channel_last(x, w, [s, s], [pad, pad], [1, 1], False, [0, 0], 1)
            d = aten.mul(y, rf)
            return (y, aten.sum(d, [0, 1, 2], True, dtype=torch.float32),
                    aten.sum(aten.mul(d, y), [0, 1, 2], True, dtype=torch.float32))

    class Dgrad(torch.nn.Module):
        def forward(self, dy, x, w):
            return convolution_backward_data_channel_last(dy, x, w, [s, s], [pad, pad], [1, 1], False, [0, 0], 1)

    class Wgrad(torch.nn.Module):
        def forward(self, dy, x, w):
            return convolution_backward_weight_channel_last(dy, x, w, [s, s], [pad, pad], [1, 1], False, [0, 0], 1)
    class FpropPlain(torch.nn.Module):
        def forward(self, x, w):
            return convolution_forward_channel_last(x, w, [s, s], [pad, pad], [1, 1], False, [0, 0], 1)
    x, w, dy = _meta((B, H, W, C), dtype), _meta((K, R, R, C), dtype), _meta((B, P, P, K), dtype)
    return {"fprop": (Fprop(), [x, w]), "dgrad": (Dgrad(), [dy, x, w]), "wgrad": (Wgrad(), [dy, x, w]),
            "fprop_plain": (FpropPlain(), [x, w])}


def stats_key(geo, dtype=torch.float16) -> str:
    """Key of the tuned table's entry that says where a convolution's batch-norm statistics are taken."""
    return "bn_stats|" + "x".join(map(str, geo)) + "|" + str(dtype).replace("torch.", "")


def separate_stats(geo, dtype=torch.float16) -> bool:
    """True where the measured table says that a plain-store convolution followed by a statistics pass
    over its output (ops.batch_norm_stat) beats the statistics in the epilogue: 1x1 convolutions from few
    to many channels, whose fused epilogue (two column reductions per 32 x 32 chunk) costs more than
    reading the output once more."""
    e = tuning.lookup_config(stats_key(geo, dtype))
    return bool(e and e.get("separate"))


def stem_modules(win: "ops.StemWindow", dtype=torch.float16):
    """The stem convolution on its window view (ops.StemWindow) as fused nodes:
    {"fprop": forward with batch-norm statistics, "wgrad": gradient of the window filter}."""
    sh = win.stride
    rf = 1.0 / (win.N * win.P * win.Q)

    class Fprop(torch.nn.Module):
        def forward(self, xv, wv):
            y = convolution_forward_channel_last(xv, wv, sh, [0, 0], [1, 1], False, [0, 0], 1)
            d = aten.mul(y, rf)
            return (y, aten.sum(d, [0, 1, 2], True, dtype=torch.float32),
                    aten.sum(aten.mul(d, y), [0, 1, 2], True, dtype=torch.float32))

    class Wgrad(torch.nn.Module):
        def forward(self, dy, xv, wv):
            return convolution_backward_weight_channel_last(dy, xv, wv, sh, [0, 0], [1, 1], False, [0, 0], 1)
    xv, wv = win.meta_image(dtype), _meta(win.filter_shape, dtype)
    dy = _meta((win.N, win.P, win.Q, win.K), dtype)
    return {"fprop": (Fprop(), [xv, wv]), "wgrad": (Wgrad(), [dy, xv, wv])}


def geometries(cfg: ResNetConfig, B: int):
    """Distinct (N, H, W, C, K, R, stride) of the fused convolutions of a step, in network order."""
    h = cfg.image // 4
    out = []
    for _, convs, down in _arch(cfg):
        hin = h
        for _, c, k, r, s in convs:
            out.append((B, h, h, c, k, r, s))
            h = (h + 2 * (r // 2) - r) // s + 1
        if down is not None:
            _, c, k, r, s = down
            out.append((B, hin, hin, c, k, r, s))
    return list(dict.fromkeys(out))


class ResNetStep:
    """`step(params, images_nhwc, labels)` -> (loss, grads).  All fused convolution nodes are built
    (and their kernels compiled) at construction, keyed by geometry and shared between layers."""

    def __init__(self, cfg: ResNetConfig, B: int, dtype=torch.float16, stem_wgrad: str = "library"):
        """stem_wgrad: "fused" runs the stem's filter gradient on the window view like its forward pass;
        "library" (default) calls the reference's leaf, which at 3 input channels is the faster of the
        two (measured at batch 128: 483 us against 684 us -- each 64-position block of the window view
        costs the fused kernel 16 KB of L2 traffic for a quarter-used 128 x 64 x 64 product)."""
        if stem_wgrad not in ("fused", "library"):
            raise ValueError("stem_wgrad must be 'fused' or 'library'")
        self.stem_wgrad_mode = stem_wgrad
        self.cfg, self.B, self.dtype = cfg, B, dtype
        self.fprop, self.dgrad, self.wgrad = {}, {}, {}
        self.ops: Dict[str, object] = {}
        self.arena = None
        self.split_stats = set()           # geometries whose statistics are a pass of their own
        self.win = ops.StemWindow((B, cfg.image, cfg.image, 3), (cfg.width, 7, 7, 3), [2, 2], [3, 3])
        mods = stem_modules(self.win, dtype)
        self.stem_fprop, self.ops["fprop_stem"] = fuse_module(*mods["fprop"])
        self.stem_wgrad, self.ops["wgrad_stem"] = fuse_module(*mods["wgrad"])
        h = cfg.image // 4                      # after the stride-2 stem and the stride-2 max-pool
        self.plan: List[tuple] = []             # (prefix, [(name, geometry)...], downsample or None)
        for pre, convs, down in _arch(cfg):
            entries = []
            hin = h
            for name, c, k, r, s in convs:
                geo = (B, h, h, c, k, r, s)
                self._build(geo)
                entries.append((name, geo))
                h = (h + 2 * (r // 2) - r) // s + 1
            dgeo = None
            if down is not None:
                name, c, k, r, s = down
                dgeo = (name, (B, hin, hin, c, k, r, s))
                self._build(dgeo[1])
            self.plan.append((pre, entries, dgeo))

    def _build(self, geo):
        if geo in self.fprop:
            return
        tag = "x".join(map(str, geo))
        mods = conv_modules(geo, self.dtype)
        if separate_stats(geo, self.dtype):
            self.split_stats.add(geo)
            mods["fprop"] = mods["fprop_plain"]
        for kind, table in (("fprop", self.fprop), ("dgrad", self.dgrad), ("wgrad", self.wgrad)):
            module, metas = mods[kind]
            table[geo], self.ops[kind + "_" + tag] = fuse_module(module, metas)

    @property
    def conv_flops(self) -> float:
        """FLOPs of the fused convolutions of one step (forward, data and weight gradients)."""
        total = self.ops["fprop_stem"].flops                                     # as executed: 64-wide windows
        if self.stem_wgrad_mode == "fused":
            total += self.ops["wgrad_stem"].flops
        for _, entries, dgeo in self.plan:
            for _, geo in entries + ([dgeo] if dgeo else []):
                tag = "x".join(map(str, geo))
                total += self.ops["fprop_" + tag].flops + self.ops["dgrad_" + tag].flops + self.ops["wgrad_" + tag].flops
        return total

    def check_status(self):
        for op in self.ops.values():
            op.check_status()

    # ---------------------------------------------------------------------------------- pieces
    def _conv_bn(self, p, name, geo, x, relu, residual=None):
        """convolution (statistics in its epilogue) + one normalise / add / ReLU pass"""
        if geo in self.split_stats:
            y = self.fprop[geo](x, p[name + ".w"])
            mean, mean_x2 = ops.batch_norm_stat(y, 1.0 / (y.shape[0] * y.shape[1] * y.shape[2]))
        else:
            y, mean, mean_x2 = self.fprop[geo](x, p[name + ".w"])
        z, m, rstd = ops.bn_apply(y, mean, mean_x2, p[name + ".bn.g"], p[name + ".bn.b"], self.cfg.eps,
                                  residual=residual, relu=relu)
        return y, z, m, rstd

    def _conv_bn_backward(self, p, name, geo, grads, g, x, y, m, rstd, act=None, g2=None, need_dx=True):
        """g (+ g2): gradient w.r.t. the activation after the batch norm (and after its ReLU if `act`
        is that activation).  Returns (masked gradient, data gradient of the convolution)."""
        rf = 1.0 / (y.shape[0] * y.shape[1] * y.shape[2])
        gm, sums = ops.bn_backward_reduce(g, y, m, rstd, act=act, grad2=g2)
        dy, dg, db = ops.bn_backward_apply(gm, y, m, rstd, p[name + ".bn.g"], sums, rf)
        grads[name + ".bn.g"], grads[name + ".bn.b"] = dg, db
        w = p[name + ".w"]
        grads[name + ".w"] = self.wgrad[geo](dy, x, w)
        return gm, (self.dgrad[geo](dy, x, w) if need_dx else None)

    # ---------------------------------------------------------------------------------- step
    def step(self, p: Dict[str, torch.Tensor], images: torch.Tensor, labels: torch.Tensor):
        grads: Dict[str, torch.Tensor] = {}
        for part in self.step_parts(p, images, labels):
            if isinstance(part, tuple):
                grads.update(part[1])
                return part[0], grads
            grads.update(part)

    def step_parts(self, p: Dict[str, torch.Tensor], images: torch.Tensor, labels: torch.Tensor, cuts=()):
        """The step as a generator, for overlapping a data-parallel gradient exchange with the backward
        pass: yields the dict of parameter gradients finished since the last yield each time the backward
        pass has completed a bottleneck block whose index (0 = first block of the network) is in `cuts`,
        and at the end the tuple (loss, remaining gradients)."""
        cfg, dt = self.cfg, self.dtype
        F = torch.nn.functional
        if self.arena is None or self.arena.buf.device != images.device:
            self.arena = ReductionArena(images.device, 1 << 19)
        self.arena.reset()
        with self.arena:
            yield from self._step(p, images, labels, {}, cfg, dt, F, set(cuts))

    def _step(self, p, images, labels, grads, cfg, dt, F, cuts):
        # stem: the 7x7 / 2 convolution on 3 channels as a 7x1 convolution over 64-wide windows of the
        # zero-padded image (statistics in its epilogue), normalise + ReLU, library max-pool
        xv, wv = self.win.image(images, dt), self.win.filter(p["stem.w"])
        y0, mean0, msq0 = self.stem_fprop(xv, wv)
        rf0 = 1.0 / (y0.shape[0] * y0.shape[1] * y0.shape[2])
        a0, m0, r0 = ops.bn_apply(y0, mean0, msq0, p["stem.bn.g"], p["stem.bn.b"], cfg.eps, relu=True)
        x, pool_idx = ops.max_pool2d_with_indices_channel_last(a0, [3, 3], [2, 2], [1, 1])
        saved = []
        for pre, entries, dgeo in self.plan:
            xin = x
            acts = []
            cur = xin
            for j, (name, geo) in enumerate(entries[:2]):
                y, out, m, rstd = self._conv_bn(p, name, geo, cur, relu=True)
                acts.append((cur, y, m, rstd, out))
                cur = out
            if dgeo is not None:
                dy_, identity, dm_, dr_ = self._conv_bn(p, dgeo[0], dgeo[1], xin, relu=False)
                dsave = (dy_, dm_, dr_)
            else:
                identity, dsave = xin, None
            name, geo = entries[2]
            y, x, m, rstd = self._conv_bn(p, name, geo, cur, relu=True, residual=identity)   # ReLU(BN(conv3) + identity)
            acts.append((cur, y, m, rstd, x))
            saved.append((xin, acts, dsave))
        feat = x.float().mean(dim=(1, 2))                                   # average pool
        # classifier + loss (summed over the batch, as the reference's nn.CrossEntropyLoss(reduction="sum"))
        feat_l = feat.detach().requires_grad_(True)
        hw = {k: p[k].detach().float().requires_grad_(True) for k in ("fc.w", "fc.b")}
        with torch.enable_grad():
            loss = F.cross_entropy(F.linear(feat_l, hw["fc.w"], hw["fc.b"]), labels, reduction="sum")
            gfeat, gw, gb = torch.autograd.grad(loss, [feat_l, hw["fc.w"], hw["fc.b"]])
        grads["fc.w"], grads["fc.b"] = gw, gb
        hw_ = x.shape[1] * x.shape[2]
        g = (gfeat / hw_).to(dt).view(x.shape[0], 1, 1, x.shape[3]).expand_as(x).contiguous()
        g2 = None
        # ---------------------------------------------------------------- backward
        for bi, (pre, entries, dgeo), (xin, acts, dsave) in zip(reversed(range(len(self.plan))), reversed(self.plan), reversed(saved)):
            # last convolution: the pass that takes the statistics also adds the two incoming
            # gradients and applies the mask of the ReLU after the residual addition
            name, geo = entries[2]
            cur, y, m, rstd, out = acts[2]
            dsum, d = self._conv_bn_backward(p, name, geo, grads, g, cur, y, m, rstd, act=out, g2=g2)
            for j in (1, 0):
                name, geo = entries[j]
                cur, y, m, rstd, out = acts[j]
                _, d = self._conv_bn_backward(p, name, geo, grads, d, cur, y, m, rstd, act=out)
            if dgeo is not None:
                dy_, dm_, dr_ = dsave
                _, d_id = self._conv_bn_backward(p, dgeo[0], dgeo[1], grads, dsum, xin, dy_, dm_, dr_)
            else:
                d_id = dsum
            g, g2 = d, d_id
            if bi in cuts and bi > 0:
                done, grads = grads, {}
                yield done
        dx = g + g2
        # max-pool, ReLU, batch norm and weight gradient of the stem (no data gradient: images)
        da0 = ops.max_pool2d_with_indices_backward_channel_last(dx, a0, [3, 3], [2, 2], [1, 1], [1, 1], False, pool_idx)
        dz0, sums0 = ops.bn_backward_reduce(da0, y0, m0, r0, act=a0)
        dy0, dg0, db0 = ops.bn_backward_apply(dz0, y0, m0, r0, p["stem.bn.g"], sums0, rf0)
        grads["stem.bn.g"], grads["stem.bn.b"] = dg0, db0
        if self.stem_wgrad_mode == "fused":
            grads["stem.w"] = self.win.unfold(self.stem_wgrad(dy0, xv, wv))
        else:
            grads["stem.w"] = ops.convolution_backward_weight_channel_last(dy0, images.to(dt), p["stem.w"], [2, 2], [3, 3],
                                                                           [1, 1], False, [0, 0], 1)
        yield loss.detach(), grads
