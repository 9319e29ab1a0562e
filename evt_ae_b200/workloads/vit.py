"""ViT training step (forward + backward) expressed as fused nodes.

Model: the reference's ViT (python/model_zoo/vit/vit_modeling.py): linear patch embedding,
class token, learned position embedding, `depth` pre-LayerNorm transformer layers in [S, B, H]
token order (attention with separate q / k / v projections, MLP with erf-GELU), LayerNorm and a
linear classification head on the class token, cross-entropy.  As in the reference the encoder
runs on fused nodes (its partitions are the ones of the BERT step plus a LayerNorm backward that
adds the residual branch's gradient) and the small ends -- patch extraction, the head on B rows,
the loss -- stay in eager PyTorch around it.

Token count: TMA needs row pitches that are multiples of 16 bytes, and the S x S attention
matrices have pitch S.  The reference pads its token count for the same reason (8 class tokens:
256 + 8 = 264, vit_modeling.py:134-137); here 197 tokens (196 patches + class token) are padded to
200 with masked tokens: padded KEYS get -10000 added to their scores (probability 0), padded ROWS
are never read by the head, so every result and gradient equals the unpadded model's.
"""
from __future__ import annotations

import math
import operator
import os
from dataclasses import dataclass
from typing import Dict

import torch

from ..fused_ops import ReductionArena
from ..fuser import fuse_module
from ..ops import colsum

aten = torch.ops.aten


@dataclass
class VitConfig:
    layers: int = 12
    dim: int = 768
    heads: int = 12
    mlp: int = 3072
    image: int = 224
    patch: int = 16
    channels: int = 3
    classes: int = 1000
    eps: float = 1e-5

    @property
    def patches(self) -> int:
        return (self.image // self.patch) ** 2

    @property
    def tokens(self) -> int:
        return self.patches + 1

    @property
    def tokens_padded(self) -> int:
        return (self.tokens + 7) // 8 * 8

    @property
    def patch_dim(self) -> int:
        return self.channels * self.patch * self.patch


VIT_BASE_16 = VitConfig()


def init_params(cfg: VitConfig, seed: int = 1237, dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, M = cfg.dim, cfg.mlp

    def w(*shape, std=0.02):
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

    def gain():
        return torch.ones(D, dtype=dtype, device=device)
    p = {"embed.w": w(D, cfg.patch_dim), "embed.b": w(D), "cls": w(D), "pos": w(cfg.tokens, D)}
    for i in range(cfg.layers):
        for nm in ("q", "k", "v", "o"):
            p[f"l{i}.{nm}.w"], p[f"l{i}.{nm}.b"] = w(D, D), w(D)
        p[f"l{i}.ln1.g"], p[f"l{i}.ln1.b"] = gain(), w(D)
        p[f"l{i}.ff1.w"], p[f"l{i}.ff1.b"] = w(M, D), w(M)
        p[f"l{i}.ff2.w"], p[f"l{i}.ff2.b"] = w(D, M), w(D)
        p[f"l{i}.ln2.g"], p[f"l{i}.ln2.b"] = gain(), w(D)
    p["head.ln.g"], p["head.ln.b"] = gain(), w(D)
    p["head.w"], p["head.b"] = w(cfg.classes, D), w(cfg.classes)
    return p


def synthetic_batch(cfg: VitConfig, B: int, seed: int = 1237):
    g = torch.Generator().manual_seed(seed + 1)
    return torch.randn(B, cfg.channels, cfg.image, cfg.image, generator=g), torch.randint(0, cfg.classes, (B,), generator=g)


def patchify(cfg: VitConfig, images: torch.Tensor) -> torch.Tensor:
    """[B, C, H, W] -> [patches, B, C * p * p], channel-major inside a patch."""
    B, C, H, W = images.shape
    p = cfg.patch
    x = images.reshape(B, C, H // p, p, W // p, p).permute(2, 4, 0, 1, 3, 5)
    return x.reshape(cfg.patches, B, C * p * p)


def _meta(shape, dtype):
    return torch.empty(tuple(shape), dtype=dtype, device="meta")


class _Nodes:
    """All fused nodes of one problem size, compiled once and shared by every layer."""

    def __init__(self, cfg: VitConfig, B: int, dtype: torch.dtype):
        self.cfg, self.B, self.dtype = cfg, B, dtype
        D, MLP, nh, S = cfg.dim, cfg.mlp, cfg.heads, cfg.tokens_padded
        d = D // nh
        T, L, Tp = S * B, B * nh, cfg.patches * B
        eps, dt, f32 = cfg.eps, dtype, torch.float32
        scale = 1.0 / math.sqrt(d)
        self.ops, self.specs = {}, {}

        def make(name, module, *metas):
            gm, op = fuse_module(module, list(metas))
            self.ops[name] = op
            self.specs[name] = (module, list(metas))
            return gm

        class LinBias(torch.nn.Module):
            def forward(self, x, w, b):
                return aten.add(aten.mm(x, aten.permute(w, [1, 0])), b)
        self.lin_dd = make("lin_dd", LinBias(), _meta((T, D), dt), _meta((D, D), dt), _meta((D,), dt))
        self.embed = make("embed", LinBias(), _meta((Tp, cfg.patch_dim), dt), _meta((D, cfg.patch_dim), dt), _meta((D,), dt))

        self.fuse_attention = S <= 512 and os.environ.get("EVT_B200_FUSE_ATTENTION", "1") == "1"

        class ScoresSoftmax(torch.nn.Module):
            def forward(self, q3, k3, ext):
                v = aten.view(aten.bmm(aten.permute(q3, [1, 0, 2]), aten.permute(k3, [1, 2, 0])), [B, nh, S, S])
                sc = aten.add(aten.mul(v, scale), ext)
                return aten.view(aten._softmax(sc, -1, False), [L, S, S])

        class Scores(torch.nn.Module):
            def forward(self, q3, k3, ext):
                v = aten.view(aten.bmm(aten.permute(q3, [1, 0, 2]), aten.permute(k3, [1, 2, 0])), [B, nh, S, S])
                return aten.add(aten.mul(v, scale), ext)

        class Softmax(torch.nn.Module):
            def forward(self, x):
                return aten.view(aten._softmax(x, -1, False), [L, S, S])
        qk = (_meta((S, L, d), dt), _meta((S, L, d), dt), _meta((B, 1, 1, S), dt))
        if self.fuse_attention:
            self.scores_softmax = make("scores_softmax", ScoresSoftmax(), *qk)
        else:
            self.scores = make("scores", Scores(), *qk)
            self.softmax = make("softmax", Softmax(), _meta((B, nh, S, S), dt))

        class Context(torch.nn.Module):
            def forward(self, v3, p):
                pm = aten.permute(aten.bmm(p, aten.permute(v3, [1, 0, 2])), [1, 0, 2])
                return aten.view(aten.clone(pm, memory_format=torch.contiguous_format), [T, D])
        self.context = make("context", Context(), _meta((S, L, d), dt), _meta((L, S, S), dt))

        class LinBiasRes(torch.nn.Module):
            def forward(self, x, w, b, r):
                return aten.add(aten.add(aten.mm(x, aten.permute(w, [1, 0])), b), r)
        self.lin_dd_res = make("lin_dd_res", LinBiasRes(), _meta((T, D), dt), _meta((D, D), dt), _meta((D,), dt), _meta((T, D), dt))
        self.lin_md_res = make("lin_md_res", LinBiasRes(), _meta((T, MLP), dt), _meta((D, MLP), dt), _meta((D,), dt), _meta((T, D), dt))

        class LayerNorm(torch.nn.Module):
            def forward(self, x, g, b):
                ln = aten.native_layer_norm(x, [D], None, None, eps)
                return aten.add(aten.mul(operator.getitem(ln, 0), g), b), operator.getitem(ln, 1), operator.getitem(ln, 2)
        self.layernorm = make("layernorm", LayerNorm(), _meta((T, D), dt), _meta((D,), dt), _meta((D,), dt))

        class LinBiasGelu(torch.nn.Module):      # erf GELU (nn.GELU() of the reference's FeedForward)
            def forward(self, x, w, b):
                f = aten.add(aten.mm(x, aten.permute(w, [1, 0])), b)
                return f, aten.gelu(f)
        self.lin_dm_gelu = make("lin_dm_gelu", LinBiasGelu(), _meta((T, D), dt), _meta((MLP, D), dt), _meta((MLP,), dt))

        # ------------------------------------------------------------------ backward
        class LayerNormBwdAdd(torch.nn.Module):   # dx of LN plus the gradient that by-passed it on the residual branch
            def forward(self, gy, x, mean, rstd, g, b, r):
                ln = aten.native_layer_norm_backward(gy, x, [D], mean, rstd, g, b, [True, False, False])
                return aten.add(operator.getitem(ln, 0), r)
        self.layernorm_bwd_add = make("layernorm_bwd_add", LayerNormBwdAdd(), _meta((T, D), dt), _meta((T, D), dt),
                                      _meta((T, 1), f32), _meta((T, 1), f32), _meta((D,), dt), _meta((D,), dt), _meta((T, D), dt))

        class Wgrad(torch.nn.Module):
            def forward(self, dy, x):
                return aten.mm(aten.permute(dy, [1, 0]), x)
        self.wgrad_dd = make("wgrad_dd", Wgrad(), _meta((T, D), dt), _meta((T, D), dt))
        self.wgrad_dm = make("wgrad_dm", Wgrad(), _meta((T, D), dt), _meta((T, MLP), dt))     # dW2 [D, MLP]
        self.wgrad_md = make("wgrad_md", Wgrad(), _meta((T, MLP), dt), _meta((T, D), dt))     # dW1 [MLP, D]
        self.wgrad_embed = make("wgrad_embed", Wgrad(), _meta((Tp, D), dt), _meta((Tp, cfg.patch_dim), dt))

        class DgradGelu(torch.nn.Module):
            def forward(self, dh, w, f):
                df = aten.gelu_backward(aten.mm(dh, w), f)
                return df, aten.sum(df, [0], dtype=torch.float32)
        self.dgrad_gelu = make("dgrad_gelu", DgradGelu(), _meta((T, D), dt), _meta((D, MLP), dt), _meta((T, MLP), dt))

        class DgradLN(torch.nn.Module):          # dx = dy W ; LayerNorm gamma / beta gradients of the LN that fed this map
            def forward(self, dy, w, xin, mean, rstd):
                dx = aten.mm(dy, w)
                xhat = aten.mul(aten.sub(xin, mean), rstd)
                return dx, aten.sum(dx, [0], dtype=torch.float32), aten.sum(aten.mul(dx, xhat), [0], dtype=torch.float32)
        self.dgrad_m_ln = make("dgrad_m_ln", DgradLN(), _meta((T, MLP), dt), _meta((MLP, D), dt), _meta((T, D), dt),
                               _meta((T, 1), f32), _meta((T, 1), f32))

        class DgradResLN(torch.nn.Module):
            def forward(self, dy, w, r, xin, mean, rstd):
                dx = aten.add(aten.mm(dy, w), r)
                xhat = aten.mul(aten.sub(xin, mean), rstd)
                return dx, aten.sum(dx, [0], dtype=torch.float32), aten.sum(aten.mul(dx, xhat), [0], dtype=torch.float32)
        self.dgrad_d_res_ln = make("dgrad_d_res_ln", DgradResLN(), _meta((T, D), dt), _meta((D, D), dt), _meta((T, D), dt),
                                   _meta((T, D), dt), _meta((T, 1), f32), _meta((T, 1), f32))

        class Dgrad(torch.nn.Module):
            def forward(self, dy, w):
                return aten.mm(dy, w)
        self.dgrad_dd = make("dgrad_dd", Dgrad(), _meta((T, D), dt), _meta((D, D), dt))

        class DgradRes(torch.nn.Module):
            def forward(self, dy, w, r):
                return aten.add(aten.mm(dy, w), r)
        self.dgrad_dd_res = make("dgrad_dd_res", DgradRes(), _meta((T, D), dt), _meta((D, D), dt), _meta((T, D), dt))

        class BmmTN(torch.nn.Module):
            def forward(self, p, x3):
                bmm = aten.bmm(aten.permute(p, [0, 2, 1]), aten.permute(x3, [1, 0, 2]))
                c = aten.clone(aten.permute(bmm, [1, 0, 2]), memory_format=torch.contiguous_format)
                v = aten.view(c, [S, B, D])
                return aten.view(v, [T, D]), aten.sum(v, [0, 1], dtype=torch.float32)
        self.bmm_tn = make("bmm_tn", BmmTN(), _meta((L, S, S), dt), _meta((S, L, d), dt))

        class BmmNN(torch.nn.Module):
            def forward(self, p, x3):
                bmm = aten.bmm(p, aten.permute(x3, [1, 0, 2]))
                c = aten.clone(aten.permute(bmm, [1, 0, 2]), memory_format=torch.contiguous_format)
                v = aten.view(c, [S, B, D])
                return aten.view(v, [T, D]), aten.sum(v, [0, 1], dtype=torch.float32)
        self.bmm_nn = make("bmm_nn", BmmNN(), _meta((L, S, S), dt), _meta((S, L, d), dt))

        class DProbsSoftmaxBwd(torch.nn.Module):
            dt_ = dt

            def forward(self, dc3, v3, y):
                dp = aten.bmm(aten.permute(dc3, [1, 0, 2]), aten.permute(v3, [1, 2, 0]))
                return aten.mul(aten._softmax_backward_data(dp, y, -1, self.dt_), scale)

        class DProbs(torch.nn.Module):
            def forward(self, dc3, v3):
                return aten.bmm(aten.permute(dc3, [1, 0, 2]), aten.permute(v3, [1, 2, 0]))

        class SoftmaxBwd(torch.nn.Module):
            dt_ = dt

            def forward(self, g, y):
                return aten.mul(aten._softmax_backward_data(g, y, -1, self.dt_), scale)
        if self.fuse_attention:
            self.dprobs_softmax_bwd = make("dprobs_softmax_bwd", DProbsSoftmaxBwd(), _meta((S, L, d), dt), _meta((S, L, d), dt),
                                           _meta((L, S, S), dt))
        else:
            self.dprobs = make("dprobs", DProbs(), _meta((S, L, d), dt), _meta((S, L, d), dt))
            self.softmax_bwd = make("softmax_bwd", SoftmaxBwd(), _meta((L, S, S), dt), _meta((L, S, S), dt))


class VitStep:
    """`step(params, tokens0, labels)` -> (loss, grads, dtokens0).

    `tokens0`: the encoder input [S_padded, B, D] (patch embeddings + class token + positions, padded
    rows zero) -- `embed_tokens` builds it from images with a fused GEMM; `head` is the eager
    LayerNorm + linear + cross-entropy on the class-token rows."""

    def __init__(self, cfg: VitConfig, B: int, dtype=torch.bfloat16):
        self.cfg, self.B, self.dtype = cfg, B, dtype
        self.n = _Nodes(cfg, B, dtype)
        self._arena = None

    def check_status(self):
        for op in self.n.ops.values():
            op.check_status()

    @property
    def gemm_flops(self) -> float:
        n, Lr = self.n.ops, self.cfg.layers
        per_layer = [("lin_dd", 3), ("context", 1), ("lin_dd_res", 1), ("lin_dm_gelu", 1), ("lin_md_res", 1), ("wgrad_dm", 1),
                     ("dgrad_gelu", 1), ("wgrad_md", 1), ("dgrad_m_ln", 1), ("wgrad_dd", 4), ("dgrad_dd", 2), ("bmm_tn", 2),
                     ("bmm_nn", 1), ("dgrad_dd_res", 1), ("dgrad_d_res_ln", 1)]
        per_layer += [("scores_softmax", 1), ("dprobs_softmax_bwd", 1)] if self.n.fuse_attention else [("scores", 1), ("dprobs", 1)]
        total = sum(n[k].flops * c for k, c in per_layer) * Lr
        return total + n["embed"].flops + n["wgrad_embed"].flops

    # ----------------------------------------------------------------------------------
    def embed_tokens(self, p, images):
        """images [B, C, H, W] -> (tokens0 [S_padded, B, D], patch matrix kept for the weight gradient)"""
        cfg, B = self.cfg, self.B
        pm = patchify(cfg, images).reshape(cfg.patches * B, cfg.patch_dim).to(self.dtype)
        e = self.n.embed(pm, p["embed.w"], p["embed.b"]).view(cfg.patches, B, cfg.dim)
        tok = torch.zeros(cfg.tokens_padded, B, cfg.dim, dtype=self.dtype, device=images.device)
        tok[0] = p["cls"] + p["pos"][0]
        tok[1:cfg.tokens] = e + p["pos"][1:].unsqueeze(1)
        return tok, pm

    def embed_backward(self, dtok, pm):
        """gradients of the embedding parameters from dtokens0"""
        cfg, B = self.cfg, self.B
        de = dtok[1:cfg.tokens].reshape(cfg.patches * B, cfg.dim).contiguous()
        g = {"embed.w": self.n.wgrad_embed(de, pm), "embed.b": colsum(de, torch.float32),
             "cls": dtok[0].float().sum(0), "pos": dtok[:cfg.tokens].float().sum(1)}
        return g

    def head(self, p, x_final, labels):
        """LayerNorm + linear + cross-entropy on the class token, eager autograd (B rows).
        Returns (loss, head gradients, d x_final)."""
        cfg = self.cfg
        cls = x_final[0].detach().float().requires_grad_(True)
        hp = {k: p[k].detach().float().requires_grad_(True) for k in ("head.ln.g", "head.ln.b", "head.w", "head.b")}
        F = torch.nn.functional
        with torch.enable_grad():
            z = F.linear(F.layer_norm(cls, (cfg.dim,), hp["head.ln.g"], hp["head.ln.b"], cfg.eps), hp["head.w"], hp["head.b"])
            loss = F.cross_entropy(z, labels)
            grads = torch.autograd.grad(loss, [cls] + list(hp.values()))
        dx = torch.zeros_like(x_final)
        dx[0] = grads[0].to(x_final.dtype)
        return loss.detach(), dict(zip(hp.keys(), grads[1:])), dx

    def step(self, p: Dict[str, torch.Tensor], tokens0: torch.Tensor, labels: torch.Tensor):
        grads: Dict[str, torch.Tensor] = {}
        for part in self.step_parts(p, tokens0, labels):
            if isinstance(part, tuple):
                loss, rest, dx = part
                grads.update(rest)
                return loss, grads, dx
            grads.update(part)

    def step_parts(self, p: Dict[str, torch.Tensor], tokens0: torch.Tensor, labels: torch.Tensor, cuts=()):
        """The step as a generator, for overlapping a data-parallel gradient exchange with the backward
        pass: yields the dict of parameter gradients finished since the last yield each time the backward
        pass has completed a layer listed in `cuts`, and at the end the tuple (loss, remaining gradients,
        dx of the tokens)."""
        cuts = set(cuts)
        cfg, n, B = self.cfg, self.n, self.B
        S, D, nh = cfg.tokens_padded, cfg.dim, cfg.heads
        d = D // nh
        T, L = S * B, B * nh
        dt = self.dtype
        if self._arena is None or self._arena.buf.device != tokens0.device:
            self._arena = ReductionArena(tokens0.device)
        self._arena.reset()
        grads: Dict[str, torch.Tensor] = {}
        # padded key positions never receive probability
        ext = torch.zeros(B, 1, 1, S, dtype=dt, device=tokens0.device)
        ext[..., cfg.tokens:] = -10000.0
        with self._arena:
            x = tokens0.reshape(T, D)
            saved = []
            for i in range(cfg.layers):
                pre = f"l{i}."
                n1, m1, r1 = n.layernorm(x, p[pre + "ln1.g"], p[pre + "ln1.b"])
                q3 = n.lin_dd(n1, p[pre + "q.w"], p[pre + "q.b"]).view(S, L, d)
                k3 = n.lin_dd(n1, p[pre + "k.w"], p[pre + "k.b"]).view(S, L, d)
                v3 = n.lin_dd(n1, p[pre + "v.w"], p[pre + "v.b"]).view(S, L, d)
                pr = n.scores_softmax(q3, k3, ext) if n.fuse_attention else n.softmax(n.scores(q3, k3, ext))
                ctx = n.context(v3, pr)
                xa = n.lin_dd_res(ctx, p[pre + "o.w"], p[pre + "o.b"], x)
                n2, m2, r2 = n.layernorm(xa, p[pre + "ln2.g"], p[pre + "ln2.b"])
                f, g = n.lin_dm_gelu(n2, p[pre + "ff1.w"], p[pre + "ff1.b"])
                xo = n.lin_md_res(g, p[pre + "ff2.w"], p[pre + "ff2.b"], xa)
                saved.append((x, n1, m1, r1, q3, k3, v3, pr, ctx, xa, n2, m2, r2, f, g))
                x = xo
            loss, hgrads, dx3 = self.head(p, x.view(S, B, D), labels)
            grads.update(hgrads)
            dx = dx3.reshape(T, D)
            for i in reversed(range(cfg.layers)):
                pre = f"l{i}."
                (xin, n1, m1, r1, q3, k3, v3, pr, ctx, xa, n2, m2, r2, f, g) = saved[i]
                # MLP: xo = g W2^T + b2 + xa
                grads[pre + "ff2.b"] = colsum(dx, torch.float32)
                grads[pre + "ff2.w"] = n.wgrad_dm(dx, g)
                df, db1 = n.dgrad_gelu(dx, p[pre + "ff2.w"], f)
                grads[pre + "ff1.b"] = db1
                grads[pre + "ff1.w"] = n.wgrad_md(df, n2)
                dn2, db_ln2, dg_ln2 = n.dgrad_m_ln(df, p[pre + "ff1.w"], xa, m2, r2)
                grads[pre + "ln2.b"], grads[pre + "ln2.g"] = db_ln2, dg_ln2
                dxa = n.layernorm_bwd_add(dn2, xa, m2, r2, p[pre + "ln2.g"], p[pre + "ln2.b"], dx)
                # attention: xa = ctx Wo^T + bo + xin
                grads[pre + "o.b"] = colsum(dxa, torch.float32)
                grads[pre + "o.w"] = n.wgrad_dd(dxa, ctx)
                dc3 = n.dgrad_dd(dxa, p[pre + "o.w"]).view(S, L, d)
                dv, dbv = n.bmm_tn(pr, dc3)
                dS = n.dprobs_softmax_bwd(dc3, v3, pr) if n.fuse_attention else n.softmax_bwd(n.dprobs(dc3, v3), pr)
                dq, dbq = n.bmm_nn(dS, k3)
                dk, dbk = n.bmm_tn(dS, q3)
                grads[pre + "q.b"], grads[pre + "k.b"], grads[pre + "v.b"] = dbq, dbk, dbv
                grads[pre + "q.w"] = n.wgrad_dd(dq, n1)
                grads[pre + "k.w"] = n.wgrad_dd(dk, n1)
                grads[pre + "v.w"] = n.wgrad_dd(dv, n1)
                t1 = n.dgrad_dd(dq, p[pre + "q.w"])
                t2 = n.dgrad_dd_res(dk, p[pre + "k.w"], t1)
                dn1, db_ln1, dg_ln1 = n.dgrad_d_res_ln(dv, p[pre + "v.w"], t2, xin, m1, r1)
                grads[pre + "ln1.b"], grads[pre + "ln1.g"] = db_ln1, dg_ln1
                dx = n.layernorm_bwd_add(dn1, xin, m1, r1, p[pre + "ln1.g"], p[pre + "ln1.b"], dxa)
                if i in cuts and i > 0:
                    done, grads = grads, {}
                    yield done
            yield loss, grads, dx.view(S, B, D)
