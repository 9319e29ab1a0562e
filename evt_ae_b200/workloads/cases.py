"""Fused-node test cases: tiny modules written in raw aten calls, one heavy op plus its
epilogue each.  Graph structures and full-size shapes follow the reference's fused-node
unit tests (unittest/evt_fuser/mm.py:30-236, bmm.py:29-94) and BASELINE configuration 0;
every case is parametrised so the same structure also runs at sizes a CPU checks in
seconds.  Inputs are seeded (numpy PCG64) so the CPU oracle and the GPU see the same bits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Sequence

import numpy as np
import torch

aten = torch.ops.aten


def seeded(shape, seed, scale=1.0, dtype=torch.float16):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal(size=tuple(shape), dtype=np.float32) * scale
    return torch.from_numpy(a).to(dtype)


@dataclass
class Case:
    name: str
    module: torch.nn.Module
    inputs: List[torch.Tensor]
    kind: str = "gemm"


# ----------------------------------------------------------------------------- GEMM cases

def mm_bias_gelu(M, N, K, s0, s1, dtype=torch.float16, approximate="tanh"):
    """x @ W^T + b, pre-activation and GELU both stored (FFN1; mm.py:30-50)."""
    class Mod(torch.nn.Module):
        def forward(self, w, x, b):
            wt = aten.permute(w, [1, 0])
            mm = aten.mm(x, wt)
            add = aten.add(mm, b)
            v = aten.view(add, [s0, s1, N])
            g = aten.gelu(v, approximate=approximate)
            v2 = aten.view(g, [M, N])
            return v2, v
    assert s0 * s1 == M
    return Case(f"mm_bias_gelu_{M}x{N}x{K}_{approximate}", Mod(),
                [seeded((N, K), 1, 0.05, dtype), seeded((M, K), 2, 1.0, dtype), seeded((N,), 3, 1.0, dtype)])


def mm_bias_tanh(M, N, K, dtype=torch.float16):
    """pooler: tanh(x @ W^T + b) (mm.py:52-69), M may be tiny."""
    class Mod(torch.nn.Module):
        def forward(self, x, w, b):
            wt = aten.permute(w, [1, 0])
            mm = aten.mm(x, wt)
            add = aten.add(mm, b)
            t = aten.tanh(add)
            return aten.add(t, b)
    return Case(f"mm_bias_tanh_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 4, 1.0, dtype), seeded((N, K), 5, 0.018, dtype), seeded((N,), 6, 0.018, dtype)])


def mm_bias_tanh_only(M, N, K, dtype=torch.float16):
    """pooler activation: tanh(x @ W^T + b), M = 4 in the reference (mm.py:52-70)."""
    class Mod(torch.nn.Module):
        def forward(self, x, w, b):
            wt = aten.permute(w, [1, 0])
            return aten.tanh(aten.add(aten.mm(x, wt), b))
    return Case(f"mm_bias_tanh_only_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 4, 1.0, dtype), seeded((N, K), 5, 0.018, dtype), seeded((N,), 6, 0.018, dtype)])


def mm_bias_tiny_view(M, N, K, dtype=torch.float16):
    """next-sentence head: a 2 x 2 result, bias added, viewed (mm.py:93-111)."""
    class Mod(torch.nn.Module):
        def forward(self, x, w, b):
            wt = aten.permute(w, [1, 0])
            return aten.view(aten.add(aten.mm(x, wt), b), [M, N])
    return Case(f"mm_bias_tiny_view_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 7, 1.0, dtype), seeded((N, K), 8, 1.0, dtype), seeded((N,), 9, 1.0, dtype)])


def mm_bias_dropout_residual(M, N, K, s0, s1, p=0.7, dtype=torch.float16):
    """x W^T + b, dropout, residual add; outputs the sum and the keep mask.  The reference writes
    `aten.native_dropout` (unittest/evt_fuser/dropout.py:33-52) and its decomposition pass turns
    it into rand_like / ge / mul / mul (pass_decomposition.py:350-379), which is the form the
    fuser sees and what is written here."""
    class Mod(torch.nn.Module):
        def forward(self, x, w, b, r):
            wt = aten.permute(w, [1, 0])
            v = aten.view(aten.add(aten.mm(x, wt), b), [s0, s1, N])
            keep = aten.ge(torch.rand_like(v), p)
            d = aten.mul(aten.mul(v, keep), 1.0 / (1.0 - p))
            return aten.add(d, r), keep
    assert s0 * s1 == M
    return Case(f"mm_bias_dropout_residual_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 28, 1.0, dtype), seeded((N, K), 29, 1.0, dtype), seeded((N,), 30, 1.0, dtype),
                 seeded((s0, s1, N), 31, 1.0, dtype)])


def mm_bias_view3(M, N, K, s0, s1, h, dtype=torch.float16):
    """QKV projection: bias added on a 3-D view, result viewed per head (mm.py:71-89)."""
    class Mod(torch.nn.Module):
        def forward(self, x, w, b):
            wt = aten.permute(w, [1, 0])
            mm = aten.mm(x, wt)
            v = aten.view(mm, [s0, s1, N])
            add = aten.add(v, b)
            return aten.view(add, [s0, s1 * h, N // h])
    return Case(f"mm_bias_view3_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 7, 1.0, dtype), seeded((N, K), 8, 0.05, dtype), seeded((N,), 9, 1.0, dtype)])


def mm_tanh_backward_sum(M, N, K, dtype=torch.float16):
    """dgrad with tanh backward and a bias-gradient reduction (mm.py:110-124)."""
    class Mod(torch.nn.Module):
        def forward(self, a, b, t):
            mm = aten.mm(a, b)
            out = aten.tanh_backward(mm, t)
            s = aten.sum(out, [0], True)
            return out, s
    return Case(f"mm_tanh_backward_sum_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 10, 1.0, dtype), seeded((K, N), 11, 0.1, dtype),
                 torch.tanh(seeded((M, N), 12, 1.0, torch.float32)).to(dtype)])


def mm_residual_permute(M, N, K, s0, s1, dtype=torch.float16):
    """two residual adds on a 3-D view and a permuted store (mm.py:126-146)."""
    class Mod(torch.nn.Module):
        def forward(self, a, b, r0, r1):
            mm = aten.mm(a, b)
            v = aten.view(mm, [s0, s1, N])
            x = aten.add(v, r0)
            y = aten.add(x, r1)
            return aten.permute(y, [1, 0, 2])
    return Case(f"mm_residual_permute_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 13, 1.0, dtype), seeded((K, N), 14, 0.05, dtype),
                 seeded((s0, s1, N), 15, 1.0, dtype), seeded((s0, s1, N), 16, 1.0, dtype)])


def mm_multi_store(M, N, K, s0, s1, dtype=torch.float16):
    """every intermediate escapes: four stores of one accumulator (mm.py:148-168)."""
    class Mod(torch.nn.Module):
        def forward(self, a, b, r0, r1):
            mm = aten.mm(a, b)
            v = aten.view(mm, [s0, s1, N])
            x = aten.add(v, r0)
            y = aten.add(x, r1)
            z = aten.view(y, [M, N])
            return v, x, y, z
    return Case(f"mm_multi_store_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 17, 1.0, dtype), seeded((K, N), 18, 0.05, dtype),
                 seeded((s0, s1, N), 19, 1.0, dtype), seeded((s0, s1, N), 20, 1.0, dtype)])


def mm_colsum(M, N, K, dtype=torch.float16):
    """plain GEMM whose column sums ride in the epilogue (mm.py:188-200)."""
    class Mod(torch.nn.Module):
        def forward(self, a, b):
            mm = aten.mm(a, b)
            s = aten.sum(mm, [0], True)
            return mm, s
    return Case(f"mm_colsum_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 21, 1.0, dtype), seeded((K, N), 22, 0.05, dtype)])


def mm_wgrad(M, N, K, dtype=torch.float16):
    """weight gradient: A^T (stored [K, M]) times B, no epilogue (mm.py:202-214)."""
    class Mod(torch.nn.Module):
        def forward(self, a, b):
            at = aten.permute(a, [1, 0])
            return aten.mm(at, b)
    return Case(f"mm_wgrad_{M}x{N}x{K}", Mod(),
                [seeded((K, M), 23, 1.0, dtype), seeded((K, N), 24, 0.05, dtype)])


def mm_relu_dropout(M, N, K, p=0.1, dtype=torch.float16):
    """bias + ReLU + mask outputs + fused dropout (mm.py:216-236).  The random mask is an
    output and is checked by reuse, as the reference's dropout test does
    (unittest/evt_fuser/dropout.py:63-75)."""
    class Mod(torch.nn.Module):
        def forward(self, w, x, b):
            wt = aten.permute(w, [1, 0])
            mm = aten.mm(x, wt)
            add = aten.add(mm, b)
            relu = aten.relu(add)
            ne = aten.ne(relu, 0)
            rnd = torch.rand_like(relu)
            ge = aten.ge(rnd, p)
            m1 = aten.mul(relu, ge)
            m2 = aten.mul(m1, 1.0 / (1.0 - p))
            return ne, ge, m2
    return Case(f"mm_relu_dropout_{M}x{N}x{K}", Mod(),
                [seeded((N, K), 25, 0.05, dtype), seeded((M, K), 26, 1.0, dtype), seeded((N,), 27, 1.0, dtype)])


def config0(M=16384, N=4096, K=1024, dtype=torch.float16):
    """BASELINE configuration 0: D = GELU(A@B + bias) + C, colsum(D), rowmax(D)."""
    class Mod(torch.nn.Module):
        def forward(self, a, b, bias, c):
            mm = aten.mm(a, b)
            add = aten.add(mm, bias)
            g = aten.gelu(add)
            d = aten.add(g, c)
            colsum = aten.sum(d, [0])
            rowmax = aten.amax(d, [1])
            return d, colsum, rowmax
    return Case(f"config0_{M}x{N}x{K}", Mod(),
                [seeded((M, K), 1234, 1.0, dtype), seeded((K, N), 1235, 0.02, dtype),
                 seeded((N,), 1236, 0.02, dtype), seeded((M, N), 1237, 1.0, dtype)])


def mm_plain(M, N, K, a_t=False, b_t=False, dtype=torch.float16):
    """plain GEMM in each operand layout (R_R, R_C, C_R, C_C of the tuner keys)."""
    class Mod(torch.nn.Module):
        def forward(self, a, b):
            if a_t:
                a = aten.permute(a, [1, 0])
            if b_t:
                b = aten.permute(b, [1, 0])
            return aten.mm(a, b)
    a = seeded((K, M) if a_t else (M, K), 31, 1.0, dtype)
    b = seeded((N, K) if b_t else (K, N), 32, 0.05, dtype)
    return Case(f"mm_plain_{M}x{N}x{K}_{'C' if a_t else 'R'}{'C' if b_t else 'R'}_{str(dtype)[6:]}", Mod(), [a, b])


# ----------------------------------------------------------------------------- BMM cases

def bmm_context_permuted_store(S, B, H, D, dtype=torch.float16):
    """probs @ V with V read through a permute and the result stored as [S, B, H*D]
    (bmm.py:29-46)."""
    L = B * H
    class Mod(torch.nn.Module):
        def forward(self, v, p):
            vt = aten.permute(v, [1, 0, 2])
            bmm = aten.bmm(p, vt)
            pm = aten.permute(bmm, [1, 0, 2])
            c = aten.clone(pm, memory_format=torch.contiguous_format)
            v8 = aten.view(c, [S, B, H * D])
            return aten.view(v8, [S * B, H * D])
    return Case(f"bmm_context_{S}_{B}_{H}_{D}", Mod(),
                [seeded((S, L, D), 41, 1.0, dtype), seeded((L, S, S), 42, 0.05, dtype)], kind="bmm")


def bmm_dgrad_sum(S, B, H, D, dtype=torch.float16):
    """backward bmm with a [1,1,H*D] reduction (bmm.py:48-67)."""
    L = B * H
    class Mod(torch.nn.Module):
        def forward(self, q, g):
            qt = aten.permute(q, [1, 2, 0])
            bmm = aten.bmm(qt, g)
            pm = aten.permute(bmm, [2, 0, 1])
            v = aten.view(pm, [S, B, H * D])
            s = aten.sum(v, [0, 1], True)
            c = aten.clone(v, memory_format=torch.contiguous_format)
            out = aten.view(c, [S * B, H * D])
            return out, aten.div(s, 20)     # the division consumes a finished reduction: stays outside
    return Case(f"bmm_dgrad_sum_{S}_{B}_{H}_{D}", Mod(),
                [seeded((S, L, D), 43, 1.0, dtype), seeded((L, S, S), 44, 0.05, dtype)], kind="bmm")


def bmm_scores_mask(S, B, H, D, dtype=torch.float16):
    """Q K^T * scale + mask, mask algebra on the side (bmm.py:69-94)."""
    L = B * H
    class Mod(torch.nn.Module):
        def forward(self, q, k, mask, c0, c1, c2):
            u = aten.unsqueeze(mask, 1)
            u1 = aten.unsqueeze(u, 2)
            m40 = aten.mul(u1, -1.0)
            a37 = aten.add(m40, c0)
            m1 = aten.mul(a37, c1)
            qp = aten.permute(q, [1, 0, 2])
            kp = aten.permute(k, [1, 2, 0])
            bmm = aten.bmm(qp, kp)
            v = aten.view(bmm, [B, H, S, S])
            mul = aten.mul(v, c2)
            add = aten.add(mul, m1)
            return add, m1
    return Case(f"bmm_scores_{S}_{B}_{H}_{D}", Mod(),
                [seeded((S, L, D), 45, 1.0, dtype), seeded((S, L, D), 46, 1.0, dtype),
                 seeded((B, S), 47, 1.0, dtype), seeded((1,), 48, 1.0, dtype), seeded((1,), 49, 1.0, dtype),
                 seeded((1,), 50, 0.2, dtype)], kind="bmm")


def small_gemm_cases(dtype=torch.float16) -> List[Case]:
    """Sizes a CPU finishes in well under a second each; cover ragged M/N/K and tiny dims."""
    return [
        mm_plain(128, 256, 64, False, True, dtype),
        mm_plain(128, 256, 64, False, False, dtype),
        mm_plain(128, 256, 64, True, False, dtype),
        mm_plain(128, 256, 64, True, True, dtype),
        mm_plain(200, 136, 72, False, True, dtype),
        mm_plain(200, 136, 72, False, False, dtype),
        mm_plain(200, 136, 72, True, False, dtype),
        mm_plain(392, 520, 264, True, True, dtype),
        mm_plain(1000, 1032, 520, False, True, dtype),
        mm_bias_gelu(1024, 512, 256, 512, 2, dtype, "tanh"),
        mm_bias_gelu(256, 384, 128, 128, 2, dtype, "none"),
        mm_bias_tanh(4, 1024, 1024, dtype),
        mm_bias_view3(1024, 256, 128, 512, 2, 4, dtype),
        mm_tanh_backward_sum(4, 1024, 8, dtype),
        mm_tanh_backward_sum(300, 200, 64, dtype),
        mm_residual_permute(2048, 256, 128, 512, 4, dtype),
        mm_multi_store(512, 128, 64, 128, 4, dtype),
        mm_colsum(1024, 512, 128, dtype),
        mm_wgrad(256, 192, 1024, dtype),
        config0(512, 384, 128, dtype),
    ]


def small_bmm_cases(dtype=torch.float16) -> List[Case]:
    return [
        bmm_context_permuted_store(128, 2, 4, 64, dtype),
        bmm_dgrad_sum(128, 2, 4, 64, dtype),
        bmm_scores_mask(128, 2, 4, 64, dtype),
    ]


# ------------------------------------------------------------------ reduce-apply cases
import operator


def softmax_plain(rows, cols, dtype=torch.float16, shape=None):
    """softmax over the last dim with a reshaped store (softmax.py:30-41)."""
    shape = shape or (rows, cols)
    class Mod(torch.nn.Module):
        def forward(self, x):
            s = aten._softmax(x, -1, False)
            return aten.view(s, [rows, cols])
    return Case(f"softmax_{'x'.join(map(str, shape))}_{str(dtype)[6:]}", Mod(), [seeded(shape, 61, 2.0, dtype)], kind="softmax")


def softmax_aux_row_col(rows, cols, dtype=torch.float16):
    """full-tensor, [cols] and [rows,1] operands in the epilogue (softmax.py:43-110)."""
    class Mod(torch.nn.Module):
        def forward(self, x, aux, row, col):
            s = aten._softmax(x, -1, False)
            a = aten.add(s, aux)
            b = aten.add(a, row)
            c = aten.add(b, col)
            return aten.mul(c, 2.0)
    return Case(f"softmax_aux_row_col_{rows}x{cols}", Mod(),
                [seeded((rows, cols), 62, 2.0, dtype), seeded((rows, cols), 63, 1.0, dtype),
                 seeded((cols,), 64, 1.0, dtype), seeded((rows, 1), 65, 1.0, dtype)], kind="softmax")


def softmax_epilogue_form(form, rows, cols, dtype=torch.float16):
    """The single-operand epilogue forms of the reference's softmax tests (softmax.py:43-110):
    `aux` full tensor added, `row` a [cols] vector added, `scalar` times two, `colreduce` times
    two plus the sum over rows, `col` a [rows, 1] vector added."""
    class Aux(torch.nn.Module):
        def forward(self, x, aux):
            return aten.add(aten._softmax(x, -1, False), aux)

    class Scalar(torch.nn.Module):
        def forward(self, x):
            return aten.mul(aten._softmax(x, -1, False), 2.)

    class ColReduce(torch.nn.Module):
        def forward(self, x):
            out = aten.mul(aten._softmax(x, -1, False), 2.)
            return out, aten.sum(out, [0], True)
    x = seeded((rows, cols), 67, 1.0, dtype)
    name = f"softmax_{form}_{rows}x{cols}"
    if form == "aux":
        return Case(name, Aux(), [x, seeded((rows, cols), 68, 1.0, dtype)], kind="softmax")
    if form == "row":
        return Case(name, Aux(), [x, seeded((cols,), 69, 1.0, dtype)], kind="softmax")
    if form == "col":
        return Case(name, Aux(), [x, seeded((rows, 1), 70, 1.0, dtype)], kind="softmax")
    if form == "scalar":
        return Case(name, Scalar(), [x], kind="softmax")
    if form == "colreduce":
        return Case(name, ColReduce(), [x], kind="softmax")
    raise ValueError(form)


def softmax_dropout(B, H, S, p=0.1, dtype=torch.float16):
    """attention probabilities: softmax, then a generated dropout mask and its product,
    three stores (tuner key (262144, 512)_..._3)."""
    class Mod(torch.nn.Module):
        def forward(self, x):
            s = aten._softmax(x, -1, False)
            r = torch.rand_like(s)
            ge = aten.ge(r, p)
            m = aten.mul(s, ge)
            o = aten.mul(m, 1.0 / (1.0 - p))
            v = aten.view(o, [B * H, S, S])
            return s, ge, v
    return Case(f"softmax_dropout_{B}_{H}_{S}", Mod(), [seeded((B, H, S, S), 66, 2.0, dtype)], kind="softmax")


def softmax_backward_plain(shape, dtype=torch.float16):
    """softmax backward on a 4-D tensor (softmax_backward.py:30-41)."""
    class Mod(torch.nn.Module):
        dt = dtype      # the oracle sets this to float32 when it upcasts the inputs
        def forward(self, g, y):
            return aten._softmax_backward_data(g, y, -1, self.dt)
    y = torch.softmax(seeded(shape, 67, 2.0, torch.float32), -1).to(dtype)
    return Case(f"softmax_backward_{'x'.join(map(str, shape))}", Mod(), [seeded(shape, 68, 1.0, dtype), y],
                kind="softmax_backward")


def softmax_backward_scaled(B, H, S, dtype=torch.float16):
    """softmax backward followed by the 1/sqrt(d) scale and a view (BERT scores gradient)."""
    class Mod(torch.nn.Module):
        dt = dtype
        def forward(self, g, y, mask):
            gm = aten.mul(g, mask)
            d = aten._softmax_backward_data(gm, y, -1, self.dt)
            m = aten.mul(d, 0.125)
            return aten.view(m, [B * H, S, S])
    shape = (B, H, S, S)
    y = torch.softmax(seeded(shape, 69, 2.0, torch.float32), -1).to(dtype)
    mask = (seeded(shape, 71, 1.0, torch.float32) > -1.0)
    return Case(f"softmax_backward_scaled_{B}_{H}_{S}", Mod(), [seeded(shape, 70, 1.0, dtype), y, mask],
                kind="softmax_backward")


def layernorm_affine(S, B, H, dtype=torch.float16, permuted=False):
    """normalise, then gamma / beta in the epilogue; mean and rstd are outputs too
    (layernorm.py:31-77; the permuted-store variant is pattern 2)."""
    class Mod(torch.nn.Module):
        def forward(self, x, g, b):
            ln = aten.native_layer_norm(x, [H], None, None, 1e-12)
            y = operator.getitem(ln, 0)
            mean = operator.getitem(ln, 1)
            rstd = operator.getitem(ln, 2)
            m = aten.mul(y, g)
            a = aten.add(m, b)
            if permuted:
                pm = aten.permute(a, [1, 0, 2])
                c = aten.clone(pm, memory_format=torch.contiguous_format)
                v = aten.view(c, [S * B, H])
                return mean, rstd, c, v
            v = aten.view(a, [S * B, H])
            return mean, rstd, a, v
    return Case(f"layernorm_affine_{S}_{B}_{H}_{'perm' if permuted else 'plain'}_{str(dtype)[6:]}", Mod(),
                [seeded((S, B, H), 72, 1.0, dtype) + 1.0, seeded((H,), 73, 1.0, dtype), seeded((H,), 74, 1.0, dtype)],
                kind="layernorm")


def layernorm_builtin_affine(rows, H, dtype=torch.float16):
    """gamma / beta passed to native_layer_norm itself."""
    class Mod(torch.nn.Module):
        def forward(self, x, g, b):
            ln = aten.native_layer_norm(x, [H], g, b, 1e-5)
            return operator.getitem(ln, 0)
    return Case(f"layernorm_builtin_{rows}_{H}", Mod(),
                [seeded((rows, H), 75, 2.0, dtype), seeded((H,), 76, 1.0, dtype), seeded((H,), 77, 1.0, dtype)],
                kind="layernorm")


def layernorm_backward_mask(S, B, H, dtype=torch.float16):
    """dx of LayerNorm, then a dropout-mask multiply and two stores
    (layernorm_backward.py:31-55)."""
    class Mod(torch.nn.Module):
        def forward(self, grad, x, mean, rstd, gamma, beta, keep):
            ln = aten.native_layer_norm_backward(grad, x, [H], mean, rstd, gamma, beta, [True, False, False])
            dx = operator.getitem(ln, 0)
            m = aten.mul(dx, keep)
            m2 = aten.mul(m, 1.0)
            v = aten.view(m2, [S * B, H])
            s = aten.sum(v, [0], True)        # reductions are never part of a reduce-apply node
            return dx, v, s
    x = seeded((S, B, H), 78, 1.0, dtype)
    xf = x.to(torch.float32)
    mean = xf.mean(-1, keepdim=True)
    rstd = 1.0 / torch.sqrt(xf.var(-1, unbiased=False, keepdim=True) + 1e-12)
    keep = seeded((S, B, H), 81, 1.0, torch.float32) > 0.0
    return Case(f"layernorm_backward_{S}_{B}_{H}_{str(dtype)[6:]}", Mod(),
                [seeded((S, B, H), 79, 1.0, dtype), x, mean, rstd, seeded((H,), 80, 1.0, dtype),
                 seeded((H,), 82, 1.0, dtype), keep], kind="layernorm_backward")


def small_row_cases(dtype=torch.float16) -> List[Case]:
    return [
        softmax_plain(512, 512, dtype),
        softmax_plain(300, 197, dtype),          # ragged rows and columns (ViT token count)
        softmax_plain(128, 1000, dtype),
        softmax_plain(64, 30528, dtype),         # vocabulary-wide rows
        softmax_plain(37, 30522, dtype),         # unpadded vocabulary: scalar path
        softmax_plain(32, 2, dtype),
        softmax_plain(2048, 512, torch.float32),
        softmax_aux_row_col(1024, 512, dtype),
        softmax_backward_plain((2, 4, 128, 128), dtype),
        softmax_backward_plain((3, 197, 197), dtype),
        softmax_backward_scaled(2, 4, 128, dtype),
        layernorm_affine(128, 2, 1024, dtype),
        layernorm_affine(128, 2, 1024, dtype, permuted=True),
        layernorm_affine(50, 3, 768, dtype),
        layernorm_builtin_affine(300, 1000, dtype),
        layernorm_backward_mask(128, 2, 1024, dtype),
        layernorm_backward_mask(50, 3, 768, dtype),
    ]


# ----------------------------------------------------------------------------- SpMM cases
from evt_ae_b200.ops import spmm, spmm_sym  # noqa: E402
torch.fx.wrap("spmm")        # leaves for symbolic_trace in this module's namespace
torch.fx.wrap("spmm_sym")

def chung_lu_graph(n, avg_edges, exponent=2.1, seed=1238):
    """Synthetic power-law graph: expected degrees w_i ~ i^(-1/(exponent-1)), directed edges
    drawn with p_ij ~ w_i w_j, symmetrised, de-duplicated, self loops added.  Returns a COO
    edge list (int32, unsorted, with duplicates left in for the CSR builder to remove)."""
    rng = np.random.default_rng(seed)
    w = np.arange(1, n + 1, dtype=np.float64) ** (-1.0 / (exponent - 1.0))
    p = w / w.sum()
    m = int(avg_edges)
    src = rng.choice(n, size=m, p=p)
    dst = rng.choice(n, size=m, p=p)
    loops = np.arange(n)
    r = np.concatenate([src, dst, loops]).astype(np.int32)
    c = np.concatenate([dst, src, loops]).astype(np.int32)
    perm = rng.permutation(r.shape[0])
    return torch.from_numpy(r[perm]), torch.from_numpy(c[perm])


def csr_reference(coo_row, coo_col, n):
    """sort + unique + searchsorted on the host (numpy): the bit-exact oracle of the CSR builder."""
    key = coo_row.numpy().astype(np.int64) << 32 | coo_col.numpy().astype(np.int64)
    key = np.unique(key)
    rows = (key >> 32).astype(np.int64)
    col = (key & 0xffffffff).astype(np.int32)
    crow = np.searchsorted(rows, np.arange(n + 1), side="left").astype(np.int32)
    return torch.from_numpy(crow), torch.from_numpy(col)


def spmm_case(n, edges, F, variant="plain", dtype=torch.float32, seed=1238):
    """A @ X and its epilogues: `self` adds the node's own feature (GraphConv, gcn_modeling.py:133-144),
    `bias_relu` adds a bias and ReLU, `sym` fuses the d_i^-1/2 d_j^-1/2 normalisation."""
    r, c = chung_lu_graph(n, edges, seed=seed)
    crow, col = csr_reference(r, c, n)
    nnz = col.shape[0]
    deg = (crow[1:] - crow[:-1]).to(torch.float32)
    dinv = (deg + 1.0) ** -0.5
    val = seeded((nnz,), 91, 0.5, torch.float32)
    x = seeded((n, F), 92, 1.0, dtype)
    bias = seeded((F,), 93, 1.0, dtype)

    class Plain(torch.nn.Module):
        def forward(self, crow, col, val, x):
            return spmm(crow, col, val, x)

    class SelfTerm(torch.nn.Module):
        def forward(self, crow, col, val, x):
            return aten.add(spmm(crow, col, val, x), x)

    class BiasRelu(torch.nn.Module):
        def forward(self, crow, col, val, x, b):
            return aten.relu(aten.add(aten.add(spmm(crow, col, val, x), x), b))

    class Sym(torch.nn.Module):
        def forward(self, crow, col, dinv, x):
            return aten.add(spmm_sym(crow, col, dinv, x), x)

    if variant == "plain":
        return Case(f"spmm_plain_{n}_{F}", Plain(), [crow, col, val, x], kind="spmm")
    if variant == "self":
        return Case(f"spmm_self_{n}_{F}", SelfTerm(), [crow, col, val, x], kind="spmm")
    if variant == "bias_relu":
        return Case(f"spmm_bias_relu_{n}_{F}", BiasRelu(), [crow, col, val, x, bias], kind="spmm")
    return Case(f"spmm_sym_{n}_{F}", Sym(), [crow, col, dinv, x], kind="spmm")


def small_spmm_cases():
    return [spmm_case(2000, 9000, 128, "plain"), spmm_case(2000, 9000, 128, "self"),
            spmm_case(3001, 20000, 256, "bias_relu"), spmm_case(2000, 9000, 40, "sym"),
            spmm_case(5000, 60000, 64, "sym"), spmm_case(700, 3000, 128, "self", torch.float16)]


# ----------------------------------------------------------------------------- convolution cases
# Shapes and graph structure of unittest/evt_fuser/conv.py:33-97 after the reference's
# decomposition pass (channels-last leaves, batch norm split into statistics + apply,
# pass_decomposition.py:66-189, evt_fuser.py:1258-1302); batch sizes reduced where noted.
from evt_ae_b200.ops import (convolution_backward_data_channel_last,      # noqa: E402
                             convolution_backward_weight_channel_last, convolution_forward_channel_last)
torch.fx.wrap("convolution_forward_channel_last")
torch.fx.wrap("convolution_backward_data_channel_last")
torch.fx.wrap("convolution_backward_weight_channel_last")


def conv_fprop_bn_stat(N, H, W, C, K, R, stride, dtype=torch.float16):
    """conv + the fusible half of training-mode batch norm: E[y], E[y^2] per channel."""
    pad = R // 2
    P_ = (H + 2 * pad - R) // stride + 1
    rf = 1.0 / (N * P_ * P_)

    class Mod(torch.nn.Module):
        def forward(self, x, w):
            y = convolution_forward_channel_last(x, w, [stride, stride], [pad, pad], [1, 1], False, [0, 0], 1)
            d = aten.mul(y, rf)
            mean = aten.sum(d, [0, 1, 2], True, dtype=torch.float32)
            mean_x2 = aten.sum(aten.mul(d, y), [0, 1, 2], True, dtype=torch.float32)
            return y, mean, mean_x2
    return Case(f"conv_fprop_bn_stat_{N}x{H}x{W}x{C}_k{K}_r{R}_s{stride}_{str(dtype)[6:]}", Mod(),
                [seeded((N, H, W, C), 41, 1.0, dtype), seeded((K, R, R, C), 42, 0.05, dtype)])


def conv_fprop_plain(N, H, W, C, K, R, stride, dtype=torch.float16):
    pad = R // 2

    class Mod(torch.nn.Module):
        def forward(self, x, w):
            return convolution_forward_channel_last(x, w, [stride, stride], [pad, pad], [1, 1], False, [0, 0], 1)
    return Case(f"conv_fprop_plain_{N}x{H}x{W}x{C}_k{K}_r{R}_s{stride}_{str(dtype)[6:]}", Mod(),
                [seeded((N, H, W, C), 43, 1.0, dtype), seeded((K, R, R, C), 44, 0.05, dtype)])


def conv_dgrad_bn_backward_stat(N, H, W, C, K, R, dtype=torch.float16):
    """data gradient + the fusible half of batch-norm backward: sum(dx), sum(dx * x_hat) per
    channel, x_hat from the saved statistics (conv.py:52-78)."""
    pad = R // 2

    class Mod(torch.nn.Module):
        def forward(self, dy, x, w, bn_in, mean, rstd):
            dx = convolution_backward_data_channel_last(dy, x, w, [1, 1], [pad, pad], [1, 1], False, [0, 0], 1)
            sum_gy = aten.sum(dx, [0, 1, 2], dtype=torch.float32)
            xhat = aten.mul(aten.add(bn_in, aten.mul(mean, -1.0)), rstd)
            sum_gy_xhat = aten.sum(aten.mul(dx, xhat), [0, 1, 2], dtype=torch.float32)
            return dx, sum_gy, sum_gy_xhat
    bn_in = seeded((N, H, W, C), 47, 2.0, dtype) + 1.0
    mean = bn_in.float().mean(dim=(0, 1, 2))
    rstd = torch.rsqrt(bn_in.float().var(dim=(0, 1, 2), unbiased=False) + 1e-5)
    return Case(f"conv_dgrad_bn_bwd_stat_{N}x{H}x{W}x{C}_k{K}_r{R}_{str(dtype)[6:]}", Mod(),
                [seeded((N, H, W, K), 45, 1.0, dtype), seeded((N, H, W, C), 46, 1.0, dtype),
                 seeded((K, R, R, C), 48, 0.05, dtype), bn_in, mean, rstd])


def conv_dgrad_strided(N, H, W, C, K, R, stride, dtype=torch.float16):
    """strided data gradient, plain store (conv.py:80-97: 28x28x128 <- 14x14x256, 3x3 / 2)."""
    pad = R // 2
    P_ = (H + 2 * pad - R) // stride + 1
    Q_ = (W + 2 * pad - R) // stride + 1

    class Mod(torch.nn.Module):
        def forward(self, dy, x, w):
            return convolution_backward_data_channel_last(dy, x, w, [stride, stride], [pad, pad], [1, 1], False, [0, 0], 1)
    return Case(f"conv_dgrad_strided_{N}x{H}x{W}x{C}_k{K}_r{R}_s{stride}_{str(dtype)[6:]}", Mod(),
                [seeded((N, P_, Q_, K), 49, 1.0, dtype), seeded((N, H, W, C), 50, 1.0, dtype),
                 seeded((K, R, R, C), 51, 0.05, dtype)])


def conv_wgrad_plain(N, H, W, C, K, R, stride, dtype=torch.float16):
    """filter gradient of a channels-last convolution, dW [K, R, R, C] (the reference's leaf
    convolution_backward_weight_channel_last, pass_decomposition.py:92-107)."""
    pad = R // 2
    P_ = (H + 2 * pad - R) // stride + 1
    Q_ = (W + 2 * pad - R) // stride + 1

    class Mod(torch.nn.Module):
        def forward(self, dy, x, w):
            return convolution_backward_weight_channel_last(dy, x, w, [stride, stride], [pad, pad], [1, 1], False, [0, 0], 1)
    return Case(f"conv_wgrad_{N}x{H}x{W}x{C}_k{K}_r{R}_s{stride}_{str(dtype)[6:]}", Mod(),
                [seeded((N, P_, Q_, K), 52, 0.25, dtype), seeded((N, H, W, C), 53, 1.0, dtype),
                 seeded((K, R, R, C), 54, 0.05, dtype)])


def small_conv_wgrad_cases():
    return [conv_wgrad_plain(4, 14, 14, 64, 64, 3, 1), conv_wgrad_plain(3, 9, 11, 128, 192, 3, 1),
            conv_wgrad_plain(4, 28, 28, 128, 256, 3, 2), conv_wgrad_plain(2, 28, 28, 64, 256, 1, 1),
            conv_wgrad_plain(5, 14, 14, 256, 64, 1, 2), conv_wgrad_plain(2, 7, 7, 512, 512, 3, 1, torch.bfloat16)]


def small_conv_cases():
    return [conv_fprop_bn_stat(4, 56, 56, 64, 64, 3, 1),          # conv2_x 3x3
            conv_fprop_bn_stat(4, 56, 56, 64, 256, 1, 1),         # 1x1 expand
            conv_fprop_plain(6, 28, 28, 128, 128, 3, 2),          # strided 3x3 (28 -> 14)
            conv_fprop_plain(6, 56, 56, 256, 512, 1, 2),          # strided 1x1 shortcut
            conv_fprop_plain(3, 13, 9, 64, 64, 3, 1, torch.bfloat16),   # ragged boxes
            conv_dgrad_bn_backward_stat(4, 56, 56, 64, 64, 3),    # conv.py:52-78 at batch 4
            conv_dgrad_strided(8, 28, 28, 128, 256, 3, 2),        # conv.py:80-97 at batch 8
            conv_dgrad_strided(4, 56, 56, 256, 512, 1, 2),        # 1x1 / 2: three of four parity classes are empty
            conv_dgrad_strided(3, 13, 9, 64, 128, 3, 2, torch.bfloat16)]


# The two supported tests of unittest/evt_fuser/conv.py with the argument lists of the reference's
# modules (NCHW tensors, conv.py:52-97).  The channels-last copies feed the anchor and therefore
# run outside the fused node; the batch-norm apply half consumes finished reductions and runs
# after it.  Outputs follow the reference's order; the weight gradient (a library call on both
# sides) is left out.
from evt_ae_b200.ops import batch_norm_backward_elemt      # noqa: E402
torch.fx.wrap("batch_norm_backward_elemt")


def _nhwc(t):
    return aten.clone(aten.permute(t, [0, 2, 3, 1]), memory_format=torch.contiguous_format)


def conv_dgrad_bn_backward_nchw(N=128, C=64, H=56, dtype=torch.float16):
    rf = 1.0 / (N * H * H)

    class Mod(torch.nn.Module):
        def forward(self, grad_y, input, weight, bn_input_, saved_mean, saved_rstd, gamma):
            dx = convolution_backward_data_channel_last(_nhwc(grad_y), _nhwc(input), _nhwc(weight), [1, 1], [1, 1], [1, 1],
                                                        False, [0, 0], 1)
            sum_gy = aten.sum(dx, [0, 1, 2], dtype=torch.float32)
            xhat = aten.mul(aten.add(bn_input_, aten.mul(saved_mean, -1.0)), saved_rstd)
            sum_gy_xhat = aten.sum(aten.mul(dx, xhat), [0, 1, 2], dtype=torch.float32)
            out = batch_norm_backward_elemt(dx, bn_input_, saved_mean, saved_rstd, C, sum_gy, sum_gy_xhat, rf, gamma)
            gx = operator.getitem(out, 0)
            return aten.permute(gx, [0, 3, 1, 2]), operator.getitem(out, 1), operator.getitem(out, 2)
    return Case(f"conv_dgrad_bn_backward_nchw_{N}x{C}x{H}", Mod(), [])


def conv_stem_bn_nchw(N=128, C=4, K=64, H=224, dtype=torch.float16):
    """7x7 / 2 stem convolution + training-mode batch norm on NCHW tensors (conv.py:33-49), restated
    on the channels-last leaves: permute, convolution, statistics, normalise, permute back."""
    from evt_ae_b200.ops import batch_norm_elemt, batch_norm_stat
    P_ = (H + 6 - 7) // 2 + 1
    rf = 1.0 / (N * P_ * P_)

    class Mod(torch.nn.Module):
        def forward(self, x, w, gamma, beta):
            y = convolution_forward_channel_last(aten.permute(x, [0, 2, 3, 1]), aten.permute(w, [0, 2, 3, 1]),
                                                 [2, 2], [3, 3], [1, 1], False, [0, 0], 1)
            mean, mean_x2 = batch_norm_stat(y, rf)
            out, m, rstd = batch_norm_elemt(y, gamma, beta, mean, mean_x2, 1e-5, K)
            return aten.permute(out, [0, 3, 1, 2]), m, rstd
    return Case(f"conv_stem_bn_nchw_{N}x{C}x{H}_k{K}_{str(dtype)[6:]}", Mod(),
                [seeded((N, C, H, H), 55, 1.0, dtype), seeded((K, C, 7, 7), 56, 1.0, dtype), seeded((K,), 57, 1.0, dtype),
                 seeded((K,), 58, 1.0, dtype)])


def conv_dgrad_strided_nchw(N=128, C=128, K=256, H=28, dtype=torch.float16):
    class Mod(torch.nn.Module):
        def forward(self, grad_y, input, weight):
            return convolution_backward_data_channel_last(_nhwc(grad_y), _nhwc(input), _nhwc(weight), [2, 2], [1, 1], [1, 1],
                                                          False, [0, 0], 1)
    return Case(f"conv_dgrad_strided_nchw_{N}x{C}x{H}_k{K}", Mod(), [])


# ----------------------------------------------------------------------------- GEMM + row-wise step
# Attention scores with their softmax, and the probability gradient with the softmax backward,
# each as ONE partition: the S x S intermediate stays in tensor memory (row-resident kernel).
# The unfused meaning is the two reference partitions back to back (bmm.py:69-94 + softmax.py:30-41;
# softmax_backward.py:30-41).

def bmm_scores_softmax(S, B, H, D, dtype=torch.bfloat16):
    L = B * H
    scale = 1.0 / (D ** 0.5)

    class Mod(torch.nn.Module):
        def forward(self, q3, k3, ext):
            qp = aten.permute(q3, [1, 0, 2])
            kp = aten.permute(k3, [1, 2, 0])
            v = aten.view(aten.bmm(qp, kp), [B, H, S, S])
            sc = aten.add(aten.mul(v, scale), ext)
            return aten.view(aten._softmax(sc, -1, False), [L, S, S])
    mask = torch.zeros(B, 1, 1, S)
    mask[:, :, :, S - S // 8:] = -10000.0          # padded keys
    return Case(f"bmm_scores_softmax_{S}_{B}_{H}_{D}_{str(dtype)[6:]}", Mod(),
                [seeded((S, L, D), 81, 1.0, dtype), seeded((S, L, D), 82, 1.0, dtype), mask.to(dtype)], kind="bmm")


def bmm_dprobs_softmax_backward(S, B, H, D, dtype=torch.bfloat16):
    L = B * H
    scale = 1.0 / (D ** 0.5)

    class Mod(torch.nn.Module):
        dt = dtype      # the oracle sets this to float32 when it upcasts the inputs

        def forward(self, dc3, v3, probs):
            dp = aten.bmm(aten.permute(dc3, [1, 0, 2]), aten.permute(v3, [1, 2, 0]))
            return aten.mul(aten._softmax_backward_data(dp, probs, -1, self.dt), scale)
    probs = torch.softmax(seeded((L, S, S), 85, 2.0, torch.float32), -1).to(dtype)
    return Case(f"bmm_dprobs_softmax_bwd_{S}_{B}_{H}_{D}_{str(dtype)[6:]}", Mod(),
                [seeded((S, L, D), 83, 1.0, dtype), seeded((S, L, D), 84, 1.0, dtype), probs], kind="bmm")


def small_row_resident_cases():
    return [bmm_scores_softmax(512, 2, 4, 64), bmm_dprobs_softmax_backward(512, 2, 4, 64),
            bmm_scores_softmax(197, 2, 3, 64),                       # ViT: 197 columns, ragged rows
            bmm_scores_softmax(256, 1, 4, 64, torch.float16), bmm_dprobs_softmax_backward(320, 1, 2, 64, torch.float16)]
