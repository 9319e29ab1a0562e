"""Thin torch-facing wrappers of the library's fixed (not generated) kernels."""
from __future__ import annotations

import ctypes
from typing import Dict, Tuple

import torch

from . import runtime



@torch.fx.wrap
def one_hot(labels: torch.Tensor, num_classes: int) -> torch.Tensor:
    """`aten.one_hot` as a traceable leaf whose shape inference also works on meta tensors
    (the aten op inspects the label values).  The fuser lowers it to a comparison of the
    label with the column coordinate (reference: `visit_one_hot`,
    python/gtl/compiler/passes/evt_fuser.py:1381-1395)."""
    if labels.device.type == "meta":
        return torch.empty(tuple(labels.shape) + (int(num_classes),), dtype=torch.int64, device="meta")
    return torch.nn.functional.one_hot(labels, num_classes=int(num_classes))


@torch.fx.wrap
def spmm(crow: torch.Tensor, col: torch.Tensor, val: torch.Tensor, feature: torch.Tensor) -> torch.Tensor:
    """Y = A @ feature with A given as CSR in three dense tensors (int32 crow / col, fp32 val).
    Leaf op the fuser anchors on -- the reference's `spmm` leaf takes a sparse-CSR tensor, which
    needs its patched torch to survive tracing (python/gtl/compiler/passes/pass_decomposition.py:61-64;
    python/torch_src/README.md).  The eager body is the unfused meaning of the node."""
    if feature.device.type == "meta":
        return torch.empty((crow.shape[0] - 1, feature.shape[1]), dtype=feature.dtype, device="meta")
    a = torch.sparse_csr_tensor(crow.to(torch.int64), col.to(torch.int64), val.to(feature.dtype),
                                size=(crow.shape[0] - 1, feature.shape[0]))
    return torch.matmul(a, feature)


@torch.fx.wrap
def spmm_sym(crow: torch.Tensor, col: torch.Tensor, dinv: torch.Tensor, feature: torch.Tensor) -> torch.Tensor:
    """Symmetrically normalised aggregation with the normalisation fused:
    Y[i] = dinv[i] * sum_{j in row i} dinv[j] * feature[j]  (dinv = (degree + 1)^-1/2 in the
    reference's GCN, python/model_zoo/gcn/gcn.py:57-62, where the products are materialised as
    edge values on the host)."""
    if feature.device.type == "meta":
        return torch.empty((crow.shape[0] - 1, feature.shape[1]), dtype=feature.dtype, device="meta")
    rows = crow.shape[0] - 1
    row_of = torch.repeat_interleave(torch.arange(rows, device=crow.device), (crow[1:] - crow[:-1]).to(torch.int64))
    val = dinv[row_of] * dinv[col.to(torch.int64)]
    return spmm(crow, col, val, feature)


# ---------------------------------------------------------------------------------------------
# Channels-last convolution and split batch-norm leaves.  Same names, argument order and meaning
# as the reference's wrapped functions (python/gtl/compiler/passes/pass_decomposition.py:66-189),
# which its decomposition pass puts in place of aten.convolution / convolution_backward /
# _native_batch_norm_legit / native_batch_norm_backward; the eager bodies below are the unfused
# meaning of each node (what the oracle runs), written against NHWC tensors.
# ---------------------------------------------------------------------------------------------

def _conv_out_hw(h, w, r, s, stride, padding, dilation):
    p = (h + 2 * padding[0] - dilation[0] * (r - 1) - 1) // stride[0] + 1
    q = (w + 2 * padding[1] - dilation[1] * (s - 1) - 1) // stride[1] + 1
    return p, q


@torch.fx.wrap
def convolution_forward_channel_last(input_channel_last, weight_channel_last, stride, padding, dilation, transposed,
                                     output_padding, groups):
    """x [N,H,W,C], w [K,R,S,C] -> y [N,P,Q,K] (all contiguous, channels last)."""
    n, h, w, c = input_channel_last.shape
    k, r, s, _ = weight_channel_last.shape
    if input_channel_last.device.type == "meta":
        p, q = _conv_out_hw(h, w, r, s, stride, padding, dilation)
        return torch.empty((n, p, q, k), dtype=input_channel_last.dtype, device="meta")
    y = torch.ops.aten.convolution(input_channel_last.permute(0, 3, 1, 2), weight_channel_last.permute(0, 3, 1, 2),
                                   None, stride, padding, dilation, transposed, output_padding, groups)
    return y.permute(0, 2, 3, 1).contiguous()


@torch.fx.wrap
def convolution_backward_data_channel_last(grad_output_channel_last, input_channel_last, weight_channel_last, stride,
                                           padding, dilation, transposed, output_padding, groups):
    """dy [N,P,Q,K], x (shape only) [N,H,W,C], w [K,R,S,C] -> dx [N,H,W,C]."""
    if grad_output_channel_last.device.type == "meta":
        return torch.empty(tuple(input_channel_last.shape), dtype=grad_output_channel_last.dtype, device="meta")
    gx = torch.ops.aten.convolution_backward(
        grad_output_channel_last.permute(0, 3, 1, 2), input_channel_last.permute(0, 3, 1, 2),
        weight_channel_last.permute(0, 3, 1, 2), [0], stride, padding, dilation, transposed, output_padding, groups,
        [True, False, False])[0]
    return gx.permute(0, 2, 3, 1).contiguous()


@torch.fx.wrap
def convolution_backward_weight_channel_last(grad_output_channel_last, input_channel_last, weight_channel_last, stride,
                                             padding, dilation, transposed, output_padding, groups):
    """dw [K,R,S,C]: no epilogue is ever fused here; as in the reference this stays a library
    call (cuDNN through aten.convolution_backward, pass_decomposition.py:92-107)."""
    if grad_output_channel_last.device.type == "meta":
        return torch.empty(tuple(weight_channel_last.shape), dtype=weight_channel_last.dtype, device="meta")
    gw = torch.ops.aten.convolution_backward(
        grad_output_channel_last.permute(0, 3, 1, 2), input_channel_last.permute(0, 3, 1, 2),
        weight_channel_last.permute(0, 3, 1, 2), [0], stride, padding, dilation, transposed, output_padding, groups,
        [False, True, False])[1]
    return gw.permute(0, 2, 3, 1).contiguous()


def _pool_args(kernel_size, stride, padding):
    k, s, p = list(kernel_size), list(stride), list(padding)
    if len(set(k)) != 1 or len(set(s)) != 1 or len(set(p)) != 1:
        raise NotImplementedError("max-pool kernels take square windows, equal strides and equal paddings")
    return int(k[0]), int(s[0]), int(p[0])


@torch.fx.wrap
def max_pool2d_with_indices_channel_last(inputs_cl, kernel_size, stride, padding):
    """The reference's leaf (pass_decomposition.py:109-118): (output, indices), both channels-last.  On
    half-precision CUDA tensors this library's kernel runs and `indices` is a uint8 tensor holding the
    place of the maximum inside its window (r * k + t) -- opaque to everything but the backward leaf;
    elsewhere the library call with its int64 indices."""
    if inputs_cl.is_cuda and inputs_cl.dtype in (torch.float16, torch.bfloat16) and inputs_cl.shape[-1] % 8 == 0:
        k, s, p = _pool_args(kernel_size, stride, padding)
        x = inputs_cl.contiguous()
        N, H, W, C = x.shape
        P, Q = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        y = torch.empty(N, P, Q, C, dtype=x.dtype, device=x.device)
        code = torch.empty(N, P, Q, C, dtype=torch.uint8, device=x.device)
        lib = runtime.load_library()
        st = lib.evtb_maxpool_forward(x.data_ptr(), _DT[x.dtype], N, H, W, C, k, s, p, y.data_ptr(), code.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
        runtime._check(lib, st, "evtb_maxpool_forward")
        runtime.KERNELS_ENQUEUED += 1
        return y, code
    out, idx = torch.ops.aten.max_pool2d_with_indices(inputs_cl.permute(0, 3, 1, 2), kernel_size, stride, padding)
    return out.permute(0, 2, 3, 1), idx.permute(0, 2, 3, 1)


@torch.fx.wrap
def max_pool2d_with_indices_backward_channel_last(grad_output_cl, x_cl, kernel_size, stride, padding, dilation, ceil_mode,
                                                  indices_cl):
    """The reference's leaf (pass_decomposition.py:120-132).  `indices_cl` is what the forward leaf
    returned: uint8 window places (this library's kernel) or int64 flat indices (the library call)."""
    if indices_cl.dtype == torch.uint8:
        if list(dilation) != [1, 1] or ceil_mode:
            raise NotImplementedError("max-pool kernels: dilation 1, floor mode")
        k, s, p = _pool_args(kernel_size, stride, padding)
        dy = grad_output_cl.contiguous()
        N, H, W, C = x_cl.shape
        dx = torch.empty(N, H, W, C, dtype=dy.dtype, device=dy.device)
        lib = runtime.load_library()
        st = lib.evtb_maxpool_backward(dy.data_ptr(), indices_cl.contiguous().data_ptr(), _DT[dy.dtype], N, H, W, C, k, s, p,
                                       dx.data_ptr(), torch.cuda.current_stream().cuda_stream)
        runtime._check(lib, st, "evtb_maxpool_backward")
        runtime.KERNELS_ENQUEUED += 1
        return dx
    g = torch.ops.aten.max_pool2d_with_indices_backward(grad_output_cl.permute(0, 3, 1, 2), x_cl.permute(0, 3, 1, 2), kernel_size,
                                                        stride, padding, dilation, ceil_mode, indices_cl.permute(0, 3, 1, 2))
    return g.permute(0, 2, 3, 1)


@torch.fx.wrap
def batch_norm_stat(input, reduction_factor):
    """Per-channel E[x], E[x^2] in fp32 over N, H, W of a channels-last tensor (the half of
    training-mode batch norm that is fusible into the producing convolution's epilogue)."""
    if input.device.type == "meta":
        v = torch.empty((input.shape[-1],), dtype=torch.float32, device="meta")
        return v, v.clone()
    if input.is_cuda and input.dtype in (torch.float16, torch.bfloat16):
        # one pass of the backward-sums kernel with mean 0 and rstd 1: sum(y) and sum(y * y)
        C = input.shape[-1]
        unit = _unit_vectors(C, input.device)
        _, sums = bn_backward_reduce(input, input, unit[0], unit[1])
        sums = sums * reduction_factor
        return sums[0], sums[1]
    x = input.to(torch.float32)
    return x.mean(dim=(0, 1, 2)), (x * x).mean(dim=(0, 1, 2))


@torch.fx.wrap
def batch_norm_elemt(input, weight, bias, mean_vec, mean_x2_vec, eps, K):
    """Normalise with the statistics of batch_norm_stat; returns (y, saved_mean, saved_rstd)."""
    if input.device.type == "meta":
        v = torch.empty((input.shape[-1],), dtype=torch.float32, device="meta")
        return torch.empty_like(input), v, v.clone()
    if input.is_cuda and input.dtype in (torch.float16, torch.bfloat16):
        return bn_apply(input, mean_vec, mean_x2_vec, weight, bias, eps)
    mean = mean_vec.reshape(-1).to(torch.float32)
    rstd = torch.rsqrt(mean_x2_vec.reshape(-1).to(torch.float32) - mean * mean + eps)
    y = (input.to(torch.float32) - mean) * (weight.to(torch.float32) * rstd) + bias.to(torch.float32)
    return y.to(input.dtype), mean, rstd


@torch.fx.wrap
def batch_norm_backward_stat(y_grad, input, saved_mean, saved_rstd, K):
    """sum(dy) and sum(dy * x_hat) per channel in fp32 (fusible into the producing data-gradient
    convolution's epilogue)."""
    if y_grad.device.type == "meta":
        v = torch.empty((input.shape[-1],), dtype=torch.float32, device="meta")
        return v, v.clone()
    if y_grad.is_cuda and y_grad.dtype in (torch.float16, torch.bfloat16):
        _, sums = bn_backward_reduce(y_grad, input, saved_mean, saved_rstd)
        return sums[0], sums[1]
    g = y_grad.to(torch.float32)
    xhat = (input.to(torch.float32) - saved_mean) * saved_rstd
    return g.sum(dim=(0, 1, 2)), (g * xhat).sum(dim=(0, 1, 2))


@torch.fx.wrap
def batch_norm_backward_elemt(y_grad, input, saved_mean, saved_rstd, K, sum_grad_y, sum_grad_y_xhat, reduction_factor,
                              gamma):
    """dx of training-mode batch norm from the two sums; returns (dx, dgamma, dbeta)."""
    if y_grad.device.type == "meta":
        v = torch.empty((input.shape[-1],), dtype=y_grad.dtype, device="meta")
        return torch.empty_like(y_grad), v, v.clone()
    if y_grad.is_cuda and y_grad.dtype in (torch.float16, torch.bfloat16):
        sums = torch.stack([sum_grad_y.reshape(-1).to(torch.float32), sum_grad_y_xhat.reshape(-1).to(torch.float32)])
        return bn_backward_apply(y_grad, input, saved_mean, saved_rstd, gamma, sums, reduction_factor)
    g = y_grad.to(torch.float32)
    xhat = (input.to(torch.float32) - saved_mean) * saved_rstd
    mean_g = sum_grad_y.reshape(-1).to(torch.float32) * reduction_factor
    mean_gx = sum_grad_y_xhat.reshape(-1).to(torch.float32) * reduction_factor
    dx = (g - mean_g - xhat * mean_gx) * (gamma.to(torch.float32) * saved_rstd)
    return (dx.to(y_grad.dtype), sum_grad_y_xhat.reshape(-1).to(y_grad.dtype),
            sum_grad_y.reshape(-1).to(y_grad.dtype))


class StemWindow:
    """A few-channel convolution (the 7 x 7 / 2 stem of a ResNet on 3- or 4-channel images,
    python/model_zoo/resnet/resnet_modeling.py:190) restated for kernels that move 64 channels at a
    time: the taps of one filter row times the channels become the "channels".

    The image is copied once into a zero-padded buffer [N, H + 2 pad, Wp, C'] (C' = channels rounded up
    to a divisor of 64); an overlapping strided view [N, Hp, Q, 64] of it -- element (n, h, q, :) is the
    64 / C' pixels starting at padded column q * stride_w -- is the activation, the filter becomes
    [K, R, 1, 64] with the S taps of a row at their place inside the window (zero elsewhere), and the
    convolution is R x 1 with stride (stride_h, 1) and no padding.  Results equal the original
    convolution's; the filter gradient comes back through `unfold`.  Window starts are 16-byte
    aligned, as the tensor-map loads of the fused kernels require."""

    def __init__(self, x_shape, w_shape, stride, padding):
        N, H, W, C = x_shape
        K, R, S, Cw = w_shape
        if Cw != C:
            raise ValueError("image and filter channel counts differ")
        Cp = next(c for c in (1, 2, 4, 8, 16, 32, 64) if c >= C)
        sh, sw = stride
        ph, pw = padding
        px = 64 // Cp                                  # pixels per window
        align = max(1, 8 // Cp)                        # window starts on 16-byte boundaries
        if Cp == 64 or (sw * Cp) % 8:
            raise NotImplementedError("window view: needs fewer than 64 channels and stride_w * channels % 8 == 0")
        pad_l = -(-pw // align) * align
        self.shift = pad_l - pw
        if S + self.shift > px:
            raise NotImplementedError(f"window view: {S} taps (+{self.shift}) do not fit {px} pixels of {Cp} channels")
        self.P, self.Q = (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1
        Wp = max(pad_l + W + pw, (self.Q - 1) * sw + px)
        while (Wp * Cp) % 8:
            Wp += 1
        self.N, self.H, self.W, self.C, self.Cp, self.K, self.R, self.S = N, H, W, C, Cp, K, R, S
        self.Hp, self.Wp, self.pad_t, self.pad_l = H + 2 * ph, Wp, ph, pad_l
        self.view_shape = (N, self.Hp, self.Q, 64)
        self.view_strides = (self.Hp * Wp * Cp, Wp * Cp, sw * Cp, 1)
        self.stride, self.padding = [sh, 1], [0, 0]    # of the restated convolution
        self.filter_shape = (K, R, 1, 64)

    def image(self, x: torch.Tensor, dtype=None) -> torch.Tensor:
        """the window view of x [N, H, W, C] (a new zero-padded buffer holds the data)"""
        buf = torch.zeros(self.N, self.Hp, self.Wp, self.Cp, dtype=dtype or x.dtype, device=x.device)
        buf[:, self.pad_t:self.pad_t + self.H, self.pad_l:self.pad_l + self.W, :self.C] = x
        return buf.as_strided(self.view_shape, self.view_strides)

    def meta_image(self, dtype) -> torch.Tensor:
        return torch.empty(self.N * self.Hp * self.Wp * self.Cp, dtype=dtype, device="meta").as_strided(
            self.view_shape, self.view_strides)

    def filter(self, w: torch.Tensor) -> torch.Tensor:
        out = torch.zeros(self.K, self.R, 64 // self.Cp, self.Cp, dtype=w.dtype, device=w.device)
        out[:, :, self.shift:self.shift + self.S, :self.C] = w
        return out.view(self.K, self.R, 1, 64)

    def unfold(self, dw_window: torch.Tensor) -> torch.Tensor:
        """filter gradient [K, R, S, C] from the gradient of the window filter [K, R, 1, 64]"""
        g = dw_window.reshape(self.K, self.R, 64 // self.Cp, self.Cp)
        return g[:, :, self.shift:self.shift + self.S, :self.C].contiguous()


_DT = {torch.float16: runtime.EVTB_F16, torch.bfloat16: runtime.EVTB_BF16, torch.float32: runtime.EVTB_F32}
_colsum_ws: Dict[Tuple[int, int, int, int], torch.Tensor] = {}


def colsum(x: torch.Tensor, out_dtype: torch.dtype = None) -> torch.Tensor:
    """Sum over all leading dims of a contiguous CUDA tensor: [..., C] -> [C], fp32 accumulate.
    Stands for the `aten.sum(x, outer_dims)` bias-gradient nodes that the reference's
    partitioner leaves outside reduce-apply kernels (evt_fuser.py:1096-1100)."""
    if not x.is_cuda:
        raise RuntimeError("colsum runs on CUDA tensors only; there is no CPU path")
    lib = runtime.load_library()
    x = x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols
    out_dtype = out_dtype or x.dtype
    stream = torch.cuda.current_stream()
    if out_dtype == torch.float32:
        # one pass with atomics into a zeroed fp32 vector (from the active reduction arena if any)
        from . import fused_ops
        arena = fused_ops._ACTIVE_ARENA
        y = arena.take((cols,), x.device) if arena is not None else None
        if y is None:
            y = torch.zeros(cols, dtype=torch.float32, device=x.device)
        st = lib.evtb_colsum_accumulate(x.data_ptr(), _DT[x.dtype], rows, cols, y.data_ptr(), stream.cuda_stream)
        runtime._check(lib, st, "evtb_colsum_accumulate")
        runtime.KERNELS_ENQUEUED += 1
        return y
    y = torch.empty(cols, dtype=out_dtype, device=x.device)
    nbytes = ctypes.c_size_t()
    runtime._check(lib, lib.evtb_colsum_workspace_bytes(rows, cols, ctypes.byref(nbytes)), "evtb_colsum_workspace_bytes")
    key = (x.device.index, rows, cols, stream.cuda_stream)
    ws = _colsum_ws.get(key)
    if ws is None:
        ws = torch.zeros((nbytes.value + 3) // 4, dtype=torch.int32, device=x.device)   # zero-filled once
        _colsum_ws[key] = ws
    st = lib.evtb_colsum(x.data_ptr(), _DT[x.dtype], rows, cols, y.data_ptr(), _DT[out_dtype], ws.data_ptr(),
                         ws.numel() * 4, stream.cuda_stream)
    runtime._check(lib, st, "evtb_colsum")
    runtime.KERNELS_ENQUEUED += 1
    return y


def _bn_operands(*tensors):
    """Activations as contiguous [rows, C] views of one half-precision CUDA dtype."""
    first = tensors[0]
    if not first.is_cuda or first.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("the batch-norm kernels run on fp16 / bf16 CUDA tensors only; there is no CPU path")
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
            continue
        if t.dtype != first.dtype or t.shape != first.shape:
            raise RuntimeError("batch-norm activations must share dtype and shape")
        out.append(t.contiguous())
    C = first.shape[-1]
    return out, first.numel() // C, C


_units: Dict[Tuple[int, str], torch.Tensor] = {}


def _unit_vectors(C, device):
    """[zeros(C), ones(C)] in fp32 on `device`, made once"""
    key = (C, str(device))
    if key not in _units:
        _units[key] = torch.stack([torch.zeros(C, dtype=torch.float32, device=device),
                                   torch.ones(C, dtype=torch.float32, device=device)])
    return _units[key]


def _zeroed_f32(shape, device):
    from . import fused_ops
    arena = fused_ops._ACTIVE_ARENA
    t = arena.take(shape, device) if arena is not None else None
    return t if t is not None else torch.zeros(shape, dtype=torch.float32, device=device)


def _f32_vec(v, C):
    v = v.reshape(-1)
    if v.dtype != torch.float32 or v.numel() != C:
        v = v.to(torch.float32)
    return v.contiguous()


def bn_apply(y, mean_vec, mean_x2_vec, gamma, beta, eps, residual=None, relu=False):
    """z = act((y - mean) * rstd * gamma + beta [+ residual]) on a channels-last activation, from the
    E[y], E[y^2] vectors of the producing convolution's epilogue: the reference's batch_norm_elemt
    leaf (pass_decomposition.py:143-157) with the following ReLU / residual addition in the same
    pass.  Returns (z, saved_mean, saved_rstd)."""
    (y, residual), rows, C = _bn_operands(y, residual)
    lib = runtime.load_library()
    z = torch.empty_like(y)
    stats = torch.empty(2, C, dtype=torch.float32, device=y.device)
    mean_vec, mean_x2_vec = _f32_vec(mean_vec, C), _f32_vec(mean_x2_vec, C)
    gamma, beta = gamma.to(y.dtype).contiguous(), beta.to(y.dtype).contiguous()
    st = lib.evtb_bn_apply(y.data_ptr(), _DT[y.dtype], rows, C, mean_vec.data_ptr(), mean_x2_vec.data_ptr(),
                           gamma.data_ptr(), beta.data_ptr(), float(eps), residual.data_ptr() if residual is not None else None,
                           1 if relu else 0, z.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
    runtime._check(lib, st, "evtb_bn_apply")
    runtime.KERNELS_ENQUEUED += 1
    return z, stats[0], stats[1]


def bn_backward_reduce(grad, y, mean, rstd, act=None, grad2=None):
    """g' = (grad [+ grad2]) [* (act > 0)] and the two per-channel sums of batch-norm backward,
    sum(g') and sum(g' * x_hat): the reference's batch_norm_backward_stat leaf
    (pass_decomposition.py:159-168) with the ReLU mask and the gradient addition in front of it
    in the same pass.  Returns (g', sums fp32 [2, C])."""
    (grad, y, act, grad2), rows, C = _bn_operands(grad, y, act, grad2)
    lib = runtime.load_library()
    changed = act is not None or grad2 is not None
    out = torch.empty_like(grad) if changed else None
    sums = _zeroed_f32((2, C), grad.device)
    mean, rstd = _f32_vec(mean, C), _f32_vec(rstd, C)
    ptr = lambda t: t.data_ptr() if t is not None else None
    st = lib.evtb_bn_backward_reduce(grad.data_ptr(), ptr(grad2), ptr(act), y.data_ptr(), _DT[grad.dtype], rows, C,
                                     mean.data_ptr(), rstd.data_ptr(), ptr(out), sums.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    runtime._check(lib, st, "evtb_bn_backward_reduce")
    runtime.KERNELS_ENQUEUED += 1
    return (out if changed else grad), sums


def bn_backward_apply(grad, y, mean, rstd, gamma, sums, reduction_factor):
    """dy = (grad - mean(grad) - x_hat * mean(grad * x_hat)) * gamma * rstd and dgamma, dbeta from the
    sums: the reference's batch_norm_backward_elemt leaf (pass_decomposition.py:170-189)."""
    (grad, y), rows, C = _bn_operands(grad, y)
    lib = runtime.load_library()
    dy = torch.empty_like(grad)
    dgb = torch.empty(2, C, dtype=grad.dtype, device=grad.device)
    mean, rstd = _f32_vec(mean, C), _f32_vec(rstd, C)
    sums = sums.reshape(2, C).to(torch.float32).contiguous()
    gamma = gamma.to(grad.dtype).contiguous()
    st = lib.evtb_bn_backward_apply(grad.data_ptr(), y.data_ptr(), _DT[grad.dtype], rows, C, mean.data_ptr(), rstd.data_ptr(),
                                    gamma.data_ptr(), sums.data_ptr(), float(reduction_factor), dy.data_ptr(),
                                    dgb[0].data_ptr(), dgb[1].data_ptr(), torch.cuda.current_stream().cuda_stream)
    runtime._check(lib, st, "evtb_bn_backward_apply")
    runtime.KERNELS_ENQUEUED += 1
    return dy, dgb[0], dgb[1]


def sddmm(crow: torch.Tensor, col: torch.Tensor, u: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """out[p] = <u[i], v[col[p]]> for every stored entry p of row i of the CSR pattern (fp32)."""
    if not u.is_cuda:
        raise RuntimeError("sddmm runs on CUDA tensors only; there is no CPU path")
    lib = runtime.load_library()
    u, v = u.contiguous(), v.contiguous()
    rows, nnz, F = crow.shape[0] - 1, col.shape[0], u.shape[1]
    if u.dtype != torch.float32 or v.dtype != torch.float32 or crow.dtype != torch.int32 or col.dtype != torch.int32:
        raise RuntimeError("sddmm needs fp32 features and int32 CSR indices")
    out = torch.empty(nnz, dtype=torch.float32, device=u.device)
    st = lib.evtb_sddmm(crow.data_ptr(), col.data_ptr(), u.data_ptr(), v.data_ptr(), rows, nnz, F, out.data_ptr(),
                        torch.cuda.current_stream().cuda_stream)
    runtime._check(lib, st, "evtb_sddmm")
    runtime.KERNELS_ENQUEUED += 1
    return out


def csr_build(coo_row: torch.Tensor, coo_col: torch.Tensor, rows: int):
    """COO (int32, any order, duplicates allowed) -> (crow, col) int32 CSR with sorted, unique
    columns per row.  Returns tensors trimmed to the number of distinct edges."""
    if not coo_row.is_cuda:
        raise RuntimeError("csr_build runs on CUDA tensors only; there is no CPU path")
    lib = runtime.load_library()
    coo_row, coo_col = coo_row.contiguous(), coo_col.contiguous()
    if coo_row.dtype != torch.int32 or coo_col.dtype != torch.int32:
        raise RuntimeError("csr_build needs int32 indices")
    n = coo_row.numel()
    nbytes = ctypes.c_size_t()
    runtime._check(lib, lib.evtb_csr_build_workspace_bytes(n, ctypes.byref(nbytes)), "evtb_csr_build_workspace_bytes")
    ws = torch.empty(nbytes.value + 256, dtype=torch.uint8, device=coo_row.device)
    off = (-ws.data_ptr()) % 256
    crow = torch.empty(rows + 1, dtype=torch.int32, device=coo_row.device)
    col = torch.empty(n, dtype=torch.int32, device=coo_row.device)
    nnz = torch.zeros(1, dtype=torch.int32, device=coo_row.device)
    st = lib.evtb_csr_build(coo_row.data_ptr(), coo_col.data_ptr(), n, rows, ws.data_ptr() + off, nbytes.value,
                            crow.data_ptr(), col.data_ptr(), nnz.data_ptr(), torch.cuda.current_stream().cuda_stream)
    runtime._check(lib, st, "evtb_csr_build")
    return crow, col[: int(nnz.item())]
