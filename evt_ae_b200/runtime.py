"""ctypes binding of the C-ABI in include/evt_b200.h.

Stands where the reference's fused ops call the CUTLASS Python runtime
(`operation.run(arguments, stream=...)`, python/gtl/compiler/passes/evt_fuser.py:546;
python/gtl/ops/reduce_apply_operation.py:147-160).  Errors become `RuntimeError`, as the
reference raises on a failing CUresult (reduce_apply_operation.py:156-158).  There is no
fallback: if the library or a kernel image is missing, calls raise.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libevt_b200.so")

(EVTB_GEMM, EVTB_BGEMM, EVTB_SOFTMAX, EVTB_SOFTMAX_BWD, EVTB_LAYERNORM, EVTB_LAYERNORM_BWD, EVTB_SPMM,
 EVTB_CONV_FPROP, EVTB_CONV_DGRAD, EVTB_CONV_WGRAD) = range(10)
EVTB_F16, EVTB_BF16, EVTB_F32 = range(3)
EVTB_MAJOR_K, EVTB_MAJOR_MN = 0, 1

EXPORTED_SYMBOLS = [
    "evtb_version", "evtb_status_string", "evtb_last_error", "evtb_plan_create", "evtb_plan_destroy",
    "evtb_plan_workspace_bytes", "evtb_plan_num_main_operands", "evtb_plan_grid",
    "evtb_plan_set_profile_buffer", "evtb_launch",
    "evtb_launch_ex", "evtb_colsum_workspace_bytes", "evtb_colsum", "evtb_colsum_accumulate", "evtb_colsum_static_max_cols",
    "evtb_colsum_static", "evtb_bn_apply", "evtb_bn_backward_reduce", "evtb_bn_backward_apply", "evtb_maxpool_forward", "evtb_maxpool_backward", "evtb_sddmm", "evtb_csr_build_workspace_bytes", "evtb_csr_build",
]


class evtb_matrix(ctypes.Structure):
    _fields_ = [("major", ctypes.c_int32), ("stride_outer", ctypes.c_int64), ("stride_batch", ctypes.c_int64)]


class evtb_conv(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("N", "H", "W", "C", "K", "R", "S", "P", "Q", "stride_h", "stride_w",
                                              "pad_h", "pad_w", "dil_h", "dil_w")] + \
               [(n, ctypes.c_int64) for n in ("x_stride_w", "x_stride_h", "x_stride_n")]


class evtb_tma_store(ctypes.Structure):
    _fields_ = [("slot", ctypes.c_int32), ("stride_row", ctypes.c_int64), ("stride_batch", ctypes.c_int64)]


class evtb_desc(ctypes.Structure):
    _fields_ = [
        ("kind", ctypes.c_int32), ("dtype", ctypes.c_int32),
        ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64), ("L", ctypes.c_int64),
        ("a", evtb_matrix), ("b", evtb_matrix),
        ("tile_n", ctypes.c_int32), ("stages", ctypes.c_int32), ("threads", ctypes.c_int32),
        ("smem_bytes", ctypes.c_int32), ("rows_per_cta", ctypes.c_int32), ("n_epilogue_ptrs", ctypes.c_int32),
        ("image_path", ctypes.c_char_p), ("entry", ctypes.c_char_p), ("sm_count", ctypes.c_int32),
        ("split_k", ctypes.c_int32), ("cta_pair", ctypes.c_int32), ("row_resident", ctypes.c_int32),
        ("n_tma_stores", ctypes.c_int32), ("tma_stores", evtb_tma_store * 4), ("conv", evtb_conv),
    ]


class evtb_scalars(ctypes.Structure):
    _fields_ = [("scalar", ctypes.c_float * 8), ("seed", ctypes.c_uint64), ("rng_offset", ctypes.c_uint64)]


_lib = None

# kernels of this library enqueued through this binding since import (a launch captured into a
# CUDA graph counts once, at capture): lets a caller state how many of them one step holds
KERNELS_ENQUEUED = 0


def load_library() -> ctypes.CDLL:
    """Load libevt_b200.so from the package directory.  Raises if it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m evt_ae_b200.build` "
            "(there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    lib.evtb_version.restype = ctypes.c_int
    lib.evtb_status_string.restype = ctypes.c_char_p
    lib.evtb_status_string.argtypes = [ctypes.c_int]
    lib.evtb_last_error.restype = ctypes.c_char_p
    lib.evtb_plan_create.argtypes = [ctypes.POINTER(evtb_desc), ctypes.POINTER(ctypes.c_void_p)]
    lib.evtb_plan_destroy.argtypes = [ctypes.c_void_p]
    lib.evtb_plan_workspace_bytes.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_size_t)]
    lib.evtb_plan_num_main_operands.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
    lib.evtb_plan_grid.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
    lib.evtb_plan_set_profile_buffer.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.evtb_launch.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.evtb_launch_ex.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.POINTER(evtb_scalars)]
    lib.evtb_colsum_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.POINTER(ctypes.c_size_t)]
    lib.evtb_colsum.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                ctypes.c_int32, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    lib.evtb_colsum_accumulate.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                           ctypes.c_void_p]
    lib.evtb_sddmm.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64] * 3 + [ctypes.c_void_p, ctypes.c_void_p]
    lib.evtb_csr_build_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.POINTER(ctypes.c_size_t)]
    lib.evtb_csr_build.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                   ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.evtb_colsum_static_max_cols.restype = ctypes.c_int
    lib.evtb_colsum_static.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                       ctypes.c_int32, ctypes.c_void_p]
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    lib.evtb_bn_apply.argtypes = [vp, i32, i64, i64, vp, vp, vp, vp, ctypes.c_float, vp, i32, vp, vp, vp, vp]
    lib.evtb_bn_backward_reduce.argtypes = [vp, vp, vp, vp, i32, i64, i64, vp, vp, vp, vp, vp]
    lib.evtb_bn_backward_apply.argtypes = [vp, vp, i32, i64, i64, vp, vp, vp, vp, ctypes.c_float, vp, vp, vp, vp]
    lib.evtb_maxpool_forward.argtypes = [vp, i32, i64, i64, i64, i64, i32, i32, i32, vp, vp, vp]
    lib.evtb_maxpool_backward.argtypes = [vp, vp, i32, i64, i64, i64, i64, i32, i32, i32, vp, vp]
    _lib = lib
    return lib


def _check(lib, status: int, what: str):
    if status != 0:
        msg = lib.evtb_status_string(status).decode()
        detail = lib.evtb_last_error().decode()
        raise RuntimeError(f"CUDA Error in {what}: {msg}: {detail}")


class Plan:
    """Owns one evtb_plan."""

    def __init__(self, desc: evtb_desc):
        self.lib = load_library()
        self._keep = desc          # keeps the char* fields alive
        self.handle = ctypes.c_void_p()
        _check(self.lib, self.lib.evtb_plan_create(ctypes.byref(desc), ctypes.byref(self.handle)), "evtb_plan_create")
        n = ctypes.c_int()
        _check(self.lib, self.lib.evtb_plan_num_main_operands(self.handle, ctypes.byref(n)), "evtb_plan_num_main_operands")
        self.num_main_operands = n.value
        ws = ctypes.c_size_t()
        _check(self.lib, self.lib.evtb_plan_workspace_bytes(self.handle, ctypes.byref(ws)), "evtb_plan_workspace_bytes")
        self.workspace_bytes = ws.value
        g = ctypes.c_int()
        _check(self.lib, self.lib.evtb_plan_grid(self.handle, ctypes.byref(g)), "evtb_plan_grid")
        self.grid = g.value
        self.n_ptrs = self.num_main_operands + desc.n_epilogue_ptrs
        self._ptr_array = (ctypes.c_void_p * self.n_ptrs)()
        self.kernels_per_launch = 2 if desc.kind == EVTB_SPMM else 1     # SpMM: task list + main kernel

    def launch(self, ptrs: Sequence[int], stream: int, status_ptr: int = 0, workspace_ptr: int = 0,
               scalars: Optional[evtb_scalars] = None):
        if len(ptrs) != self.n_ptrs:
            raise RuntimeError(f"plan expects {self.n_ptrs} pointers, got {len(ptrs)}")
        arr = self._ptr_array
        for i, p in enumerate(ptrs):
            arr[i] = p
        if scalars is None:
            st = self.lib.evtb_launch(self.handle, arr, self.n_ptrs, workspace_ptr, status_ptr, stream)
        else:
            st = self.lib.evtb_launch_ex(self.handle, arr, self.n_ptrs, workspace_ptr, status_ptr, stream,
                                         ctypes.byref(scalars))
        _check(self.lib, st, "evtb_launch")
        global KERNELS_ENQUEUED
        KERNELS_ENQUEUED += self.kernels_per_launch

    def set_profile_buffer(self, device_ptr: int):
        """grid x 8 int64 counters written by kernels built with EVT_B200_KPROFILE=1."""
        _check(self.lib, self.lib.evtb_plan_set_profile_buffer(self.handle, device_ptr), "evtb_plan_set_profile_buffer")

    def __del__(self):
        try:
            if self.handle:
                self.lib.evtb_plan_destroy(self.handle)
                self.handle = None
        except Exception:
            pass
