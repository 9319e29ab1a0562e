"""Fused-operator objects: the callables the fuser plants in the fx graph.

Same surface as the reference's wrappers in python/gtl/compiler/passes/evt_fuser.py
(`FusedOpBase` :62-280, `FusedGEMM` :453-558, `FusedBMM` :561-697, ...): constructed from the
anchor node and the traced epilogue, exposing `__name__`, `target`,
`mainloop_fusion_targets`, `args`, `input_names`, `outputs`, and called as

    outs = fused(*epilogue_inputs, *mainloop_operands)      # -> list[Tensor]

Below that surface everything is new: the epilogue is compiled by `codegen` + `jit` into a
cubin and launched through the C-ABI (`runtime.Plan`).  No CUTLASS, no cuBLAS, no eager
fallback: a missing library or image raises.
"""
from __future__ import annotations

import math
import os
from typing import Any, Dict, List, Optional, Sequence

import torch

from . import codegen, jit, runtime, tuning
from .codegen import GemmTileConfig
from .ir import EpilogueIR
from .ops import _conv_out_hw
from .tracer import OperandSpec, PartitionTrace, _shape, _dtype, _meta

SM_COUNT_DEFAULT = 148
SMEM_LIMIT = 227 * 1024

_DT = {torch.float16: runtime.EVTB_F16, torch.bfloat16: runtime.EVTB_BF16, torch.float32: runtime.EVTB_F32}


def _sm_count() -> int:
    if torch.cuda.is_available():
        return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return SM_COUNT_DEFAULT


def pick_gemm_tile(M: int, N: int, K: int, L: int, b_major: str, sms: int = SM_COUNT_DEFAULT,
                   epilogue_bytes_per_elem: float = 2.0) -> GemmTileConfig:
    """Tile choice, the job of the reference's two-stage tuner
    (python/gtl/compiler/autotuner/gemm_tuner.py:126-153) reduced to a closed form: the
    accumulator tile is always 128 rows (one TMEM lane per row); pick the widest tile_n that
    still gives every SM work, preferring fewer, fuller waves."""
    cands = [256, 128, 64] if b_major == "MN" else [256, 128, 64, 32]
    best, best_cost = None, None
    tiles_m = (M + 127) // 128
    for bn in cands:
        if bn > 32 and bn // 2 >= N and bn // 2 in cands:
            continue  # a narrower tile covers N just as well
        tiles = tiles_m * ((N + bn - 1) // bn) * L
        waves = (tiles + sms - 1) // sms
        # time model: per tile, main loop ~ bn * K, epilogue ~ bn * const; small tiles pay
        # more shared-memory traffic per flop (A tile re-read per column strip)
        per_tile = bn * (K + 64) * (1.0 + 0.12 * (256 / bn - 1))
        cost = waves * per_tile
        if best_cost is None or cost < best_cost * 0.98:
            best, best_cost = bn, cost
    # too few tiles for the machine but a long K: keep the wide tile and cut K instead
    # (the reference's tuner reaches for StreamK on the same weight-gradient shapes)
    split = 1
    wide = 256 if N >= 256 else best
    tiles_wide = tiles_m * ((N + wide - 1) // wide) * L
    num_k = (K + 63) // 64
    if tiles_wide * 2 <= sms and num_k >= 32:
        split = max(1, min(sms // tiles_wide, num_k // 8, 16))
        if split > 1:
            best = wide
    # wide tiles go to CTA pairs (cluster of two, tcgen05 cta_group::2): a third less operand
    # traffic from L2 per flop, which is what limits the lone CTA; needs at least two row tiles,
    # and a K loop long enough to be the limit (short-K batched GEMMs are bound by their stores)
    pair = best == 256 and M > 128 and num_k // split >= 4
    stage_bytes = 128 * 64 * 2 + (best // 2 if pair else best) * 64 * 2
    stages = max(2, min(8, (SMEM_LIMIT - 2048) // stage_bytes))
    return GemmTileConfig(bn=best, stages=int(stages), split_k=int(split), cta_pair=pair)


PROFILE_EVENTS: list = []


def profile_summary(names: Optional[Dict[int, str]] = None):
    """Per fused node: (label, launches, total ms) from the events MODE=PROFILE collected
    (call after torch.cuda.synchronize()); clears the event list."""
    agg: Dict[int, list] = {}
    for op, e0, e1 in PROFILE_EVENTS:
        a = agg.setdefault(id(op), [op, 0, 0.0])
        a[1] += 1
        a[2] += e0.elapsed_time(e1)
    PROFILE_EVENTS.clear()
    out = []
    for op, n, ms in agg.values():
        label = (names or {}).get(id(op), type(op).__name__)
        out.append((label, n, ms, op))
    return sorted(out, key=lambda r: -r[2])


class ReductionArena:
    """One zero-filled fp32 buffer that the sum-type reduction targets of many fused nodes are
    carved from, so that a step pays one memset instead of one fill kernel per reduction (the
    reference zero-fills each target separately, evt_fuser.py:217-225).  Results are views into
    the arena: they stay valid until the next `reset()`.

        arena = ReductionArena(device)
        arena.reset()                      # start of a step (captured as one memset in a CUDA graph)
        with arena:
            ... call fused nodes ...
    """

    def __init__(self, device, floats: int = 4 << 20):
        self.buf = torch.zeros(floats, dtype=torch.float32, device=device)
        self.off = 0

    def reset(self):
        self.buf.zero_()
        self.off = 0

    def take(self, shape, device):
        n = int(math.prod(shape))
        if self.buf.device != torch.device(device) or self.off + n > self.buf.numel():
            return None                    # the caller falls back to its own fill
        t = self.buf[self.off:self.off + n].view(tuple(shape))
        self.off += (n + 63) // 64 * 64    # 256-byte granules
        return t

    def __enter__(self):
        global _ACTIVE_ARENA
        self._prev = _ACTIVE_ARENA
        _ACTIVE_ARENA = self
        return self

    def __exit__(self, *exc):
        global _ACTIVE_ARENA
        _ACTIVE_ARENA = self._prev
        return False


_ACTIVE_ARENA: Optional[ReductionArena] = None


def _view_strides(node) -> Optional[tuple]:
    """Strides of a convolution activation that is a strided view with unit channel stride, else None."""
    tm = _meta(node)
    st = tuple(int(v) for v in getattr(tm, "stride", ()) or ())
    shape = tuple(int(v) for v in tm.shape)
    if len(st) != 4:
        return None
    dense = (shape[1] * shape[2] * shape[3], shape[2] * shape[3], shape[3], 1)
    if st == dense:
        return None
    if st[3] != 1 or any(v <= 0 or v % 8 for v in st[:3]):
        raise NotImplementedError(f"activation view with strides {st}: the channel stride must be 1 and the others "
                                  "positive multiples of 8 elements")
    return st


class FusedOpBase:
    """Base of all fused operators (reference: evt_fuser.py:62-280)."""
    __name__ = "evt_b200_fused_op"
    view_operand = -1          # index (among the main operands) of an activation that may be a strided view
    view_strides = None        # its strides when the plan was made for a view
    target = None
    mainloop_fusion_targets: list = []

    def __init__(self, trace: PartitionTrace):
        self.trace = trace
        self.node = trace.anchor
        self.ir: EpilogueIR = trace.ir
        self.outputs = trace.outputs
        self.output_stores = trace.output_stores
        self.inputs = trace.inputs
        self.input_names = trace.input_names
        self.args = list(trace.mainloop_args)
        self.output_shapes = [_shape(o) for o in self.outputs]
        self.output_dtypes = [_dtype(o) for o in self.outputs]
        self.stream = None
        self.mode = os.environ.get("MODE", "RUN")
        self.plan: Optional[runtime.Plan] = None
        self.slots: List[codegen.OperandSlot] = []
        self._status = None
        self.seed = 0
        self.rng_offset = 0

    # -- status word -----------------------------------------------------------------
    def _workspace_ptr(self, device) -> int:
        return 0

    def _status_ptr(self, device) -> int:
        if self._status is None or self._status.device != device:
            self._status = torch.zeros(1, dtype=torch.int32, device=device)
        return self._status.data_ptr()

    def check_status(self):
        """Synchronises and raises if a bounded device-side wait ran out."""
        if self._status is not None:
            code = int(self._status.item())
            if code != 0:
                raise RuntimeError(f"CUDA Error: device status {code} from {self.__name__} (bounded wait ran out)")

    # -- call ------------------------------------------------------------------------
    def _main_ptrs(self, main_tensors: Sequence[torch.Tensor], keep: list) -> List[int]:
        raise NotImplementedError

    def __call__(self, *args_):
        n_epi = len(self.input_names)
        args = []
        for i, a in enumerate(args_):
            if isinstance(a, torch.Tensor):
                if self.view_strides is not None and i - n_epi == self.view_operand:
                    # the plan was made for this strided view (a convolution activation)
                    if tuple(a.stride()) != self.view_strides:
                        raise RuntimeError(f"{self.__name__}: activation strides {tuple(a.stride())} differ from the "
                                           f"plan's {self.view_strides}")
                elif not a.is_contiguous():
                    a = a.contiguous()
            args.append(a)
        if len(args) != n_epi + len(self.args):
            raise RuntimeError(f"{self.__name__} expects {n_epi + len(self.args)} arguments, got {len(args)}")
        device = args[-1].device
        if device.type != "cuda":
            raise RuntimeError(f"{self.__name__} runs on CUDA tensors only (got {device}); there is no CPU path")
        default_stream = torch.cuda.current_stream()
        if self.stream is not None:
            self.stream.wait_stream(default_stream)
            stream = self.stream
        else:
            stream = default_stream
        with torch.cuda.stream(stream):
            ptrs, bufs, keep, sc = self._prepare(args, device)
            if self.mode == "PROFILE":
                # MODE=PROFILE: CUDA-event time of every launch, summed per fused node
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                self.plan.launch(ptrs, stream.cuda_stream, self._status_ptr(device), self._workspace_ptr(device), sc)
                e1.record(stream)
                PROFILE_EVENTS.append((self, e0, e1))
            else:
                self.plan.launch(ptrs, stream.cuda_stream, self._status_ptr(device), self._workspace_ptr(device), sc)
            if self.mode == "DEBUG":
                # MODE=DEBUG (the reference's switch, evt_fuser.py:85): finish every launch
                # before the next one so a failing node is named
                try:
                    stream.synchronize()
                except RuntimeError as e:
                    info = [(tuple(a.shape), str(a.dtype), str(a.device), a.is_contiguous(), hex(a.data_ptr()),
                             a.untyped_storage().nbytes(), a.storage_offset())
                            for a in args if isinstance(a, torch.Tensor)]
                    outs = [(k, tuple(v.shape), hex(v.data_ptr())) for k, v in bufs.items()]
                    raise RuntimeError(f"{self.__name__} [{type(self).__name__}] failed: {e}\n args={info}\n "
                                       f"ptrs={[hex(x) for x in ptrs]}\n outs={outs}\n status_ptr={hex(self._status_ptr(device))}")
                self.check_status()
            if self.stream is not None:
                for a in args:
                    if isinstance(a, torch.Tensor):
                        a.record_stream(self.stream)
            return self._collect(bufs)

    def _prepare(self, args, device):
        """Device pointers in plan order; allocates outputs (reduction targets pre-filled
        with their identity, as evt_fuser.py:217-225 zero-fills atomics targets)."""
        n_epi = len(self.input_names)
        by_name: Dict[str, torch.Tensor] = {nm: args[i] for i, nm in enumerate(self.input_names)}
        keep: list = []
        ptrs = self._main_ptrs(args[n_epi:], keep)
        bufs: Dict[str, torch.Tensor] = {}
        for s in self.slots:
            if s.role == "in":
                t = by_name[s.name]
                if t.dtype != s.dtype:
                    raise RuntimeError(f"epilogue input {s.name}: expected {s.dtype}, got {t.dtype}")
                if t.data_ptr() % 16 != 0:
                    t = t.clone()
                    keep.append(t)
                ptrs.append(t.data_ptr())
            elif s.role == "out":
                t = torch.empty(s.shape, dtype=s.dtype, device=device)
                bufs[s.name] = t
                ptrs.append(t.data_ptr())
            else:  # reduction target: fp32, pre-filled with the identity
                arena = _ACTIVE_ARENA
                t = arena.take(s.shape, device) if (arena is not None and s.init == 0.0) else None
                if t is None:
                    t = torch.full(s.shape, s.init, dtype=torch.float32, device=device)
                bufs[s.name] = t
                ptrs.append(t.data_ptr())
        sc = None
        if self.uses_rand:
            sc = runtime.evtb_scalars()
            sc.seed = self.seed
            sc.rng_offset = self.rng_offset
            self.rng_offset += (self.ir.L * self.ir.M * self.ir.N + 3) // 4
        return ptrs, bufs, keep, sc

    def _collect(self, bufs):
        results = []
        for store_name, shape, dt in zip(self.output_stores, self.output_shapes, self.output_dtypes):
            tname = self.ir.by_name(store_name).tensor.name
            t = bufs[tname]
            if t.dtype != dt:
                t = t.to(dt)
            results.append(t.view(shape))
        return results

    def time_kernel(self, args, iters: int = 20, warmup: int = 3, graph: bool = True):
        """CUDA-event time (ms per launch, list of `iters` equal entries when timed through a
        graph) of the bare kernel launches, reusing one set of output buffers (reduction targets
        are not re-initialised: timing only).  The launches are captured into one CUDA graph
        and replayed, so the host cost of a launch (tensor-map encoding, ctypes) does not bound
        the result for kernels of a few microseconds; `graph=False` times eager launches with
        an event after each."""
        args = [a.contiguous() if isinstance(a, torch.Tensor) else a for a in args]
        device = args[-1].device
        ptrs, bufs, keep, sc = self._prepare(args, device)
        status, ws = self._status_ptr(device), self._workspace_ptr(device)
        stream = torch.cuda.current_stream()
        for _ in range(warmup):
            self.plan.launch(ptrs, stream.cuda_stream, status, ws, sc)
        torch.cuda.synchronize()
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                cs = torch.cuda.current_stream().cuda_stream
                for _ in range(iters):
                    self.plan.launch(ptrs, cs, status, ws, sc)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            return [e0.elapsed_time(e1) / iters] * iters
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
        ev[0].record()
        for i in range(iters):
            self.plan.launch(ptrs, stream.cuda_stream, status, ws, sc)
            ev[i + 1].record()
        torch.cuda.synchronize()
        return [ev[i].elapsed_time(ev[i + 1]) for i in range(iters)]


class _FusedMatmulBase(FusedOpBase):
    batched = False

    def __init__(self, trace: PartitionTrace, tile: Optional[GemmTileConfig] = None):
        super().__init__(trace)
        ir = self.ir
        a_node, b_node = self.node.args[0], self.node.args[1]
        a_shape, b_shape = _shape(a_node), _shape(b_node)
        self.M, self.K = a_shape[-2], a_shape[-1]
        self.N = b_shape[-1]
        self.L = a_shape[0] if self.batched else 1
        self.dtype = _dtype(a_node)
        if self.dtype not in (torch.float16, torch.bfloat16) or _dtype(b_node) != self.dtype:
            raise NotImplementedError(f"GEMM operands must both be fp16 or bf16, got {self.dtype}/{_dtype(b_node)}")
        self.operand_modes = []
        mats = []
        for i, spec in enumerate(trace.operands):
            if spec.needs_copy:
                # materialise [.., M, K] (A) or [.., K, N] (B) with the inner dim padded to 8
                inner = self.K if i == 0 else self.N
                outer = self.M if i == 0 else self.K
                inner_p = (inner + 7) // 8 * 8
                major = "K" if i == 0 else "MN"
                self.operand_modes.append(("copy", inner, inner_p))
                mats.append((major, inner_p, inner_p * outer))
            else:
                self.operand_modes.append(("direct",))
                mats.append((spec.major, spec.stride_outer, spec.stride_batch))
        self.a_major, self.b_major = mats[0][0], mats[1][0]
        import copy
        self.tune_key = tuning.key_for(ir, self.M, self.N, self.K, self.L, self.a_major, self.b_major, self.dtype)
        if tile is not None:
            self.tile = copy.copy(tile)
        elif trace.attrs.get("row_resident"):
            # whole rows per CTA (128 x 512 accumulator): a short ring, many epilogue warps
            self.tile = GemmTileConfig(bn=512, stages=2, epi_warps=16, row_resident=True)
        else:
            self.tile = tuning.lookup(self.tune_key) or pick_gemm_tile(self.M, self.N, self.K, self.L, self.b_major, _sm_count())
        if self.b_major == "MN" and self.tile.bn % 64 != 0:
            raise ValueError("MN-major B needs tile_n % 64 == 0")
        src, epi, entry = codegen.gemm_source(ir, self.a_major, self.b_major, self.dtype, self.tile)
        self.source = src
        self.slots = epi.slots
        self.uses_rand = epi.uses_rand
        self.image = jit.compile_cubin(src)
        d = runtime.evtb_desc()
        d.kind = runtime.EVTB_BGEMM if self.batched else runtime.EVTB_GEMM
        d.dtype = _DT[self.dtype]
        d.M, d.N, d.K, d.L = self.M, self.N, self.K, self.L
        d.a.major = runtime.EVTB_MAJOR_K if self.a_major == "K" else runtime.EVTB_MAJOR_MN
        d.a.stride_outer, d.a.stride_batch = mats[0][1], mats[0][2]
        d.b.major = runtime.EVTB_MAJOR_K if self.b_major == "K" else runtime.EVTB_MAJOR_MN
        d.b.stride_outer, d.b.stride_batch = mats[1][1], mats[1][2]
        d.tile_n = self.tile.bn
        d.stages = self.tile.stages
        d.threads = self.tile.threads
        d.smem_bytes = codegen.gemm_smem_bytes(self.tile)
        d.n_epilogue_ptrs = len(self.slots)
        d.image_path = self.image.encode()
        d.entry = entry.encode()
        d.sm_count = 0
        d.split_k = self.tile.split_k
        d.cta_pair = 1 if self.tile.cta_pair else 0
        d.row_resident = 1 if self.tile.row_resident else 0
        d.n_tma_stores = len(epi.tma_stores)
        for i, ts in enumerate(epi.tma_stores):
            d.tma_stores[i].slot, d.tma_stores[i].stride_row, d.tma_stores[i].stride_batch = ts.slot, ts.stride_row, ts.stride_batch
        self.desc = d
        self.plan = runtime.Plan(d) if torch.cuda.is_available() else None
        self._workspace = None

    def _workspace_ptr(self, device) -> int:
        """Split-K scratch (fp32 partial tiles + arrival counters), allocated and zero-filled
        once per fused node; launches of one node are ordered on one stream."""
        if self.plan is None or self.plan.workspace_bytes == 0:
            return 0
        if self._workspace is None or self._workspace.device != device:
            self._workspace = torch.zeros((self.plan.workspace_bytes + 3) // 4, dtype=torch.int32, device=device)
        return self._workspace.data_ptr()

    @property
    def flops(self) -> float:
        return 2.0 * self.L * self.M * self.N * self.K

    def _main_ptrs(self, main_tensors, keep):
        if self.plan is None:
            raise RuntimeError("no CUDA device: the fused GEMM has no CPU path")
        ptrs = []
        for t, mode in zip(main_tensors, self.operand_modes):
            if t.dtype != self.dtype:
                raise RuntimeError(f"GEMM operand dtype {t.dtype} != {self.dtype}")
            if mode[0] == "copy":
                _, inner, inner_p = mode
                if inner_p != inner:
                    t = torch.nn.functional.pad(t, (0, inner_p - inner))
                t = t.contiguous()
                keep.append(t)
            if t.data_ptr() % 16 != 0:
                t = t.clone()
                keep.append(t)
            ptrs.append(t.data_ptr())
        return ptrs


class FusedGEMM(_FusedMatmulBase):
    """epilogue(A @ B)   (reference: FusedGEMM, evt_fuser.py:453-558)"""
    __name__ = "evt_b200_gemm_with_visitor"
    target = torch.ops.aten.mm
    mainloop_fusion_targets = [torch.ops.aten.permute]
    batched = False


class FusedBMM(_FusedMatmulBase):
    """epilogue(bmm(A, B)) with operand permutes folded into TMA strides
    (reference: FusedBMM, evt_fuser.py:561-697; stride baking in python/gtl/ops/bmm.py:36-56)"""
    __name__ = "evt_b200_bmm_with_visitor"
    target = torch.ops.aten.bmm
    mainloop_fusion_targets = [torch.ops.aten.permute]
    batched = True


class _FusedRowBase(FusedOpBase):
    """Softmax / LayerNorm family: one generated row kernel (reference: the reduce-apply
    wrappers, evt_fuser.py:700-970, and python/gtl/ops/reduce_apply_operation.py)."""
    kind = ""
    plan_kind = -1
    max_vpt = 4

    def __init__(self, trace: PartitionTrace, row_config: Optional[codegen.RowKernelConfig] = None):
        super().__init__(trace)
        ir = self.ir
        self.rows, self.cols = ir.M, ir.N
        self.dtype = _dtype(self.args[0])
        if self.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            raise NotImplementedError(f"row kernel on {self.dtype}")
        self.tune_key = tuning.key_for_node("row", ir, (self.rows, self.cols), self.dtype)
        self.cfg = row_config or self._tuned_row_config() or codegen.pick_row_config(self.cols, self.max_vpt)
        self.eps = trace.attrs.get("eps", 1e-12)
        gamma_dtype = None
        if self.kind == "layernorm_backward" and len(self.args) > 4 and self.args[4] is not None:
            gamma_dtype = _dtype(self.args[4])
        src, epi, entry = codegen.row_kernel_source(self.kind, ir, self.dtype, self.cfg, self.eps, gamma_dtype)
        self.source = src
        self.slots = epi.slots
        self.uses_rand = epi.uses_rand
        self.image = jit.compile_cubin(src)
        d = runtime.evtb_desc()
        d.kind = self.plan_kind
        d.dtype = _DT[self.dtype]
        d.M, d.N, d.K, d.L = self.rows, self.cols, 1, 1
        d.threads = self.cfg.threads
        d.smem_bytes = self.cfg.smem_bytes
        d.rows_per_cta = self.cfg.rows_per_cta
        d.n_epilogue_ptrs = len(self.slots)
        d.image_path = self.image.encode()
        d.entry = entry.encode()
        self.desc = d
        self.plan = runtime.Plan(d) if torch.cuda.is_available() else None
        self._aux = {}

    def _tuned_row_config(self):
        e = tuning.lookup_config(self.tune_key)
        if e is None:
            return None
        return codegen.RowKernelConfig(tpr=int(e["tpr"]), vpt=int(e["vpt"]), threads=int(e["threads"]), vec=self.cols % 8 == 0)

    def _main_ptrs(self, main_tensors, keep):
        if self.plan is None:
            raise RuntimeError("no CUDA device: the fused row kernel has no CPU path")
        ptrs = []
        for t in main_tensors:
            if t is None:
                ptrs.append(0)
                continue
            if t.data_ptr() % 16 != 0:
                t = t.clone()
                keep.append(t)
            ptrs.append(t.data_ptr())
        return ptrs

    @property
    def bytes_moved(self) -> float:
        """algorithmic bytes: main operands read once, every epilogue tensor once"""
        eb = {torch.float16: 2, torch.bfloat16: 2, torch.float32: 4, torch.bool: 1, torch.uint8: 1, torch.int64: 8}
        n_main = {"softmax": 1, "softmax_backward": 2, "layernorm": 1, "layernorm_backward": 2}[self.kind]
        total = n_main * self.rows * self.cols * eb[self.dtype]
        for s in self.slots:
            total += math.prod(s.shape) * eb.get(s.dtype, 4)
        return float(total)


class FusedSoftmax(_FusedRowBase):
    """epilogue(softmax(x, -1))   (reference: FusedSoftmax, evt_fuser.py:700-762)"""
    __name__ = "evt_b200_softmax_with_visitor"
    target = torch.ops.aten._softmax
    kind = "softmax"
    plan_kind = runtime.EVTB_SOFTMAX
    max_vpt = 4
    # set to True to keep the per-row max and sum of exp of the last call in
    # `self.row_max` / `self.row_sum` (fp32); a loss can be formed from them without
    # another pass over the logits
    keep_row_stats = False

    def _main_ptrs(self, main_tensors, keep):
        ptrs = super()._main_ptrs(main_tensors, keep)
        if self.keep_row_stats:
            x = main_tensors[0]
            self.row_max = torch.empty(self.rows, dtype=torch.float32, device=x.device)
            self.row_sum = torch.empty(self.rows, dtype=torch.float32, device=x.device)
            return ptrs + [self.row_max.data_ptr(), self.row_sum.data_ptr()]
        return ptrs + [0, 0]


class FusedSoftmaxBackward(_FusedRowBase):
    """epilogue(y * (g - sum(g * y)))   (reference: FusedSoftmaxBackward, evt_fuser.py:765-826)"""
    __name__ = "evt_b200_softmax_backward_with_visitor"
    target = torch.ops.aten._softmax_backward_data
    kind = "softmax_backward"
    plan_kind = runtime.EVTB_SOFTMAX_BWD
    max_vpt = 2


class FusedLayerNorm(_FusedRowBase):
    """epilogue((x - mean) * rstd) plus mean / rstd per row
    (reference: FusedLayerNorm, evt_fuser.py:829-902)"""
    __name__ = "evt_b200_layernorm_with_visitor"
    target = torch.ops.aten.native_layer_norm
    kind = "layernorm"
    plan_kind = runtime.EVTB_LAYERNORM
    max_vpt = 4

    def _main_ptrs(self, main_tensors, keep):
        ptrs = super()._main_ptrs(main_tensors, keep)
        x = main_tensors[0]
        stat_shape = tuple(x.shape[:-1]) + (1,)
        mean = torch.empty(stat_shape, dtype=torch.float32, device=x.device)
        rstd = torch.empty(stat_shape, dtype=torch.float32, device=x.device)
        self._aux = {"aux_mean": mean, "aux_rstd": rstd}
        return ptrs + [mean.data_ptr(), rstd.data_ptr()]

    def _collect(self, bufs):
        results = []
        for store_name, shape, dt in zip(self.output_stores, self.output_shapes, self.output_dtypes):
            if store_name in ("aux_mean", "aux_rstd"):
                t = self._aux[store_name]
                results.append(t if t.dtype == dt else t.to(dt))
                continue
            tname = self.ir.by_name(store_name).tensor.name
            t = bufs[tname]
            if t.dtype != dt:
                t = t.to(dt)
            results.append(t.view(shape))
        return results


class FusedLayerNormBackward(_FusedRowBase):
    """epilogue(dx of LayerNorm); operands [grad, x, mean, invstd, gamma]
    (reference: FusedLayerNormBackward, evt_fuser.py:905-970)"""
    __name__ = "evt_b200_layernorm_backward_with_visitor"
    target = torch.ops.aten.native_layer_norm_backward
    kind = "layernorm_backward"
    plan_kind = runtime.EVTB_LAYERNORM_BWD
    max_vpt = 2

    def _main_ptrs(self, main_tensors, keep):
        fixed = []
        for i, t in enumerate(main_tensors):
            if i in (2, 3) and t is not None and t.dtype != torch.float32:
                t = t.to(torch.float32)
                keep.append(t)
            fixed.append(t)
        return super()._main_ptrs(fixed, keep)


class FusedSpmm(FusedOpBase):
    """epilogue(A_csr @ X); operands [crow, col, val | dinv, X]
    (reference: FusedSpmm, evt_fuser.py:973-1035; python/gtl/ops/spmm.py:114-157)"""
    __name__ = "evt_b200_spmm_with_visitor"
    target = "spmm"

    def __init__(self, trace: PartitionTrace, spmm_config: Optional[codegen.SpmmConfig] = None):
        super().__init__(trace)
        ir = self.ir
        crow, col, w, x = self.args
        self.rows, self.F = ir.M, ir.N
        self.nnz = _shape(col)[0]
        self.dtype = _dtype(x)
        self.fused_norm = bool(trace.attrs.get("fused_norm", False))
        if _dtype(crow) != torch.int32 or _dtype(col) != torch.int32:
            raise NotImplementedError("SpMM needs int32 CSR indices")
        self.tune_key = tuning.key_for_node("spmm", ir, (self.rows, self.F, self.nnz), self.dtype)
        self.cfg = spmm_config or codegen.pick_spmm_config(self.F)
        e = None if spmm_config else tuning.lookup_config(self.tune_key)
        if e is not None:
            for f in ("t_long", "task_len", "u_short", "u_long", "min_ctas"):
                setattr(self.cfg, f, int(e[f]))
        src, epi, entry = codegen.spmm_source(ir, self.dtype, self.cfg, self.fused_norm)
        self.source = src
        self.slots = epi.slots
        self.uses_rand = epi.uses_rand
        self.image = jit.compile_cubin(src)
        d = runtime.evtb_desc()
        d.kind = runtime.EVTB_SPMM
        d.dtype = _DT[self.dtype]
        d.M, d.N, d.K, d.L = self.rows, self.F, self.nnz, 1
        d.threads = self.cfg.threads
        d.smem_bytes = 0
        d.rows_per_cta = self.cfg.t_long
        d.stages = self.cfg.task_len
        d.tile_n = self.cfg.f_pad
        d.n_epilogue_ptrs = len(self.slots)
        d.image_path = self.image.encode()
        d.entry = entry.encode()
        self.desc = d
        self.plan = runtime.Plan(d) if torch.cuda.is_available() else None
        self._workspace = None

    def _workspace_ptr(self, device) -> int:
        if self._workspace is None or self._workspace.device != device:
            self._workspace = torch.zeros((self.plan.workspace_bytes + 3) // 4 + 4, dtype=torch.int32, device=device)
        return self._workspace.data_ptr()

    def _main_ptrs(self, main_tensors, keep):
        if self.plan is None:
            raise RuntimeError("no CUDA device: the fused SpMM has no CPU path")
        crow, col, w, x = main_tensors
        if w.dtype != torch.float32:
            w = w.to(torch.float32)
            keep.append(w)
        if col.shape[0] != self.nnz:
            raise RuntimeError(f"SpMM plan was built for {self.nnz} nonzeros, got {col.shape[0]}")
        wp = w.data_ptr()
        if x.data_ptr() % 32 != 0:           # fp32 feature rows are gathered with 256-bit loads
            x = x.clone()
            keep.append(x)
        return [crow.data_ptr(), col.data_ptr(), 0 if self.fused_norm else wp, wp if self.fused_norm else 0, x.data_ptr()]

    @property
    def bytes_moved(self) -> float:
        """compulsory bytes: CSR once, X once, every epilogue tensor once"""
        eb = {torch.float16: 2, torch.bfloat16: 2, torch.float32: 4, torch.bool: 1, torch.uint8: 1}
        total = 4 * (self.rows + 1) + self.nnz * (4 + (0 if self.fused_norm else 4)) + (4 * self.rows if self.fused_norm else 0)
        total += self.rows * self.F * eb[self.dtype]
        for s in self.slots:
            total += math.prod(s.shape) * eb.get(s.dtype, 4)
        return float(total)


class _FusedConvBase(FusedOpBase):
    """NHWC implicit-GEMM convolution + epilogue over the (positions, channels) result matrix."""
    dgrad = False

    def __init__(self, trace: PartitionTrace, conv_tile: Optional[codegen.ConvTileConfig] = None):
        super().__init__(trace)
        a = trace.attrs
        act, w = self.args
        self.dtype = _dtype(act)
        if self.dtype not in (torch.float16, torch.bfloat16) or _dtype(w) != self.dtype:
            raise NotImplementedError(f"convolution operands must both be fp16 or bf16, got {self.dtype}/{_dtype(w)}")
        if a["groups"] != 1 or a["transposed"]:
            raise NotImplementedError("grouped / transposed convolutions are not fused")
        K, R, S, C = _shape(w)
        if self.dgrad:
            N, P, Q, K2 = _shape(act)
            _, H, W, C2 = a["input_shape"]
        else:
            N, H, W, C2 = _shape(act)
            P, Q = _conv_out_hw(H, W, R, S, a["stride"], a["padding"], a["dilation"])
            K2 = K
        if K2 != K or C2 != C:
            raise ValueError("convolution operand shapes do not agree")
        self.geom = dict(N=N, H=H, W=W, C=C, K=K, R=R, S=S, P=P, Q=Q, stride_h=a["stride"][0], stride_w=a["stride"][1],
                         pad_h=a["padding"][0], pad_w=a["padding"][1], dil_h=a["dilation"][0], dil_w=a["dilation"][1])
        nt = C if self.dgrad else K
        if not self.dgrad:
            self.view_operand, self.view_strides = 0, _view_strides(act)
        if C % 64 or K % 64:
            raise NotImplementedError("fused convolutions need channel counts that are multiples of 64 "
                                      "(a few-channel stem is passed as a 64-wide window view, ops.stem_window)")
        import copy
        g = self.geom
        self.tune_key = tuning.key_for_node("conv_dgrad" if self.dgrad else "conv_fprop", self.ir,
                                            [g[k] for k in ("N", "H", "W", "C", "K", "R", "S", "stride_h", "pad_h")], self.dtype)
        e = None if conv_tile else tuning.lookup_config(self.tune_key)
        if conv_tile:
            self.tile = copy.copy(conv_tile)
        elif e is not None:
            self.tile = codegen.ConvTileConfig(bn=int(e["bn"]), stages=int(e["stages"]), epi_warps=int(e["epi_warps"]))
        else:
            self.tile = codegen.ConvTileConfig(bn=256 if nt >= 256 else 128 if nt >= 128 else 64)
        src, epi, entry = codegen.conv_source(self.ir, self.dgrad, self.dtype, self.tile)
        self.source = src
        self.slots = epi.slots
        self.uses_rand = epi.uses_rand
        self.image = jit.compile_cubin(src)
        d = runtime.evtb_desc()
        d.kind = runtime.EVTB_CONV_DGRAD if self.dgrad else runtime.EVTB_CONV_FPROP
        d.dtype = _DT[self.dtype]
        d.M, d.N, d.K, d.L = self.ir.M, self.ir.N, (K if self.dgrad else C) * R * S, 1
        d.tile_n = self.tile.bn
        d.stages = self.tile.stages
        d.threads = self.tile.threads
        d.smem_bytes = codegen.conv_smem_bytes(self.tile)
        d.n_epilogue_ptrs = len(self.slots)
        d.image_path = self.image.encode()
        d.entry = entry.encode()
        for k, v in self.geom.items():
            setattr(d.conv, k, int(v))
        if self.view_strides is not None:
            d.conv.x_stride_n, d.conv.x_stride_h, d.conv.x_stride_w = self.view_strides[:3]
        self.desc = d
        self.plan = runtime.Plan(d) if torch.cuda.is_available() else None

    @property
    def flops(self) -> float:
        g = self.geom
        return 2.0 * g["N"] * g["P"] * g["Q"] * g["K"] * g["C"] * g["R"] * g["S"]

    def _main_ptrs(self, main_tensors, keep):
        if self.plan is None:
            raise RuntimeError("no CUDA device: the fused convolution has no CPU path")
        act, w = main_tensors
        if act.dtype != self.dtype or w.dtype != self.dtype:
            raise RuntimeError(f"convolution operand dtype {act.dtype}/{w.dtype} != {self.dtype}")
        return [act.data_ptr(), w.data_ptr()]


class FusedConvFprop(_FusedConvBase):
    """epilogue(conv(x, w)); operands [x (N,H,W,C), w (K,R,S,C)] (reference: FusedConvFprop,
    evt_fuser.py:282-362)"""
    __name__ = "evt_b200_conv2d_fprop_with_visitor"
    target = "convolution_forward_channel_last"
    dgrad = False


class FusedConvDgrad(_FusedConvBase):
    """epilogue(conv_backward_data(dy, w)); operands [dy (N,P,Q,K), w (K,R,S,C)] (reference:
    FusedConvDgrad, evt_fuser.py:365-450)"""
    __name__ = "evt_b200_conv2d_dgrad_with_visitor"
    target = "convolution_backward_data_channel_last"
    dgrad = True


class FusedConvWgrad(FusedOpBase):
    """epilogue(conv_backward_weight(dy, x)) as the [K, R*S*C] matrix of the channels-last filter
    gradient; operands [dy (N,P,Q,K), x (N,H,W,C)].  The reference leaves this leaf to cuDNN
    (convolution_backward_weight_channel_last, pass_decomposition.py:92-107); here it is an implicit
    GEMM over boxes of output positions, cut along that reduction so that every SM has a share."""
    __name__ = "evt_b200_conv2d_wgrad_with_visitor"
    target = "convolution_backward_weight_channel_last"

    def __init__(self, trace: PartitionTrace, tile: Optional[GemmTileConfig] = None):
        super().__init__(trace)
        a = trace.attrs
        dy, x = self.args
        self.dtype = _dtype(dy)
        if self.dtype not in (torch.float16, torch.bfloat16) or _dtype(x) != self.dtype:
            raise NotImplementedError(f"convolution operands must both be fp16 or bf16, got {self.dtype}/{_dtype(x)}")
        if a["groups"] != 1 or a["transposed"]:
            raise NotImplementedError("grouped / transposed convolutions are not fused")
        K, R, S, C = a["filter_shape"]
        N, P, Q, K2 = _shape(dy)
        N2, H, W, C2 = _shape(x)
        if K2 != K or C2 != C or N2 != N:
            raise ValueError("convolution operand shapes do not agree")
        self.view_operand, self.view_strides = 1, _view_strides(x)
        if C % 64 or K % 8:
            raise NotImplementedError("the fused weight gradient needs C % 64 == 0 and K % 8 == 0 "
                                      "(a few-channel stem is passed as a 64-wide window view, ops.stem_window)")
        self.geom = dict(N=N, H=H, W=W, C=C, K=K, R=R, S=S, P=P, Q=Q, stride_h=a["stride"][0], stride_w=a["stride"][1],
                         pad_h=a["padding"][0], pad_w=a["padding"][1], dil_h=a["dilation"][0], dil_w=a["dilation"][1])
        import copy
        self.tune_key = tuning.key_for_node("conv_wgrad", self.ir, [N, H, W, C, K, R, S, a["stride"][0], a["padding"][0]], self.dtype)
        if tile is not None:
            self.tile = copy.copy(tile)
        else:
            e = tuning.lookup_config(self.tune_key)
            bn = int(e["bn"]) if e else (256 if C % 256 == 0 else 128 if C % 128 == 0 else 64)
            tiles = ((K + 127) // 128) * (R * S * C // bn)
            boxes = max(1, (N * P * Q) // 64)
            split = int(e["split_k"]) if e else max(1, min(_sm_count() // max(tiles, 1), boxes // 8, 64))
            self.tile = GemmTileConfig(bn=bn, stages=int(e["stages"]) if e else 6, epi_warps=int(e["epi_warps"]) if e else 8,
                                       split_k=split)
        if C % self.tile.bn:
            raise ValueError("the weight-gradient tile width must divide C")
        src, epi, entry = codegen.conv_wgrad_source(self.ir, self.dtype, self.tile)
        self.source = src
        self.slots = epi.slots
        self.uses_rand = epi.uses_rand
        self.image = jit.compile_cubin(src)
        d = runtime.evtb_desc()
        d.kind = runtime.EVTB_CONV_WGRAD
        d.dtype = _DT[self.dtype]
        d.M, d.N, d.K, d.L = K, R * S * C, N * P * Q, 1
        d.tile_n = self.tile.bn
        d.stages = self.tile.stages
        d.threads = self.tile.threads
        d.smem_bytes = codegen.gemm_smem_bytes(self.tile)
        d.n_epilogue_ptrs = len(self.slots)
        d.image_path = self.image.encode()
        d.entry = entry.encode()
        d.split_k = self.tile.split_k
        d.n_tma_stores = len(epi.tma_stores)
        for i, ts in enumerate(epi.tma_stores):
            d.tma_stores[i].slot, d.tma_stores[i].stride_row, d.tma_stores[i].stride_batch = ts.slot, ts.stride_row, ts.stride_batch
        for k, v in self.geom.items():
            setattr(d.conv, k, int(v))
        if self.view_strides is not None:
            d.conv.x_stride_n, d.conv.x_stride_h, d.conv.x_stride_w = self.view_strides[:3]
        self.desc = d
        self.plan = runtime.Plan(d) if torch.cuda.is_available() else None
        self._workspace = None

    def _workspace_ptr(self, device) -> int:
        if self.plan is None or self.plan.workspace_bytes == 0:
            return 0
        if self._workspace is None or self._workspace.device != device:
            self._workspace = torch.zeros((self.plan.workspace_bytes + 3) // 4, dtype=torch.int32, device=device)
        return self._workspace.data_ptr()

    @property
    def flops(self) -> float:
        g = self.geom
        return 2.0 * g["N"] * g["P"] * g["Q"] * g["K"] * g["C"] * g["R"] * g["S"]

    def _main_ptrs(self, main_tensors, keep):
        if self.plan is None:
            raise RuntimeError("no CUDA device: the fused weight gradient has no CPU path")
        dy, x = main_tensors
        if dy.dtype != self.dtype or x.dtype != self.dtype:
            raise RuntimeError(f"convolution operand dtype {dy.dtype}/{x.dtype} != {self.dtype}")
        return [dy.data_ptr(), x.data_ptr()]


FUSED_CLASSES = {"conv_fprop": FusedConvFprop, "conv_dgrad": FusedConvDgrad, "conv_wgrad": FusedConvWgrad, "spmm": FusedSpmm, "gemm": FusedGEMM, "bmm": FusedBMM, "softmax": FusedSoftmax,
                 "softmax_backward": FusedSoftmaxBackward, "layernorm": FusedLayerNorm,
                 "layernorm_backward": FusedLayerNormBackward}
