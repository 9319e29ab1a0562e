"""Epilogue DAG -> CUDA source.

The reference emits a C++ visitor-tree type from its DAG IR and lets NVCC/NVRTC
instantiate the CUTLASS kernel around it (python/gtl/compiler/passes/evt_fuser.py:481-518,
738-746).  Here the DAG becomes one plain struct with four inlined methods that the
hand-written kernels in `csrc/` call:

    tile_begin(c)            once per (thread, accumulator row): row offsets, per-row
                             broadcast operands, reduction identities
    visit8<G>(c, n, acc8)    8 consecutive columns of that row: loads, math, stores,
                             reduction bookkeeping
    chunk_end(c, n)          after 32 columns: [N]-vector ("row") reductions leave the warp
    tile_end(c)              [M]-vector ("column") reductions leave the thread

Problem sizes, strides and index maps are compile-time constants of the generated text, as
in the reference where every kernel is specialised to its problem (`dynamic=False`).
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .ir import EpilogueIR, Factor, Node, TensorRef

CTYPE = {
    torch.float16: "__half",
    torch.bfloat16: "__nv_bfloat16",
    torch.float32: "float",
    torch.bool: "uint8_t",
    torch.uint8: "uint8_t",
    torch.int64: "long long",
    torch.int32: "int",
}
ELEM_BYTES = {torch.float16: 2, torch.bfloat16: 2, torch.float32: 4, torch.bool: 1, torch.uint8: 1,
              torch.int64: 8, torch.int32: 4}


def DEBUG_DEFINE() -> str:
    """MODE=DEBUG (the reference's debug switch, evt_fuser.py:85) builds the epilogues with a
    bounds check on every global access; a violation is recorded in the status word and the
    access is skipped instead of faulting."""
    import os
    out = "#define EVTB_BOUNDS_CHECK 1\n" if os.environ.get("MODE", "RUN") == "DEBUG" else ""
    if os.environ.get("EVT_B200_KPROFILE", "0") == "1":
        # per-role wait counters in the GEMM kernel (Plan.set_profile_buffer reads them back)
        out += "#define EVTB_PROFILE 1\n"
    return out


def _fexpr(coord: str, f: Factor, extent: int) -> str:
    """((coord / unit) % size) * stride with the trivial parts folded away."""
    e = coord
    if f.unit != 1:
        e = f"({e} / {f.unit})"
    if f.unit * f.size < extent:
        e = f"({e} % {f.size})"
    if f.stride != 1:
        e = f"({e} * {f.stride}LL)"
    return e


def _sum(parts: List[str]) -> str:
    return " + ".join(parts) if parts else "0"


@dataclass
class OperandSlot:
    """One pointer the caller passes: order == slot number in EpiParams::ptr."""
    name: str            # tensor name (fx node name)
    role: str            # 'in' | 'out' | 'reduce'
    dtype: torch.dtype
    shape: Tuple[int, ...]
    init: Optional[float] = None   # required initial fill for reduction targets
    reduce_dtype: Optional[torch.dtype] = None   # caller-visible dtype of a reduction result


@dataclass
class TmaStore:
    """A full-tensor result that leaves through TMA: address = base + l*stride_batch + m*stride_row + n."""
    slot: int
    stride_row: int
    stride_batch: int


@dataclass
class EpilogueSource:
    struct_code: str
    slots: List[OperandSlot]
    uses_rand: bool = False
    stage_tiles: int = 0
    tma_stores: List[TmaStore] = field(default_factory=list)   # index in the list = EpiParams::tmap index


class EpilogueGenerator:
    def __init__(self, ir: EpilogueIR, struct_name: str = "Epi", row_tile: int = 128, col_group: int = 32,
                 staged: bool = False, max_stage_tiles: int = 8, tma_store: bool = False,
                 defer_col_reductions: bool = False, double_buffer: bool = False):
        """row_tile: rows a CTA covers per step (a row predicate is needed unless M is a
        multiple of it; 0 = always predicate); col_group: columns the kernel guarantees to be
        in range whenever it calls visit8 with an in-range first column."""
        self.ir = ir
        self.struct_name = struct_name
        self.slots: List[OperandSlot] = []
        self.slot_of: Dict[str, int] = {}
        self.members: List[str] = []
        self.begin: List[str] = []
        self.body_pre: List[str] = []     # per 8-group, before the element loop (vector loads)
        self.body_elem: List[str] = []    # inside `for j` element loop
        self.body_post: List[str] = []    # per 8-group, after the loop (vector stores)
        self.chunk_end: List[str] = []
        self.end: List[str] = []
        self.methods: List[str] = []      # extra member functions (flush of deferred reductions)
        # [N]-vector reductions of a tensor-core kernel (32-column chunks, per-warp staging memory) may
        # collect a column strip's partial results before they go to global memory
        self.defer_col_reductions = defer_col_reductions and col_group == 32
        # two sets of staging tiles used by alternate chunks: the pack of chunk i + 1 does not wait for
        # the copy engine to finish reading chunk i's tiles
        self.double_buffer = double_buffer
        self.deferred = 0
        self.finish: List[str] = []       # once per warp after its last tile
        self.uses_rand = False
        # predicates known at generation time disappear from the code
        self.staged = staged
        self.max_stage_tiles = max_stage_tiles
        self.stage_tiles = 0            # staging tiles (2 KB each) one epilogue warp needs
        self.chunk_begin: List[str] = []
        self.chunk_stores: List[str] = []
        # results with a linear (batch, row, column) address leave their staging tile through a
        # TMA bulk store instead of per-lane global stores (GEMM kernels only, at most 4)
        self.tma_store = tma_store and os.environ.get("MODE", "RUN") != "DEBUG"
        self.tma_stores: List[TmaStore] = []
        self.tma_issue: List[str] = []
        # A staged result may reuse the staging tile of a staged aux load: within one 8-column
        # group a thread reads its 16 bytes of every load tile before it writes the same 16 bytes
        # of a result tile.  With TMA stores the next chunk's aux loads must then wait until the
        # copy engine has read the tile.
        self.load_tiles_free: List[int] = []
        self.alias_wait = False
        # row-wise reduce-apply step fused into a row-resident GEMM: the nodes it depends on are
        # generated twice, once into the statistics pass and once into the apply pass
        self.rowop: Optional[Node] = None
        self.stat_pre: List[str] = []
        self.stat_elem: List[str] = []
        self.stat_post: List[str] = []
        self.merge: List[str] = []
        self.stat_ab = ("0.f", "0.f")
        # optional second statistics pass (softmax: exponentials written back to tensor memory)
        self.stat1_elem: List[str] = []
        self.merge1: List[str] = []
        self.stat1_ab = ("0.f", "0.f")
        self.write_back = False
        self.pre_marks: List[Tuple[int, int, int, int]] = []   # body_pre / body_elem ranges of the row step's inputs
        self.rows_full = bool(row_tile and ir.M % row_tile == 0)
        self.ROW_OK = "true" if (row_tile and ir.M % row_tile == 0) else "c.row_ok"
        self.full_cols = ir.N % col_group == 0

    def _col_ok(self, expr: str) -> str:
        return "true" if self.full_cols else f"({expr} < {self.ir.N})"

    # -- operand slots ------------------------------------------------------------------
    def _slot(self, t: TensorRef, role: str, init=None, dtype=None, reduce_dtype=None) -> int:
        key = f"{role}:{t.name}"
        if key in self.slot_of:
            return self.slot_of[key]
        idx = len(self.slots)
        self.slots.append(OperandSlot(t.name, role, dtype or t.dtype, t.shape, init, reduce_dtype))
        self.slot_of[key] = idx
        return idx

    # -- index-map helpers --------------------------------------------------------------
    def _extent(self, axis: str) -> int:
        return {"l": self.ir.L, "m": self.ir.M, "n": self.ir.N}[axis]

    def _row_offset(self, t: TensorRef, m: str = "c.m", l: str = "c.l") -> str:
        parts = []
        for f in t.factors:
            if f.axis == "l":
                parts.append(_fexpr(f"(long long){l}", f, self.ir.L))
            elif f.axis == "m":
                parts.append(_fexpr(f"(long long){m}", f, self.ir.M))
        return _sum(parts)

    def _can_stage_shape(self, t: TensorRef) -> bool:
        return (self.staged and self._vec_ok(t) and t.dtype in (torch.float16, torch.bfloat16)
                and "m" in t.axes_used())

    def _can_stage(self, t: TensorRef) -> bool:
        """Full tensors of a 16-bit type go through the warp staging tile (coalesced
        global access); everything else keeps the direct per-row path."""
        return self.stage_tiles < self.max_stage_tiles and self._can_stage_shape(t)

    def _stage_copy_loop(self, body: List[str]) -> List[str]:
        out = ["#pragma unroll", "for (int i = 0; i < 4; ++i) {",
               "  const int row = i * 8 + (c.lane >> 2), seg = c.lane & 3;",
               "  const int m = EVTB_ROW_M(c, row), nn = n + seg * 8;"]
        out += ["  " + b for b in body]
        out.append("}")
        return out

    def _col_offset(self, t: TensorRef, n: str) -> str:
        parts = [_fexpr(f"(long long)({n})", f, self.ir.N) for f in t.factors if f.axis == "n"]
        return _sum(parts)

    def _owner_pred(self, t: TensorRef, axes=("l", "m"), m: str = "c.m", l: str = "c.l") -> str:
        """True for the one thread among those that alias the same element (broadcast
        values stored from the epilogue are written once)."""
        conds = []
        for axis, coord in (("l", l), ("m", m)):
            if axis not in axes:
                continue
            fs = [f for f in t.factors if f.axis == axis]
            ext = self._extent(axis)
            covered = 1
            for f in fs:
                covered *= f.size
            if covered == ext:
                continue
            if not fs:
                conds.append(f"({coord} == 0)")
            else:
                rebuilt = " + ".join(f"(({coord} / {f.unit}) % {f.size}) * {f.unit}" for f in fs)
                conds.append(f"({coord} == {rebuilt})")
        return " && ".join(conds) if conds else "true"

    def _vec_ok(self, t: TensorRef) -> bool:
        """8 consecutive columns (start % 8 == 0) are 8 consecutive, aligned elements."""
        nf = [f for f in t.factors if f.axis == "n"]
        if not nf:
            return False
        inner = min(nf, key=lambda f: f.unit)
        if inner.unit != 1 or inner.stride != 1 or inner.size % 8 != 0:
            return False
        if self.ir.N % 8 != 0:
            return False
        for f in t.factors:
            if f is inner:
                continue
            if f.stride % 8 != 0:
                return False
        if t.dtype not in (torch.float16, torch.bfloat16, torch.float32, torch.bool, torch.uint8):
            return False
        return True

    # -- generation -----------------------------------------------------------------------
    def generate(self) -> EpilogueSource:
        ir = self.ir
        val: Dict[str, str] = {}   # IR node -> C expression valid inside the element loop
        rowops = [n for n in ir.nodes if n.kind == "rowop"]
        if len(rowops) > 1:
            raise NotImplementedError("one row-wise step per fused GEMM")
        pre: set = set()
        if rowops:
            stack = list(rowops[0].args)
            by_name = {n.name: n for n in ir.nodes}
            while stack:
                x = stack.pop()
                if x in pre:
                    continue
                pre.add(x)
                stack.extend(by_name[x].args)
        # the inputs of the row-wise step can be dropped from the apply pass (softmax written back
        # to tensor memory) only if nothing else reads them and none of them is a staged load
        self.pre_private = bool(rowops) and all(
            all(u.name in pre or u is rowops[0] for u in ir.nodes if x in u.args)
            for x in pre if by_name[x].kind != "accum")
        for node in ir.nodes:
            k = node.kind
            mark = (len(self.body_pre), len(self.body_elem), len(self.chunk_begin))
            self._gen_node(node, val)
            if node.name in pre:
                self.stat_pre += self.body_pre[mark[0]:]
                self.stat_elem += self.body_elem[mark[1]:]
                self.pre_marks.append((mark[0], len(self.body_pre), mark[1], len(self.body_elem)))
                if len(self.chunk_begin) != mark[2]:
                    self.pre_private = False
        code = self._assemble()
        return EpilogueSource(code, self.slots, self.uses_rand, self.stage_tiles * (2 if self.double_buffer else 1), self.tma_stores)

    def _gen_node(self, node: Node, val: Dict[str, str]):
        ir = self.ir
        if True:
            k = node.kind
            if k == "accum":
                val[node.name] = "acc[j]"
            elif k == "const":
                v = float(node.value)
                if v == float("inf"):
                    val[node.name] = "INFINITY"
                elif v == float("-inf"):
                    val[node.name] = "(-INFINITY)"
                else:
                    val[node.name] = f"{v!r}f" if ("e" in repr(v) or "." in repr(v)) else f"{v!r}.0f"
            elif k == "load":
                val[node.name] = self._gen_load(node)
            elif k == "rand":
                self.uses_rand = True
                self.body_pre.append(f"float r_{node.name}[8];")
                self.body_pre.append(
                    f"rand8(c.ep->seed, c.ep->rng_offset, ((unsigned long long)c.l * {ir.M}ULL + (unsigned long long)c.m) * {ir.N}ULL + (unsigned long long)n, r_{node.name});")
                val[node.name] = f"r_{node.name}[j]"
            elif k == "compute":
                expr = self._compute_expr(node, val)
                self.body_elem.append(f"const float v_{node.name} = {expr};")
                val[node.name] = f"v_{node.name}"
            elif k == "store":
                self._gen_store(node, val)
            elif k == "reduce":
                self._gen_reduce(node, val)
            elif k == "rowop":
                val[node.name] = self._gen_rowop(node, val)
            else:
                raise NotImplementedError(k)

    def _gen_rowop(self, node: Node, val: Dict[str, str]) -> str:
        """Statistics pass + apply expression of a row-wise step (softmax / softmax backward) that
        runs over the accumulator row held in tensor memory."""
        self.rowop = node
        nm = node.name
        a = [val[x] for x in node.args]
        colok = self._col_ok("n + j")
        if node.op == "softmax" and self.pre_private:
            # pass 0: row maximum.  pass 1: e = exp(v - max), row sum, e written back over the
            # accumulator.  apply: e / sum.  One exponential per element.
            self.members += ["float st_m;", "float st_s;", "float st_inv;"]
            self.begin += ["st_m = -INFINITY;", "st_s = 0.f;", "st_inv = 0.f;"]
            self.stat1_elem = list(self.stat_elem) + [
                f"const float e_{nm} = {colok} ? __expf(({a[0]}) - st_m) : 0.f;",
                f"st_s += e_{nm};",
                f"acc[j] = e_{nm};"]
            self.stat_elem.append(f"st_m = fmaxf(st_m, {colok} ? ({a[0]}) : -INFINITY);")
            self.stat_ab = ("st_m", "0.f")
            self.merge += ["float m = pa[0];", "for (int i = 1; i < cnt; ++i) m = fmaxf(m, pa[i]);",
                           "st_m = m > -INFINITY ? m : 0.f;"]
            self.stat1_ab = ("st_s", "0.f")
            self.merge1 += ["float sum = 0.f;", "for (int i = 0; i < cnt; ++i) sum += pa[i];",
                            "st_inv = sum > 0.f ? 1.f / sum : 0.f;"]
            self.write_back = True
            # the apply pass reads the exponentials: drop the code of the step's inputs from it
            for b0, b1, e0, e1 in reversed(self.pre_marks):
                del self.body_pre[b0:b1]
                del self.body_elem[e0:e1]
            self.body_elem.append(f"const float v_{nm} = acc[j] * st_inv;")
            return f"v_{nm}"
        if node.op == "softmax":
            self.members += ["float st_m;", "float st_s;", "float st_inv;"]
            self.begin += ["st_m = -INFINITY;", "st_s = 0.f;", "st_inv = 0.f;"]
            self.stat_pre.append("float sv[8];")
            self.stat_elem.append(f"sv[j] = {colok} ? ({a[0]}) : -INFINITY;")
            self.stat_post += [
                "float gm = sv[0];",
                "#pragma unroll",
                "for (int j = 1; j < 8; ++j) gm = fmaxf(gm, sv[j]);",
                "const float mn = fmaxf(st_m, gm);",
                "if (mn > -INFINITY) {   // online update of (row maximum, sum of exponentials)",
                "  float add = 0.f;",
                "#pragma unroll",
                "  for (int j = 0; j < 8; ++j) add += __expf(sv[j] - mn);",
                "  st_s = st_s * __expf(st_m - mn) + add;",
                "  st_m = mn;",
                "}"]
            self.stat_ab = ("st_m", "st_s")
            self.merge += [
                "float m = pa[0];",
                "for (int i = 1; i < cnt; ++i) m = fmaxf(m, pa[i]);",
                "float sum = 0.f;",
                "for (int i = 0; i < cnt; ++i) sum += (pa[i] > -INFINITY) ? pb[i] * __expf(pa[i] - m) : 0.f;",
                "st_m = m;",
                "st_inv = sum > 0.f ? 1.f / sum : 0.f;"]
            self.body_elem.append(f"const float v_{nm} = __expf({a[0]} - st_m) * st_inv;")
        elif node.op == "softmax_backward":
            self.members += ["float st_t;"]
            self.begin += ["st_t = 0.f;"]
            self.stat_elem.append(f"st_t += {colok} ? ({a[0]}) * ({a[1]}) : 0.f;")
            self.stat_ab = ("st_t", "0.f")
            self.merge += ["float t = 0.f;", "for (int i = 0; i < cnt; ++i) t += pa[i];", "st_t = t;"]
            self.body_elem.append(f"const float v_{nm} = (({a[0]}) - st_t) * ({a[1]});")
        else:
            raise NotImplementedError(node.op)
        return f"v_{nm}"

    def _gen_load(self, node: Node) -> str:
        t = node.tensor
        slot = self._slot(t, "in")
        ct = CTYPE[t.dtype]
        eb = ELEM_BYTES[t.dtype]
        axes = t.axes_used()
        base = f"(const char*)c.ep->ptr[{slot}]"
        nm = node.name
        if "n" not in axes:
            # per-row (column broadcast) or scalar operand: one load per accumulator row
            self.members.append(f"float b_{nm};")
            self.begin.append(
                f"b_{nm} = ({self.ROW_OK} && EVTB_CHK(c, {self._row_offset(t)}, 1, {t.numel}LL, {slot})) ? Vec8<{ct}>::load1({base} + ({self._row_offset(t)}) * {eb}) : 0.f;")
            return f"b_{nm}"
        if self._can_stage(t):
            r = self.stage_tiles
            self.stage_tiles += 1
            self.load_tiles_free.append(r)
            row_in = "true" if self.rows_full else f"m < {self.ir.M}"
            off = f"{self._row_offset(t, 'm', 'c.l')} + {self._col_offset(t, 'nn')}"
            self.chunk_begin.append(f"{{ // {nm}: global -> staging tile {r}, 8 rows x 64 contiguous bytes per instruction")
            self.chunk_begin += ["  " + x for x in self._stage_copy_loop([
                "uint4 v = make_uint4(0u, 0u, 0u, 0u);",
                f"const long long off = {off};",
                f"if ({row_in} && {self._col_ok('nn')} && EVTB_CHK(c, off, 8, {t.numel}LL, {slot})) v = __ldg(reinterpret_cast<const uint4*>({base} + off * {eb}));",
                f"stage_write16(stg(c, {r}), row, seg, v);"])]
            self.chunk_begin.append("}")
            self.body_pre.append(f"float a_{nm}[8];")
            self.body_pre.append(f"Pack8<{ct}>::unpack(stage_read16(stg(c, {r}), c.lane, G), a_{nm});")
            return f"a_{nm}[j]"
        self.members.append(f"long long ro_{nm};")
        self.begin.append(f"ro_{nm} = {self._row_offset(t)};")
        self.body_pre.append(f"float a_{nm}[8];")
        if self._vec_ok(t):
            self.body_pre.append(
                f"Vec8<{ct}>::load({base} + (ro_{nm} + {self._col_offset(t, 'n')}) * {eb}, {self.ROW_OK} && {self._col_ok('n')} && EVTB_CHK(c, ro_{nm} + {self._col_offset(t, 'n')}, 8, {t.numel}LL, {slot}), a_{nm});")
        else:
            self.body_pre.append("#pragma unroll")
            self.body_pre.append(
                f"for (int j = 0; j < 8; ++j) a_{nm}[j] = ({self.ROW_OK} && {self._col_ok('n + j')} && EVTB_CHK(c, ro_{nm} + {self._col_offset(t, 'n + j')}, 1, {t.numel}LL, {slot})) ? "
                f"Vec8<{ct}>::load1({base} + (ro_{nm} + {self._col_offset(t, 'n + j')}) * {eb}) : 0.f;")
        return f"a_{nm}[j]"

    def _compute_expr(self, node: Node, val: Dict[str, str]) -> str:
        a = [val[x] for x in node.args]
        op = node.op
        if op == "add":
            return f"{a[0]} + {a[1]}"
        if op == "sub":
            return f"{a[0]} - {a[1]}"
        if op == "mul":
            return f"{a[0]} * {a[1]}"
        if op == "div":
            return f"{a[0]} / {a[1]}"
        if op == "neg":
            return f"-({a[0]})"
        if op == "relu":
            return f"op_relu({a[0]})"
        if op == "tanh":
            return f"op_tanh_precise({a[0]})"
        if op == "sigmoid":
            return f"op_sigmoid({a[0]})"
        if op == "exp":
            return f"__expf({a[0]})"
        if op == "rsqrt":
            return f"rsqrtf({a[0]})"
        if op == "identity":
            return a[0]
        if op == "tanh_backward":
            return f"op_tanh_backward({a[0]}, {a[1]})"
        if op == "ge":
            return f"(({a[0]} >= {a[1]}) ? 1.f : 0.f)"
        if op == "gt":
            return f"(({a[0]} > {a[1]}) ? 1.f : 0.f)"
        if op == "ne":
            return f"(({a[0]} != {a[1]}) ? 1.f : 0.f)"
        if op == "maximum":
            return f"fmaxf({a[0]}, {a[1]})"
        if op == "gelu":
            fn = "op_gelu_tanh" if node.attrs.get("approximate", "none") == "tanh" else "op_gelu_erf"
            return f"{fn}({a[0]})"
        if op == "gelu_backward":
            fn = "op_gelu_backward_tanh" if node.attrs.get("approximate", "none") == "tanh" else "op_gelu_backward_erf"
            return f"{fn}({a[0]}, {a[1]})"
        if op == "one_hot":
            return f"(((int){a[0]} == n + j) ? 1.f : 0.f)"
        raise NotImplementedError(f"compute op {op}")

    def _linear_strides(self, t: TensorRef):
        """(stride_row, stride_batch) if the tensor covers the canonical space exactly once with
        address = l * stride_batch + m * stride_row + n, else None."""
        out = {}
        for axis, ext in (("n", self.ir.N), ("m", self.ir.M), ("l", self.ir.L)):
            fs = [f for f in t.factors if f.axis == axis]
            if ext == 1:
                out[axis] = 0
                continue
            cover = 1
            ratio = None
            for f in fs:
                if f.size == 1:
                    continue
                if f.stride % f.unit != 0:
                    return None
                r = f.stride // f.unit
                if ratio is not None and r != ratio:
                    return None
                ratio = r
                cover *= f.size
            if cover != ext or ratio is None:
                return None
            # the factors must tile the axis without gaps: units are the running products of sizes
            units = sorted((f.unit, f.size) for f in fs if f.size > 1)
            run = 1
            for u, sz in units:
                if u != run:
                    return None
                run *= sz
            out[axis] = ratio
        if out["n"] != 1 and self.ir.N > 1:
            return None
        if out["m"] % 8 != 0 or out["l"] % 8 != 0:
            return None        # TMA strides are multiples of 16 bytes
        if t.numel != self.ir.L * self.ir.M * self.ir.N:
            return None
        return out["m"], out["l"]

    def _gen_store(self, node: Node, val: Dict[str, str]):
        t = node.tensor
        slot = self._slot(t, "out")
        ct = CTYPE[t.dtype]
        eb = ELEM_BYTES[t.dtype]
        nm = node.name
        base = f"(char*)c.ep->ptr[{slot}]"
        if self.load_tiles_free and self._can_stage_shape(t):
            r = self.load_tiles_free.pop(0)       # written in place over a staged aux load
            aliased = True
        elif self._can_stage(t):
            r = self.stage_tiles
            self.stage_tiles += 1
            aliased = False
        else:
            r = None
        if r is not None:
            self.body_pre.append(f"float o_{nm}[8];")
            self.body_elem.append(f"o_{nm}[j] = {val[node.args[0]]};")
            self.body_post.append(f"stage_write16(stg(c, {r}), c.lane, G, Pack8<{ct}>::pack(o_{nm}));")
            lin = self._linear_strides(t) if (self.tma_store and len(self.tma_stores) < 4) else None
            if lin is not None:
                j = len(self.tma_stores)
                self.tma_stores.append(TmaStore(slot, lin[0], lin[1]))
                self.tma_issue.append(f"tma_store_3d(&c.ep->tmap[{j}], stg(c, {r}), n, c.m_warp, c.l);   // {nm}")
                self.alias_wait = self.alias_wait or aliased
                return
            row_in = "true" if self.rows_full else f"m < {self.ir.M}"
            off = f"{self._row_offset(t, 'm', 'c.l')} + {self._col_offset(t, 'nn')}"
            self.chunk_stores.append(f"{{ // {nm}: staging tile {r} -> global, coalesced")
            self.chunk_stores += ["  " + x for x in self._stage_copy_loop([
                f"const long long off = {off};",
                f"if ({row_in} && {self._owner_pred(t, m='m', l='c.l')} && {self._col_ok('nn')} && EVTB_CHK(c, off, 8, {t.numel}LL, {slot}))",
                f"  *reinterpret_cast<uint4*>({base} + off * {eb}) = stage_read16(stg(c, {r}), row, seg);"])]
            self.chunk_stores.append("}")
            return
        self.members.append(f"long long ro_{nm};")
        self.members.append(f"bool ok_{nm};")
        self.begin.append(f"ro_{nm} = {self._row_offset(t)};")
        self.begin.append(f"ok_{nm} = {self.ROW_OK} && {self._owner_pred(t)};")
        self.body_pre.append(f"float o_{nm}[8];")
        self.body_elem.append(f"o_{nm}[j] = {val[node.args[0]]};")
        has_n = "n" in t.axes_used()
        if has_n and self._vec_ok(t):
            self.body_post.append(
                f"Vec8<{ct}>::store({base} + (ro_{nm} + {self._col_offset(t, 'n')}) * {eb}, ok_{nm} && {self._col_ok('n')} && EVTB_CHK(c, ro_{nm} + {self._col_offset(t, 'n')}, 8, {t.numel}LL, {slot}), o_{nm});")
        else:
            colpred = "" if has_n else " && (n + j == 0)"
            if has_n:
                nf = [f for f in t.factors if f.axis == "n"]
                cov = 1
                for f in nf:
                    cov *= f.size
                if cov != self.ir.N:
                    rebuilt = " + ".join(f"(((n + j) / {f.unit}) % {f.size}) * {f.unit}" for f in nf)
                    colpred = f" && ((n + j) == {rebuilt})"
            self.body_post.append("#pragma unroll")
            self.body_post.append(
                f"for (int j = 0; j < 8; ++j) if (ok_{nm} && {self._col_ok('n + j')}{colpred} && EVTB_CHK(c, ro_{nm} + {self._col_offset(t, 'n + j')}, 1, {t.numel}LL, {slot})) "
                f"Vec8<{ct}>::store1({base} + (ro_{nm} + {self._col_offset(t, 'n + j')}) * {eb}, o_{nm}[j]);")

    def _gen_reduce(self, node: Node, val: Dict[str, str]):
        t = node.tensor
        axes = node.attrs["axes"]
        nm = node.name
        opc = "SumOp" if node.op == "sum" else "MaxOp"
        ident = "0.f" if node.op == "sum" else "(-INFINITY)"
        red = "red_add_f32" if node.op == "sum" else "red_max_f32"
        # reductions accumulate in fp32 memory; the host converts to the node's dtype
        slot = self._slot(t, "reduce", init=0.0 if node.op == "sum" else float("-inf"),
                          dtype=torch.float32, reduce_dtype=t.dtype)
        base = f"(float*)c.ep->ptr[{slot}]"
        src = val[node.args[0]]
        if "m" in axes:
            # [N]-vector result: collect 32 columns, transpose-reduce over the warp's rows
            self.members.append(f"float rr_{nm}[32];")
            self.body_elem.append(
                f"rr_{nm}[G * 8 + j] = ({self.ROW_OK} && {self._col_ok('n + j')}) ? ({src}) : {ident};")
            lpart = [_fexpr("(long long)c.l", f, self.ir.L) for f in t.factors if f.axis == "l"]
            if lpart or not self.defer_col_reductions:
                off = _sum(lpart + [self._col_offset(t, "n + c.lane")])
                self.chunk_end.append("{")
                self.chunk_end.append(f"  const float r = warp_transpose_reduce32<{opc}>(rr_{nm}, c.lane);")
                self.chunk_end.append(f"  if ({self._col_ok('n + c.lane')} && EVTB_CHK(c, {off}, 1, {t.numel}LL, {slot})) {red}({base} + ({off}), r);")
                self.chunk_end.append("}")
            else:
                # A persistent CTA walks many tiles of one column strip in a row (row tiles run
                # fastest in every tile order): the warp keeps the strip's partial results -- one
                # word per lane and 32-column chunk, in its own staging memory -- and sends them to
                # global memory when the strip changes and after its last tile: one atomic per
                # column, warp and strip instead of one per tile.  With 3136 row tiles over 256
                # columns (a 1x1 convolution on 128 x 56 x 56 positions) the atomics on the 512
                # result words otherwise cost more than the convolution.
                if self.deferred % 2 == 0:
                    self.deferred_tile = self.stage_tiles
                    self.stage_tiles += 1
                part = (f"(reinterpret_cast<float*>(c.stage + {self.deferred_tile} * kStageTileBytes) + "
                        f"{(self.deferred % 2) * 256} + c.lane)")
                self.deferred += 1
                self.members += [f"unsigned dr_mask_{nm} = 0u;", f"int dr_n0_{nm} = 0;"]
                off = self._col_offset(t, "col")
                self.methods += [
                    f"__device__ __forceinline__ void flush_{nm}(const EpiCtx& c) {{",
                    f"  const float* d = {part};",
                    "#pragma unroll",
                    "  for (int k = 0; k < 8; ++k) {",
                    f"    const int col = dr_n0_{nm} + k * 32 + c.lane;",
                    f"    if (((dr_mask_{nm} >> k) & 1u) && {self._col_ok('col')} && EVTB_CHK(c, {off}, 1, {t.numel}LL, {slot})) "
                    f"{red}({base} + ({off}), d[k * 32]);",
                    "  }",
                    f"  dr_mask_{nm} = 0u;",
                    "}"]
                self.begin.append(f"if (dr_mask_{nm} != 0u && dr_n0_{nm} != c.n0) flush_{nm}(c);")
                self.begin.append(f"dr_n0_{nm} = c.n0;")
                self.chunk_end.append("{")
                self.chunk_end.append(f"  const float r = warp_transpose_reduce32<{opc}>(rr_{nm}, c.lane);")
                self.chunk_end.append("  const int k = ((n - c.n0) >> 5) & 7;")
                self.chunk_end.append(f"  float* d = {part} + k * 32;     // a word only this lane touches")
                self.chunk_end.append(f"  *d = ((dr_mask_{nm} >> k) & 1u) ? {opc}::apply(*d, r) : r;")
                self.chunk_end.append(f"  dr_mask_{nm} |= 1u << k;")
                self.chunk_end.append("}")
                self.finish.append(f"flush_{nm}(c);")
        elif "n" in axes:
            # [M]-vector result: stays in the thread across the whole tile row
            self.members.append(f"float cr_{nm};")
            self.begin.append(f"cr_{nm} = {ident};")
            self.body_elem.append(
                f"if ({self._col_ok('n + j')}) cr_{nm} = {opc}::apply(cr_{nm}, {src});")
            self.end.append(f"if ({self.ROW_OK} && EVTB_CHK(c, {self._row_offset(t)}, 1, {t.numel}LL, {slot})) {red}({base} + ({self._row_offset(t)}), cr_{nm});")
        else:
            raise NotImplementedError("reduction over the batch axis only")

    def _assemble(self) -> str:
        ind = lambda lines, k: "\n".join(" " * k + s for s in lines)
        s = []
        s.append(f"struct {self.struct_name} {{")
        s.append(ind(self.members, 2))
        if self.double_buffer and self.stage_tiles:
            sets = self.stage_tiles
            s.append("  int dbuf_ = 0;   // which of the two sets of staging tiles this chunk uses")
            s.append("  __device__ __forceinline__ char* stg(const EpiCtx& c, const int r) const {")
            s.append(f"    return c.stage + (r + dbuf_ * {sets}) * kStageTileBytes;")
            s.append("  }")
        else:
            s.append("  __device__ __forceinline__ char* stg(const EpiCtx& c, const int r) const { return c.stage + r * kStageTileBytes; }")
        s.append(ind(self.methods, 2))
        s.append("  __device__ __forceinline__ void tile_begin(const EpiCtx& c) {")
        s.append(ind(self.begin, 4))
        s.append("  }")
        s.append("  template <int G>")
        s.append("  __device__ __forceinline__ void visit8(const EpiCtx& c, const int n, const float* __restrict__ acc) {")
        s.append(ind(self.body_pre, 4))
        s.append("#pragma unroll")
        s.append("    for (int j = 0; j < 8; ++j) {")
        s.append(ind(self.body_elem, 6))
        s.append("    }")
        s.append(ind(self.body_post, 4))
        s.append("  }")
        if self.rowop is not None:
            passes = 2 if self.stat1_elem else 1
            s.append(f"  static constexpr int kStatPasses = {passes};")
            s.append(f"  static constexpr bool kWriteBack = {'true' if self.write_back else 'false'};")
            for pidx, elem, post, ab, merge in ((0, self.stat_elem, self.stat_post, self.stat_ab, self.merge),
                                                (1, self.stat1_elem, [], self.stat1_ab, self.merge1)):
                if pidx == 1 and passes == 1:
                    elem, ab, merge = [], ("0.f", "0.f"), []
                s.append(f"  // statistics pass {pidx} of the row-wise step: the element values of visit8, no stores")
                s.append("  template <int G>")
                s.append(f"  __device__ __forceinline__ void stat8_{pidx}(const EpiCtx& c, const int n, float* __restrict__ acc) {{")
                s.append(ind(self.stat_pre, 4))
                s.append("#pragma unroll")
                s.append("    for (int j = 0; j < 8; ++j) {")
                s.append(ind(elem, 6))
                s.append("    }")
                s.append(ind(post, 4))
                s.append("  }")
                s.append(f"  __device__ __forceinline__ void stat_body{pidx}(const EpiCtx& c, const int n, float (&acc)[32]) {{")
                for g in range(4):
                    s.append(f"    stat8_{pidx}<{g}>(c, n + {8 * g}, acc + {8 * g});")
                s.append("  }")
                s.append(f"  __device__ __forceinline__ float stat_a{pidx}() const {{ return {ab[0]}; }}")
                s.append(f"  __device__ __forceinline__ float stat_b{pidx}() const {{ return {ab[1]}; }}")
                s.append("  // partial statistics of the warps that share this row -> final statistics")
                s.append(f"  __device__ __forceinline__ void merge{pidx}(const float* pa, const float* pb, const int cnt) {{")
                s.append(ind(merge, 4))
                s.append("  }")
        s.append("  __device__ __forceinline__ void chunk_begin(const EpiCtx& c, const int n) {")
        if self.alias_wait:
            s.append("    // a result tile doubles as an aux-load tile: the copy engine must have read it")
            s.append(f"    if (c.lane == 0) tma_store_wait_read<{1 if self.double_buffer else 0}>();")
            s.append("    __syncwarp();")
        s.append(ind(self.chunk_begin, 4))
        if self.chunk_begin:
            s.append("    __syncwarp();")
        s.append("  }")
        s.append("  __device__ __forceinline__ void chunk_end(const EpiCtx& c, const int n) {")
        if self.tma_issue:
            s.append("    // staging tiles -> global, one TMA bulk store per result, warp and chunk")
            s.append("    fence_proxy_async_smem();   // this lane's tile writes become visible to the copy engine")
        if self.stage_tiles:
            s.append("    __syncwarp();   // every lane's staging-tile traffic of this chunk is done")
        if self.tma_issue:
            s.append("    if (c.lane == 0 && c.m_warp < c.M) {")
            s.append(ind(self.tma_issue, 6))
            s.append("      tma_store_commit();")
            s.append("    }")
        s.append(ind(self.chunk_stores, 4))
        if self.chunk_stores:
            s.append("    __syncwarp();   // tiles may be overwritten by the next chunk")
        s.append(ind(self.chunk_end, 4))
        if self.double_buffer and self.stage_tiles:
            s.append("    dbuf_ ^= 1;")
        s.append("  }")
        s.append("  __device__ __forceinline__ void body(const EpiCtx& c, const int n, const float (&acc)[32]) {")
        if self.tma_stores:
            if self.double_buffer:
                s.append("    // the copy engine must be done reading this set of staging tiles (the chunk before the previous one)")
                s.append("    if (c.lane == 0) tma_store_wait_read<1>();")
            else:
                s.append("    // the copy engine must be done reading the staging tiles of the previous chunk")
                s.append("    if (c.lane == 0) tma_store_wait_read<0>();")
            s.append("    __syncwarp();")
        s.append("    visit8<0>(c, n, acc);")
        s.append("    visit8<1>(c, n + 8, acc + 8);")
        s.append("    visit8<2>(c, n + 16, acc + 16);")
        s.append("    visit8<3>(c, n + 24, acc + 24);")
        s.append("  }")
        s.append("  __device__ __forceinline__ void visit(const EpiCtx& c, const int n, const float (&acc)[32]) {")
        s.append("    chunk_begin(c, n);")
        s.append("    body(c, n, acc);")
        s.append("    chunk_end(c, n);")
        s.append("  }")
        s.append("  __device__ __forceinline__ void tile_end(const EpiCtx& c) {")
        s.append(ind(self.end, 4))
        s.append("  }")
        s.append("  // once per warp after its last tile: bulk stores still in flight complete before the CTA leaves")
        s.append("  __device__ __forceinline__ void finish(const EpiCtx& c) {")
        s.append(ind(self.finish, 4))
        if self.tma_stores:
            s.append("    if (c.lane == 0) tma_store_wait_all<0>();")
            s.append("    __syncwarp();")
        s.append("  }")
        s.append("};")
        return "\n".join(s)


# ----------------------------------------------------------------------------------------
# kernel wrappers
# ----------------------------------------------------------------------------------------

@dataclass
class GemmTileConfig:
    bn: int = 256
    stages: int = 4
    epi_warps: int = 8
    stage_tiles: int = 0      # staging tiles per epilogue warp (set by the code generator)
    split_k: int = 1          # K is cut into this many work units per tile (fp32 partials in a workspace)
    k_rotate: bool = False    # every CTA starts its K loop at a different k-block
    cta_pair: bool = False    # two CTAs of a cluster share a 256 x bn tile (tcgen05 cta_group::2)
    tma_store: bool = True    # results with a linear address leave through TMA bulk stores
    staged: bool = True       # full tensors of the epilogue pass through shared-memory staging tiles
    row_resident: bool = False  # 128 x 512 tile = whole rows: a row-wise step runs in the epilogue (set by gemm_source)
    double_buffer: bool = False  # two sets of staging tiles used by alternate chunks (TMA-store epilogues)

    @property
    def threads(self) -> int:
        return 64 + 32 * self.epi_warps


def gemm_source(ir: EpilogueIR, a_major: str, b_major: str, dtype: torch.dtype,
                cfg: GemmTileConfig) -> Tuple[str, EpilogueSource, str]:
    """Full translation unit for one fused GEMM / batched GEMM.  Returns (source, epilogue
    description, entry-point name)."""
    # a CTA pair covers 256 rows per tile: rows 128..255 of the last tile are out of range unless
    # M is a multiple of 256
    epi = EpilogueGenerator(ir, row_tile=256 if cfg.cta_pair else 128, staged=cfg.staged, tma_store=cfg.tma_store and cfg.staged,
                            double_buffer=cfg.double_buffer and cfg.tma_store and cfg.staged).generate()
    cfg.stage_tiles = epi.stage_tiles
    # the staging tiles come out of the shared memory the operand ring would otherwise get
    while cfg.stages > 2 and gemm_smem_bytes(cfg) > 227 * 1024:
        cfg.stages -= 1
    a_mn = "true" if a_major == "MN" else "false"
    b_mn = "true" if b_major == "MN" else "false"
    bf16 = "true" if dtype == torch.bfloat16 else "false"
    if any(n.kind == "rowop" for n in ir.nodes):
        # row-resident kernel: one 128 x 512 accumulator, two epilogue passes
        cfg.row_resident, cfg.cta_pair, cfg.split_k, cfg.bn = True, False, 1, 512
        if cfg.epi_warps not in (8, 16):
            cfg.epi_warps = 16
        epi = EpilogueGenerator(ir, row_tile=128, staged=True, tma_store=cfg.tma_store,
                                double_buffer=cfg.double_buffer and cfg.tma_store).generate()
        cfg.stage_tiles = epi.stage_tiles
        cfg.stages = min(cfg.stages, 4)
        while cfg.stages > 2 and gemm_smem_bytes(cfg) > 227 * 1024:
            cfg.stages -= 1
        if gemm_smem_bytes(cfg) > 227 * 1024 and cfg.epi_warps == 16:
            cfg.epi_warps = 8          # half the staging tiles
        if gemm_smem_bytes(cfg) > 227 * 1024:
            raise NotImplementedError("row-resident GEMM: epilogue staging does not fit shared memory")
        body = f"""// generated by evt_ae_b200.codegen -- do not edit
{DEBUG_DEFINE()}#include "gemm_sm100_rows.cuh"
#include "epilogue_ops.cuh"
using namespace evtb;

{epi.struct_code}

using Cfg = GemmRowsConfig<{cfg.stages}, {a_mn}, {b_mn}, {bf16}, {cfg.epi_warps}, {cfg.stage_tiles * 2048}>;

extern "C" __global__ void __launch_bounds__(Cfg::THREADS, 1)
evtb_gemm_kernel(const __grid_constant__ GemmParams p) {{
  gemm_rows_kernel_body<Cfg, Epi>(p);
}}

extern "C" __global__ void evtb_kernel_info(int* out) {{
  out[0] = Cfg::SMEM_BYTES;
  out[1] = Cfg::THREADS;
}}
"""
        return body, epi, "evtb_gemm_kernel"
    if cfg.cta_pair:
        if cfg.bn not in (128, 256):
            raise ValueError("CTA-pair tiles are 256 x 128 or 256 x 256")
        body = f"""// generated by evt_ae_b200.codegen -- do not edit
{DEBUG_DEFINE()}#include "gemm_sm100_pair.cuh"
#include "epilogue_ops.cuh"
using namespace evtb;

{epi.struct_code}

using Cfg = GemmPairConfig<{cfg.bn}, {cfg.stages}, {a_mn}, {b_mn}, {bf16}, {cfg.epi_warps}, {cfg.stage_tiles * 2048}, {'true' if cfg.split_k > 1 else 'false'}>;

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::THREADS, 1)
evtb_gemm_kernel(const __grid_constant__ GemmParams p) {{
  gemm_pair_kernel_body<Cfg, Epi>(p);
}}

extern "C" __global__ void evtb_kernel_info(int* out) {{
  out[0] = Cfg::SMEM_BYTES;
  out[1] = Cfg::THREADS;
}}
"""
        return body, epi, "evtb_gemm_kernel"
    body = f"""// generated by evt_ae_b200.codegen -- do not edit
{DEBUG_DEFINE()}#include "gemm_sm100.cuh"
#include "epilogue_ops.cuh"
using namespace evtb;

{epi.struct_code}

using Cfg = GemmConfig<{cfg.bn}, {cfg.stages}, {a_mn}, {b_mn}, {bf16}, {cfg.epi_warps}, {cfg.stage_tiles * 2048}, {'true' if cfg.split_k > 1 else 'false'}, {'true' if cfg.k_rotate else 'false'}>;

extern "C" __global__ void __launch_bounds__(Cfg::THREADS, 1)
evtb_gemm_kernel(const __grid_constant__ GemmParams p) {{
  gemm_kernel_body<Cfg, Epi>(p);
}}

extern "C" __global__ void evtb_kernel_info(int* out) {{
  out[0] = Cfg::SMEM_BYTES;
  out[1] = Cfg::THREADS;
}}
"""
    return body, epi, "evtb_gemm_kernel"


@dataclass
class ConvTileConfig:
    bn: int = 128             # output channels per accumulator tile (64, 128 or 256)
    stages: int = 6
    epi_warps: int = 8
    stage_tiles: int = 0

    @property
    def threads(self) -> int:
        return 64 + 32 * self.epi_warps


def conv_wgrad_source(ir: EpilogueIR, dtype: torch.dtype, cfg: GemmTileConfig) -> Tuple[str, EpilogueSource, str]:
    """Translation unit for a convolution weight gradient: the GEMM kernel (one CTA per tile, both
    operands MN-major, split along the reduction) with its operand tiles fetched as boxes of the two
    channels-last tensors.  The epilogue sees the [K, R*S*C] result matrix."""
    cfg.cta_pair, cfg.row_resident = False, False
    epi = EpilogueGenerator(ir, row_tile=128, staged=cfg.staged, tma_store=cfg.tma_store and cfg.staged).generate()
    cfg.stage_tiles = epi.stage_tiles
    while cfg.stages > 2 and gemm_smem_bytes(cfg) > 227 * 1024:
        cfg.stages -= 1
    bf16 = "true" if dtype == torch.bfloat16 else "false"
    body = f"""// generated by evt_ae_b200.codegen -- do not edit
{DEBUG_DEFINE()}#include "gemm_sm100.cuh"
#include "epilogue_ops.cuh"
using namespace evtb;

{epi.struct_code}

using Cfg = GemmConfig<{cfg.bn}, {cfg.stages}, true, true, {bf16}, {cfg.epi_warps}, {cfg.stage_tiles * 2048}, {'true' if cfg.split_k > 1 else 'false'}, false, true>;

extern "C" __global__ void __launch_bounds__(Cfg::THREADS, 1)
evtb_gemm_kernel(const __grid_constant__ GemmParams p) {{
  gemm_kernel_body<Cfg, Epi>(p);
}}

extern "C" __global__ void evtb_kernel_info(int* out) {{
  out[0] = Cfg::SMEM_BYTES;
  out[1] = Cfg::THREADS;
}}
"""
    return body, epi, "evtb_gemm_kernel"


def conv_smem_bytes(cfg: ConvTileConfig) -> int:
    return 1024 + cfg.stages * (128 * 64 * 2 + cfg.bn * 64 * 2) + 1024 + cfg.epi_warps * cfg.stage_tiles * 2048


def conv_source(ir: EpilogueIR, dgrad: bool, dtype: torch.dtype, cfg: ConvTileConfig) -> Tuple[str, EpilogueSource, str]:
    """Translation unit for one fused convolution (forward or data gradient).  The epilogue is
    generated exactly as for a GEMM over the (N*P*Q, K) result matrix; rows are always
    predicated because an accumulator tile is a box of output positions, not a row range."""
    # measured at the ResNet-50 shapes: holding the column sums back pays with tiles of up to 128
    # columns (1x1 convolutions to 64 channels: 75 -> 50 us) and costs with 256-column tiles, whose
    # epilogue is short of registers already (64 -> 256 channels: 145 -> 200 us)
    epi = EpilogueGenerator(ir, row_tile=0, staged=True, defer_col_reductions=cfg.bn <= 128).generate()
    cfg.stage_tiles = epi.stage_tiles
    while cfg.stages > 2 and conv_smem_bytes(cfg) > 227 * 1024:
        cfg.stages -= 1
    bf16 = "true" if dtype == torch.bfloat16 else "false"
    body = f"""// generated by evt_ae_b200.codegen -- do not edit
{DEBUG_DEFINE()}#define EVTB_ROW_M(c, row) ((c).m_rows[((row) >> 3) & 3])   /* row = i * 8 + lane / 4: mapped once per tile */
#include "conv_sm100.cuh"
#include "epilogue_ops.cuh"
using namespace evtb;

{epi.struct_code}

using Cfg = ConvConfig<{cfg.bn}, {cfg.stages}, {'true' if dgrad else 'false'}, {bf16}, {cfg.epi_warps}, {cfg.stage_tiles * 2048}>;

extern "C" __global__ void __launch_bounds__(Cfg::THREADS, 1)
evtb_conv_kernel(const __grid_constant__ ConvParams p) {{
  conv_kernel_body<Cfg, Epi>(p);
}}

extern "C" __global__ void evtb_kernel_info(int* out) {{
  out[0] = Cfg::SMEM_BYTES;
  out[1] = Cfg::THREADS;
}}
"""
    return body, epi, "evtb_conv_kernel"


# ----------------------------------------------------------------------------------------
# row-wise (reduce-apply) kernels
# ----------------------------------------------------------------------------------------

@dataclass
class RowKernelConfig:
    tpr: int          # threads per row
    vpt: int          # 8-element vectors per thread
    threads: int      # CTA size
    vec: bool         # aligned 128-bit operand loads

    @property
    def rows_per_cta(self) -> int:
        return self.threads // self.tpr

    @property
    def smem_bytes(self) -> int:
        return 4 * self.rows_per_cta * max(1, self.tpr // 32)


def pick_row_config(cols: int, max_vpt: int = 4) -> RowKernelConfig:
    """Threads per row and register tile, the search space of the reference's reduce-apply
    tuner (python/gtl/compiler/autotuner/reduce_apply_tuner.py:33-48: rows per CTA x warps x
    input cache) collapsed: the row always lives in registers, a row gets the fewest threads
    that keep at most `max_vpt` 128-bit vectors each, CTAs are 128 threads or one row wide."""
    vectors = (cols + 7) // 8
    tpr = 8
    while tpr < 1024 and (vectors + tpr - 1) // tpr > max_vpt:
        tpr *= 2
    vpt = (vectors + tpr - 1) // tpr
    threads = max(128, tpr)
    return RowKernelConfig(tpr=tpr, vpt=vpt, threads=threads, vec=(cols % 8 == 0))


ROW_KINDS = {
    "softmax": ("softmax_body", 1),
    "softmax_backward": ("softmax_backward_body", 2),
    "layernorm": ("layernorm_body", 1),
    "layernorm_backward": ("layernorm_backward_body", 2),
}


def row_kernel_source(kind: str, ir: EpilogueIR, dtype: torch.dtype, cfg: RowKernelConfig,
                      eps: float = 1e-12, gamma_dtype: Optional[torch.dtype] = None):
    """Translation unit for one fused softmax / LayerNorm (forward or backward) node."""
    epi = EpilogueGenerator(ir, row_tile=0, col_group=8).generate()
    body, _ = ROW_KINDS[kind]
    ct = CTYPE[dtype]
    vec = "true" if cfg.vec else "false"
    if kind == "layernorm":
        call = f"{body}<{ct}, {cfg.tpr}, {cfg.vpt}, {vec}, Epi>(p, {float(eps)!r}f);"
    elif kind == "layernorm_backward":
        call = f"{body}<{ct}, {CTYPE[gamma_dtype or dtype]}, {cfg.tpr}, {cfg.vpt}, {vec}, Epi>(p);"
    else:
        call = f"{body}<{ct}, {cfg.tpr}, {cfg.vpt}, {vec}, Epi>(p);"
    src = f"""// generated by evt_ae_b200.codegen -- do not edit
{DEBUG_DEFINE()}#include "reduce_apply.cuh"
using namespace evtb;

{epi.struct_code}

extern "C" __global__ void __launch_bounds__({cfg.threads})
evtb_row_kernel(const __grid_constant__ RowParams p) {{
  {call}
}}
"""
    return src, epi, "evtb_row_kernel"


# ----------------------------------------------------------------------------------------
# CSR SpMM
# ----------------------------------------------------------------------------------------

@dataclass
class SpmmConfig:
    g: int            # lanes that share one nonzero's feature row (power of two, 8 columns each)
    vpt: int          # 8-column vectors per lane
    threads: int = 256
    t_long: int = 128         # a lane group handles rows up to this many nonzeros alone
    task_len: int = 1024      # nonzeros per task (one CTA) of the longer rows
    u_short: int = 4          # nonzeros of a short row in flight per lane group
    u_long: int = 4           # batches of 32 / g nonzeros in flight per warp in a task
    min_ctas: int = 4         # resident CTAs per SM the register allocation is held to

    @property
    def f_pad(self) -> int:
        return self.g * self.vpt * 8


def pick_spmm_config(F: int) -> SpmmConfig:
    groups = (F + 7) // 8
    g = 1
    while g < 32 and g < groups:
        g *= 2
    return SpmmConfig(g=g, vpt=(groups + g - 1) // g)


def spmm_source(ir: EpilogueIR, dtype: torch.dtype, cfg: SpmmConfig, fused_norm: bool):
    """Translation unit for one fused SpMM node: main kernel + the launch that lists the tasks of
    the long rows."""
    if ir.N % 8 != 0:
        raise NotImplementedError("SpMM needs a feature width that is a multiple of 8")
    epi = EpilogueGenerator(ir, row_tile=0, col_group=8).generate()
    ct = CTYPE[dtype]
    norm = "true" if fused_norm else "false"
    src = f"""// generated by evt_ae_b200.codegen -- do not edit
{DEBUG_DEFINE()}#include "spmm.cuh"
using namespace evtb;

{epi.struct_code}

extern "C" __global__ void __launch_bounds__({cfg.threads}, {cfg.min_ctas})
evtb_spmm_kernel(const __grid_constant__ SpmmParams p) {{
  spmm_body<{ct}, {cfg.g}, {cfg.vpt}, {norm}, {cfg.u_short}, {cfg.u_long}, {cfg.threads // 32}, Epi>(p);
}}

extern "C" __global__ void __launch_bounds__(256)
evtb_spmm_prep_kernel(const __grid_constant__ SpmmParams p) {{
  spmm_prep_body(p);
}}
"""
    return src, epi, "evtb_spmm_kernel"


def gemm_smem_bytes(cfg: GemmTileConfig) -> int:
    if cfg.row_resident:
        return (1024 + cfg.stages * (128 * 64 * 2 + 512 * 64 * 2) + 1024 + cfg.epi_warps * cfg.stage_tiles * 2048
                + 2 * 4 * (cfg.epi_warps // 4) * 32 * 8)
    b_rows = cfg.bn // 2 if cfg.cta_pair else cfg.bn      # a CTA of a pair stages half of B's columns
    return 1024 + cfg.stages * (128 * 64 * 2 + b_rows * 64 * 2) + 1024 + cfg.epi_warps * cfg.stage_tiles * 2048


def source_hash(src: str) -> str:
    return hashlib.sha256(src.encode()).hexdigest()[:20]
