"""fx partition -> (main-loop operands, epilogue DAG).

Plays the role of `EVTFuser.trace` (python/gtl/compiler/passes/evt_fuser.py:1065-1235) and
of its `visit_*` methods (:1308-1485), with the CUTLASS-fork DAG IR replaced by
`evt_ae_b200.ir`.  The anchor ("heavy") op of the partition defines a canonical (l, m, n)
index space; shapes and strides of every other value are pushed through the partition's
view / permute / unsqueeze / squeeze nodes on *meta* tensors, so layout nodes turn into
index maps and never run.

A partition is a list of node names of a `torch.fx.GraphModule` whose nodes carry
`meta["tensor_meta"]` (run `ShapeProp` first), exactly what the reference's partitioner
hands to its fuser (python/gtl/compiler/passes/pass_fusion.py:1364-1372).
"""
from __future__ import annotations

import math
import operator
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from torch.fx import GraphModule, Node as FxNode

from .ir import EpilogueIR, Factor, Node, TensorRef

# ----------------------------------------------------------------------------------------
# target normalisation
# ----------------------------------------------------------------------------------------

ANCHOR_OPS = {
    "mm": "gemm",
    "bmm": "bmm",
    "_softmax": "softmax",
    "_softmax_backward_data": "softmax_backward",
    "native_layer_norm": "layernorm",
    "native_layer_norm_backward": "layernorm_backward",
    "spmm": "spmm",
    "spmm_sym": "spmm",
    "convolution_forward_channel_last": "conv_fprop",
    "convolution_backward_data_channel_last": "conv_dgrad",
    "convolution_backward_weight_channel_last": "conv_wgrad",
}

ROW_EPILOGUE_OPS = {"_softmax": "softmax", "_softmax_backward_data": "softmax_backward"}
ROW_EPILOGUE_MAX_N = 512      # one accumulator row must fit the 512 tensor-memory columns

LAYOUT_OPS = {"view", "_unsafe_view", "reshape", "permute", "unsqueeze", "squeeze", "clone",
              "contiguous", "detach", "alias", "expand"}
PASSTHROUGH_OPS = {"clone", "contiguous", "detach", "alias", "to", "_to_copy"}
BINARY_OPS = {"add", "sub", "mul", "div", "ge", "gt", "ne", "tanh_backward", "maximum"}
UNARY_OPS = {"neg", "relu", "tanh", "sigmoid", "exp", "rsqrt"}


def op_name(target) -> str:
    """aten overload packets, overloads, builtins and wrapped leaf functions -> short name."""
    if isinstance(target, str):
        return target
    if isinstance(target, torch._ops.OpOverload):
        return target.overloadpacket.__name__
    if isinstance(target, torch._ops.OpOverloadPacket):
        return target.__name__
    if target is operator.getitem:
        return "getitem"
    name = getattr(target, "__name__", str(target))
    return name


def _meta(node: FxNode):
    tm = node.meta.get("tensor_meta")
    if tm is None:
        raise ValueError(f"node {node.name} has no tensor_meta; run ShapeProp first")
    return tm


def _shape(node: FxNode) -> Tuple[int, ...]:
    tm = _meta(node)
    if not hasattr(tm, "shape"):   # tuple-returning op: describe its first result
        tm = tm[0]
    return tuple(int(s) for s in tm.shape)


def _dtype(node: FxNode) -> torch.dtype:
    tm = _meta(node)
    if not hasattr(tm, "dtype"):
        tm = tm[0]
    return tm.dtype


def _contig_strides(shape: Sequence[int]) -> Tuple[int, ...]:
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= max(int(s), 1)
    return tuple(reversed(st))


# ----------------------------------------------------------------------------------------
# layout algebra on meta tensors
# ----------------------------------------------------------------------------------------

class Layout:
    """Canonical map of a value: for every logical dim a list of (size, cstride) sub-factors,
    outer to inner, where cstride counts steps of the canonical linear index
    c = (l*M + m)*N + n.  A dim of extent 1 (or a broadcast dim) has no sub-factors.
    Unlike plain strides this survives `view` after `permute` (a merged dim simply keeps
    several sub-factors)."""

    def __init__(self, dims: List[List[Tuple[int, int]]]):
        self.dims = [[(int(s), int(c)) for s, c in d if int(s) != 1] for d in dims]

    @staticmethod
    def contiguous(shape: Sequence[int]) -> "Layout":
        return Layout([[(s, cs)] for s, cs in zip(shape, _contig_strides(shape))])

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(int(math.prod(s for s, _ in d)) for d in self.dims)

    def dim(self) -> int:
        return len(self.dims)

    def permute(self, perm: Sequence[int]) -> "Layout":
        perm = [int(p) % len(self.dims) for p in perm]
        return Layout([self.dims[p] for p in perm])

    def unsqueeze(self, d: int) -> "Layout":
        d = int(d)
        if d < 0:
            d += len(self.dims) + 1
        return Layout(self.dims[:d] + [[]] + self.dims[d:])

    def squeeze(self, d: Optional[int] = None) -> "Layout":
        if d is None:
            return Layout([x for x in self.dims if x])
        d = int(d) % len(self.dims)
        if self.dims[d]:
            return self
        return Layout(self.dims[:d] + self.dims[d + 1:])

    def view(self, new_shape: Sequence[int]) -> "Layout":
        new_shape = [int(x) for x in new_shape]
        total = int(math.prod(self.shape))
        if -1 in new_shape:
            known = -int(math.prod(new_shape))
            new_shape[new_shape.index(-1)] = total // known
        if int(math.prod(new_shape)) != total:
            raise RuntimeError(f"view {self.shape} -> {new_shape}: element count differs")
        flat = [f for d in self.dims for f in d]
        out: List[List[Tuple[int, int]]] = []
        i = 0
        for want in new_shape:
            cur: List[Tuple[int, int]] = []
            need = want
            while need > 1:
                if i >= len(flat):
                    raise RuntimeError("view ran out of factors")
                sz, cs = flat[i]
                if sz <= need:
                    if need % sz != 0:
                        raise RuntimeError(f"view {self.shape} -> {new_shape}: factor {sz} does not divide {need}")
                    cur.append((sz, cs))
                    need //= sz
                    i += 1
                else:
                    if sz % need != 0:
                        raise RuntimeError(f"view {self.shape} -> {new_shape}: cannot split factor {sz} by {need}")
                    rest = sz // need
                    cur.append((need, cs * rest))
                    flat[i] = (rest, cs)
                    need = 1
            out.append(cur)
        return Layout(out)

    def broadcast_to_operand(self, op_shape: Sequence[int]) -> "Layout":
        """Layout of an operand of shape `op_shape` that broadcasts (right-aligned) against
        a value with this layout."""
        pad = len(self.dims) - len(op_shape)
        if pad < 0:
            raise RuntimeError("operand has more dims than the value it broadcasts to")
        dims = []
        for i, sz in enumerate(op_shape):
            full = self.dims[pad + i]
            if int(sz) == 1:
                dims.append([])
            else:
                if int(math.prod(s for s, _ in full)) != int(sz):
                    raise RuntimeError("operand does not broadcast against the value")
                dims.append(list(full))
        return Layout(dims)

    def pad_left(self, ndim: int) -> "Layout":
        return Layout([[]] * (ndim - len(self.dims)) + self.dims)


def _apply_layout(node: FxNode, t: "Layout") -> "Layout":
    """Apply the layout op of `node` to the layout of node.args[0]."""
    name = op_name(node.target)
    if name in ("view", "_unsafe_view", "reshape"):
        return t.view(node.args[1])
    if name == "permute":
        return t.permute(node.args[1])
    if name == "unsqueeze":
        return t.unsqueeze(node.args[1])
    if name == "squeeze":
        if len(node.args) > 1:
            d = node.args[1]
            if isinstance(d, (list, tuple)):
                for x in sorted([int(v) % t.dim() for v in d], reverse=True):
                    t = t.squeeze(x)
                return t
            return t.squeeze(d)
        return t.squeeze()
    if name == "expand":
        return t.pad_left(len(node.args[1]))
    if name in PASSTHROUGH_OPS:
        return t
    raise NotImplementedError(f"layout op {name}")


def _invert_layout(node: FxNode, out_t: "Layout") -> "Layout":
    """Layout of the *input* of layout node `node`, given the layout of its output."""
    name = op_name(node.target)
    src = node.args[0]
    in_shape = _shape(src)
    if name in ("view", "_unsafe_view", "reshape"):
        return out_t.view(in_shape)
    if name == "permute":
        perm = [int(i) % len(in_shape) for i in node.args[1]]
        inv = [0] * len(perm)
        for i, p in enumerate(perm):
            inv[p] = i
        return out_t.permute(inv)
    if name == "unsqueeze":
        return out_t.squeeze(int(node.args[1]) % out_t.dim())
    if name == "squeeze":
        t = out_t
        for i, sz in enumerate(in_shape):
            if i >= t.dim() or t.shape[i] != sz:
                t = t.unsqueeze(i)
        assert tuple(t.shape) == tuple(in_shape)
        return t
    if name == "expand":
        return out_t.broadcast_to_operand(in_shape)
    if name in PASSTHROUGH_OPS:
        return out_t
    raise NotImplementedError(f"cannot invert layout op {name}")


def _strided_meta(shape, strides) -> torch.Tensor:
    return torch.empty_strided(tuple(shape), tuple(strides), device="meta")


def _split_dim(size: int, cstride: int, memstride: int, L: int, M: int, N: int) -> List[Factor]:
    """One sub-factor that walks canonical index `cstride * i` (i < size) -> axis factors."""
    out: List[Factor] = []
    bounds = [("n", 1, N), ("m", N, M), ("l", M * N, L)]
    for axis, base, extent in bounds:
        if size <= 1:
            break
        hi = base * extent  # first canonical stride that belongs to the next axis
        if cstride >= hi:
            continue
        if cstride % base != 0:
            raise NotImplementedError(f"dim (size {size}, stride {cstride}) is not aligned to axis {axis}")
        unit = cstride // base
        if extent % max(unit, 1) != 0:
            raise NotImplementedError("dim does not tile its axis")
        room = extent // unit  # how many steps fit in this axis
        if size <= room:
            out.append(Factor(axis, unit, size, memstride))
            size = 1
            break
        if size % room != 0:
            raise NotImplementedError(f"dim of size {size} straddles axis {axis} unevenly")
        out.append(Factor(axis, unit, room, memstride))
        memstride *= room
        cstride = hi
        size //= room
    if size > 1:
        raise NotImplementedError("dim exceeds canonical space")
    return out


def _factors(lay: "Layout", memstrides: Sequence[int], L: int, M: int, N: int) -> Tuple[Factor, ...]:
    fs: List[Factor] = []
    for sub, ms in zip(lay.dims, memstrides):
        ms = int(ms)
        for size, cs in reversed(sub):          # inner sub-factor first
            fs.extend(_split_dim(int(size), int(cs), ms, L, M, N))
            ms *= int(size)
    order = {"l": 0, "m": 1, "n": 2}
    fs.sort(key=lambda f: (order[f.axis], -f.unit))
    return tuple(_simplify(fs, L, M, N))


def _simplify(fs: List[Factor], L: int, M: int, N: int) -> List[Factor]:
    """Merge neighbouring factors of one axis whose strides chain (so a plain row-major
    tensor collapses to one factor per axis)."""
    out: List[Factor] = []
    for f in fs:
        if out:
            g = out[-1]
            # g is the outer factor (bigger unit): g.unit == f.unit * f.size and g.stride == f.stride * f.size
            if g.axis == f.axis and g.unit == f.unit * f.size and g.stride == f.stride * f.size:
                out[-1] = Factor(f.axis, f.unit, f.size * g.size, f.stride)
                continue
        out.append(f)
    return out


# ----------------------------------------------------------------------------------------
# main-loop operand description
# ----------------------------------------------------------------------------------------

@dataclass
class OperandSpec:
    """A GEMM operand as the TMA descriptor needs it: which fx node holds the memory, which
    logical dim is contiguous and the element strides of the other two."""
    source: FxNode
    major: str            # 'K' (reduction dim contiguous) or 'MN'
    stride_outer: int     # element stride of the non-contiguous matrix dim
    stride_batch: int     # element stride between batches (0 when L == 1)
    needs_copy: bool = False   # neither dim contiguous: caller materialises the operand first
    dtype: torch.dtype = torch.float16


def _operand_spec(node: FxNode, partition: set, is_a: bool, batched: bool) -> Tuple[OperandSpec, List[FxNode]]:
    """Walk back through permute/view nodes that belong to the partition and feed only the
    anchor (the reference folds such permutes into the operand layout,
    evt_fuser.py:548-558 and :682-697)."""
    chain: List[FxNode] = []
    cur = node
    while (isinstance(cur, FxNode) and cur.op == "call_function" and cur.name in partition
           and op_name(cur.target) in ("permute", "view", "_unsafe_view", "clone", "expand")
           and len(cur.users) == 1):
        chain.append(cur)
        cur = cur.args[0]
    src = cur
    shape = _shape(src)
    t = Layout.contiguous(shape)   # "cstride" here = element stride in the source's memory
    ok = True
    try:
        for ln in reversed(chain):
            t = _apply_layout(ln, t)
    except RuntimeError:
        ok = False
    if ok and (tuple(t.shape) != _shape(node) or any(len(d) > 1 for d in t.dims)):
        ok = False
    if not ok:
        return OperandSpec(node, "K" if is_a else "MN", 0, 0, True, _dtype(node)), []
    st = [int(d[0][1]) if d else 0 for d in t.dims]
    sh = [int(x) for x in t.shape]
    if batched:
        sb, s0, s1 = st
        d0, d1 = sh[1], sh[2]
    else:
        sb = 0
        s0, s1 = st
        d0, d1 = sh
    # A is [M, K]: K contiguous -> 'K'; B is [K, N]: K contiguous (s0 == 1) -> 'K'
    k_stride, mn_stride = (s1, s0) if is_a else (s0, s1)
    k_size, mn_size = (d1, d0) if is_a else (d0, d1)
    def aligned(v):
        return v % 8 == 0
    if (k_stride == 1 or k_size == 1) and aligned(mn_stride) and aligned(sb):
        return OperandSpec(src, "K", mn_stride, sb, False, _dtype(node)), chain
    if (mn_stride == 1 or mn_size == 1) and aligned(k_stride) and aligned(sb):
        return OperandSpec(src, "MN", k_stride, sb, False, _dtype(node)), chain
    # strides a TMA descriptor cannot express: materialise the operand as written
    return OperandSpec(node, "K" if is_a else "MN", 0, 0, True, _dtype(node)), []


# ----------------------------------------------------------------------------------------
# the trace
# ----------------------------------------------------------------------------------------

@dataclass
class PartitionTrace:
    kind: str                                   # gemm | bmm | softmax | ...
    anchor: FxNode
    ir: EpilogueIR
    inputs: List[FxNode]                        # epilogue inputs, in call order
    outputs: List[FxNode]                       # fx nodes whose values leave the partition
    output_stores: List[str]                    # IR node name holding each output
    mainloop_args: List[FxNode] = field(default_factory=list)
    operands: List[OperandSpec] = field(default_factory=list)
    consumed: List[FxNode] = field(default_factory=list)   # every fx node the fused op replaces
    attrs: dict = field(default_factory=dict)

    @property
    def input_names(self) -> List[str]:
        return [n.name for n in self.inputs]


class _Tracer:
    def __init__(self, gm: GraphModule, partition: Sequence[str]):
        self.gm = gm
        self.names = set(partition)
        self.nodes = [n for n in gm.graph.nodes if n.name in self.names]
        anchors = [n for n in self.nodes if n.op == "call_function" and op_name(n.target) in ANCHOR_OPS]
        # a softmax (or its backward) that follows a GEMM / batched GEMM in the same partition is
        # lowered into that GEMM's epilogue as a row-wise reduce-apply step (row-resident kernel)
        self.row_nodes = []
        mains = [n for n in anchors if ANCHOR_OPS[op_name(n.target)] in ("gemm", "bmm")]
        if len(anchors) == 2 and len(mains) == 1:
            other = [n for n in anchors if n is not mains[0]][0]
            if op_name(other.target) in ROW_EPILOGUE_OPS:
                self.row_nodes = [other]
                anchors = mains
        if len(anchors) != 1:
            raise ValueError(f"partition must hold exactly one heavy op, found {[a.name for a in anchors]}")
        self.anchor = anchors[0]
        self.kind = ANCHOR_OPS[op_name(self.anchor.target)]
        self.cmap: Dict[FxNode, Layout] = {}
        self.value: Dict[FxNode, str] = {}     # fx node -> IR node name producing its value
        self.ir: Optional[EpilogueIR] = None
        self.inputs: List[FxNode] = []
        self._const_id = 0

    # -- canonical space --------------------------------------------------------------
    def _setup_canonical(self):
        a = self.anchor
        shape = _shape(a)
        if self.kind == "gemm":
            L, (M, N) = 1, shape
        elif self.kind == "bmm":
            L, M, N = shape
        elif self.kind == "spmm":
            L, M, N = 1, int(math.prod(shape[:-1])), shape[-1]
        elif self.kind == "conv_wgrad":     # [K, R, S, C] filter gradient = the [K, R*S*C] matrix
            L, M, N = 1, shape[0], int(math.prod(shape[1:]))
        else:  # reduce-apply: rows x last dim
            L, M, N = 1, int(math.prod(shape[:-1])), shape[-1]
        self.ir = EpilogueIR(L, M, N)
        return shape

    # -- helpers ----------------------------------------------------------------------
    def _is_scalar_like(self, n: FxNode) -> bool:
        return math.prod(_shape(n)) == 1

    def _accum_result_nodes(self) -> Dict[FxNode, None]:
        """fx nodes standing for the accumulator value itself."""
        return {self.anchor: None}

    def run(self) -> PartitionTrace:
        a = self.anchor
        acc_shape = self._setup_canonical()
        ir = self.ir
        L, M, N = ir.L, ir.M, ir.N
        part = self.names

        # main-loop operands and the layout nodes folded into them
        operands: List[OperandSpec] = []
        mainloop_args: List[FxNode] = []
        folded: List[FxNode] = []
        unfolded: List[FxNode] = []
        if self.kind in ("gemm", "bmm"):
            for i, arg in enumerate(a.args[:2]):
                spec, chain = _operand_spec(arg, part, is_a=(i == 0), batched=(self.kind == "bmm"))
                operands.append(spec)
                mainloop_args.append(spec.source)
                folded.extend(chain)
                if spec.needs_copy:
                    # a layout chain that could not be folded stays outside the fused node: it
                    # runs as written and its result is materialised as the operand
                    cur = arg
                    while (isinstance(cur, FxNode) and cur.op == "call_function" and cur.name in part
                           and op_name(cur.target) in ("permute", "view", "_unsafe_view", "clone", "expand")
                           and len(cur.users) == 1):
                        unfolded.append(cur)
                        cur = cur.args[0]
        elif self.kind == "softmax":
            mainloop_args = [a.args[0]]                       # (input, dim, half_to_float)
        elif self.kind == "softmax_backward":
            mainloop_args = [a.args[0], a.args[1]]            # (grad, output, dim, dtype)
        elif self.kind == "layernorm":
            mainloop_args = [a.args[0]]                       # (input, shape, weight, bias, eps)
        elif self.kind == "layernorm_backward":
            # (grad, input, shape, mean, rstd, weight, bias, mask) -> [grad, x, mean, rstd, gamma]
            mainloop_args = [a.args[0], a.args[1], a.args[3], a.args[4], a.args[5]]
            mask = a.args[7] if len(a.args) > 7 else [True, False, False]
            if mask[1] or mask[2]:
                raise NotImplementedError(
                    "native_layer_norm_backward must be split first: gamma / beta gradients are "
                    "separate sum nodes (the reference's decomposition, pass_decomposition.py:546-598)")
        elif self.kind == "conv_fprop":
            mainloop_args = [a.args[0], a.args[1]]            # (x, w, stride, padding, dilation, ...)
        elif self.kind == "conv_dgrad":
            mainloop_args = [a.args[0], a.args[2]]            # (dy, x [shape only], w, stride, ...)
        elif self.kind == "conv_wgrad":
            mainloop_args = [a.args[0], a.args[1]]            # (dy, x, w [shape only], stride, ...)
        else:
            mainloop_args = [x for x in a.args if isinstance(x, FxNode)]
        if self.kind in ("softmax", "softmax_backward"):
            dim = int(a.args[1] if self.kind == "softmax" else a.args[2])
            if dim % len(acc_shape) != len(acc_shape) - 1:
                raise NotImplementedError("softmax over a dim other than the last")
        if self.kind in ("layernorm", "layernorm_backward"):
            nshape = a.args[1] if self.kind == "layernorm" else a.args[2]
            if len(nshape) != 1 or int(nshape[0]) != acc_shape[-1]:
                raise NotImplementedError("LayerNorm over more than the last dim")
        folded_set = set(folded)

        # the accumulator and, for tuple-returning anchors, its getitem(…, 0)
        accum_nodes = {a}
        tuple_anchor = self.kind in ("layernorm", "layernorm_backward")
        aux_getitems: Dict[int, FxNode] = {}
        if tuple_anchor:
            accum_nodes = set()
            for u in a.users:
                if op_name(u.target) == "getitem":
                    if u.args[1] == 0:
                        accum_nodes.add(u)
                    else:
                        aux_getitems[int(u.args[1])] = u
        ir.add(Node("accum", "accum"))
        for n in accum_nodes:
            self.value[n] = "accum"
            self.cmap[n] = Layout.contiguous(_shape(n))

        if self.kind == "layernorm":
            # gamma / beta given to the op itself become the first two epilogue nodes
            cur = "accum"
            acc_layout = Layout.contiguous(acc_shape)
            for i, opn in ((2, "mul"), (3, "add")):
                w = a.args[i] if len(a.args) > i else None
                if isinstance(w, FxNode):
                    self.cmap[w] = acc_layout.broadcast_to_operand(_shape(w))
                    ld = self._load(w)
                    nm = f"ln_{opn}_{w.name}"
                    ir.add(Node(nm, "compute", op=opn, args=(cur, ld)))
                    cur = nm
            for n in accum_nodes:
                self.value[n] = cur

        epi_nodes = [n for n in self.nodes
                     if n is not a and n not in folded_set and n not in unfolded and n not in accum_nodes
                     and n not in aux_getitems.values() and n.op == "call_function"]

        # reduce-apply kernels never carry reductions (evt_fuser.py:1096-1100)
        if self.kind not in ("gemm", "bmm", "conv_fprop", "conv_dgrad", "conv_wgrad"):
            epi_nodes = [n for n in epi_nodes if op_name(n.target) not in ("sum", "amax")]
        epi_set = set(epi_nodes)

        # ---- pass 1: forward propagation of canonical maps from the accumulator -------
        changed = True
        while changed:
            changed = False
            for n in epi_nodes:
                if n in self.cmap:
                    continue
                name = op_name(n.target)
                srcs = [x for x in n.all_input_nodes]
                if name in LAYOUT_OPS or name in PASSTHROUGH_OPS:
                    s = n.args[0]
                    if s in self.cmap:
                        self.cmap[n] = _apply_layout(n, self.cmap[s])
                        changed = True
                elif name in ("sum", "amax"):
                    continue
                else:
                    known = [x for x in srcs if x in self.cmap and _shape(x) == _shape(n)]
                    if known:
                        self.cmap[n] = self.cmap[known[0]]
                        changed = True
                    else:
                        # broadcast: an operand with fewer / unit dims still fixes the others
                        kn = [x for x in srcs if x in self.cmap]
                        if kn and math.prod(_shape(kn[0])) == math.prod(_shape(n)):
                            self.cmap[n] = self.cmap[kn[0]].pad_left(len(_shape(n)))
                            changed = True
            # ---- backward: operands of mapped elementwise nodes and layout inputs -----
            for n in reversed(epi_nodes):
                if n not in self.cmap:
                    continue
                name = op_name(n.target)
                if name in ("sum", "amax"):
                    continue
                if name in LAYOUT_OPS or name in PASSTHROUGH_OPS:
                    s = n.args[0]
                    if isinstance(s, FxNode) and s not in self.cmap:
                        try:
                            self.cmap[s] = _invert_layout(n, self.cmap[n])
                            changed = True
                        except RuntimeError as e:
                            raise NotImplementedError(f"cannot fold layout of {n.name}: {e}")
                    continue
                out_map = self.cmap[n]
                if name == "one_hot":
                    # the class axis is new: the label operand has every dim but the last
                    out_map = Layout(out_map.dims[:-1])
                for s in n.all_input_nodes:
                    if s in self.cmap:
                        continue
                    sshape = _shape(s)
                    if len(sshape) > out_map.dim():
                        continue
                    self.cmap[s] = out_map.broadcast_to_operand(sshape)
                    changed = True

        # ---- pass 2: emit IR in graph order ------------------------------------------
        outputs: List[FxNode] = []
        for n in list(accum_nodes) + epi_nodes:
            if any(u not in epi_set and u is not a and u not in accum_nodes for u in n.users):
                outputs.append(n)
        if self.kind in ("gemm", "bmm", "spmm", "softmax", "softmax_backward", "conv_fprop", "conv_dgrad", "conv_wgrad") and not epi_nodes:
            outputs = [a]
        # keep graph order
        order = {n: i for i, n in enumerate(self.gm.graph.nodes)}
        outputs.sort(key=lambda n: order[n])

        for n in epi_nodes:
            self._emit(n, epi_set)

        output_stores: List[str] = []
        final_outputs: List[FxNode] = []
        for n in outputs:
            name = op_name(n.target) if n.op == "call_function" else ""
            if name in ("sum", "amax") and n in self.value and ir.by_name(self.value[n]).kind == "reduce":
                output_stores.append(self.value[n])
                final_outputs.append(n)
                continue
            # a pure layout node whose source is already stored shares that store
            store_name = f"store_{n.name}"
            cm = self.cmap.get(n)
            if cm is None:
                raise NotImplementedError(f"output {n.name} has no canonical map")
            shape = _shape(n)
            tref = TensorRef(n.name, _dtype(n), shape, _factors(cm, _contig_strides(shape), L, M, N))
            ir.add(Node(store_name, "store", args=(self.value[n],), tensor=tref))
            output_stores.append(store_name)
            final_outputs.append(n)

        attrs = {}
        if self.row_nodes:
            attrs["row_resident"] = True
        if self.kind == "spmm":
            attrs["fused_norm"] = op_name(a.target) == "spmm_sym"
        if self.kind in ("conv_fprop", "conv_dgrad", "conv_wgrad"):
            off = 2 if self.kind == "conv_fprop" else 3
            attrs["stride"], attrs["padding"], attrs["dilation"] = (list(a.args[off]), list(a.args[off + 1]),
                                                                    list(a.args[off + 2]))
            attrs["transposed"], attrs["groups"] = bool(a.args[off + 3]), int(a.args[off + 5])
            if self.kind == "conv_dgrad":
                attrs["input_shape"] = tuple(_shape(a.args[1]))
            if self.kind == "conv_wgrad":
                attrs["filter_shape"] = tuple(_shape(a.args[2]))
        if tuple_anchor:
            attrs["aux_getitems"] = aux_getitems
        if self.kind == "layernorm":
            attrs["eps"] = float(a.args[4]) if len(a.args) > 4 else 1e-5
            # mean / inv-std leave the kernel directly (fp32 per row), not through the epilogue
            for idx, nm in ((1, "aux_mean"), (2, "aux_rstd")):
                g = aux_getitems.get(idx)
                if g is not None and any(u.name not in part for u in g.users):
                    final_outputs.append(g)
                    output_stores.append(nm)
        consumed = [a] + folded + list(accum_nodes - {a}) + epi_nodes + list(aux_getitems.values())
        return PartitionTrace(self.kind, a, ir, self.inputs, final_outputs, output_stores,
                              mainloop_args, operands, consumed, attrs)

    # -- IR emission ------------------------------------------------------------------
    def _const(self, v) -> str:
        name = f"imm{self._const_id}"
        self._const_id += 1
        self.ir.add(Node(name, "const", value=float(v)))
        return name

    def _operand(self, x, epi_set) -> str:
        """IR value name for fx argument x (node or python scalar)."""
        if not isinstance(x, FxNode):
            if isinstance(x, bool):
                return self._const(1.0 if x else 0.0)
            if isinstance(x, (int, float)):
                return self._const(x)
            raise NotImplementedError(f"operand {x!r}")
        if x in self.value:
            return self.value[x]
        if x in epi_set:
            raise RuntimeError(f"{x.name} used before definition")
        # an input of the partition: becomes a load
        return self._load(x)

    def _load(self, x: FxNode) -> str:
        ir = self.ir
        cm = self.cmap.get(x)
        shape = _shape(x)
        if cm is None:
            if math.prod(shape) == 1:
                cm = Layout([[] for _ in shape])
            else:
                raise NotImplementedError(f"input {x.name} has no canonical map")
        tref = TensorRef(x.name, _dtype(x), shape, _factors(cm, _contig_strides(shape), ir.L, ir.M, ir.N))
        name = f"ld_{x.name}"
        ir.add(Node(name, "load", tensor=tref))
        self.value[x] = name
        if x not in self.inputs:
            self.inputs.append(x)
        return name

    def _emit(self, n: FxNode, epi_set):
        ir = self.ir
        name = op_name(n.target)
        if name in LAYOUT_OPS or name in PASSTHROUGH_OPS:
            src = n.args[0]
            if src in self.value:
                self.value[n] = self.value[src]
            elif src in epi_set:
                raise RuntimeError(f"{src.name} used before definition")
            else:
                # layout op on a partition input: load the input itself through the map
                # that backward propagation gave it (the view / permute never runs)
                self.value[n] = self._load(src) if isinstance(src, FxNode) else self._const(src)
            return
        if name in BINARY_OPS:
            a0 = self._operand(n.args[0], epi_set)
            a1 = self._operand(n.args[1], epi_set)
            extra = {}
            if name in ("add", "sub") and (len(n.args) > 2 or "alpha" in n.kwargs):
                alpha = n.args[2] if len(n.args) > 2 else n.kwargs["alpha"]
                if alpha != 1:
                    sc = self._const(alpha)
                    tmp = f"{n.name}_alpha"
                    ir.add(Node(tmp, "compute", op="mul", args=(a1, sc)))
                    a1 = tmp
            ir.add(Node(n.name, "compute", op=name, args=(a0, a1), attrs=extra))
        elif name in UNARY_OPS:
            ir.add(Node(n.name, "compute", op=name, args=(self._operand(n.args[0], epi_set),)))
        elif name == "rsub":
            a0 = self._operand(n.args[0], epi_set)
            a1 = self._operand(n.args[1], epi_set)
            ir.add(Node(n.name, "compute", op="sub", args=(a1, a0)))
        elif name == "gelu":
            approx = n.kwargs.get("approximate", n.args[1] if len(n.args) > 1 else "none")
            ir.add(Node(n.name, "compute", op="gelu", args=(self._operand(n.args[0], epi_set),),
                        attrs={"approximate": approx}))
        elif name == "gelu_backward":
            approx = n.kwargs.get("approximate", n.args[2] if len(n.args) > 2 else "none")
            ir.add(Node(n.name, "compute", op="gelu_backward",
                        args=(self._operand(n.args[0], epi_set), self._operand(n.args[1], epi_set)),
                        attrs={"approximate": approx}))
        elif name == "rand_like":
            ir.add(Node(n.name, "rand"))
        elif name == "one_hot":
            ir.add(Node(n.name, "compute", op="one_hot", args=(self._operand(n.args[0], epi_set),),
                        attrs={"num_classes": int(n.kwargs.get("num_classes", n.args[1] if len(n.args) > 1 else -1))}))
        elif name in ("sum", "amax"):
            self._emit_reduce(n, "sum" if name == "sum" else "max", epi_set)
            return
        elif name in ROW_EPILOGUE_OPS and n in self.row_nodes:
            shape = _shape(n)
            dim = int(n.args[1] if name == "_softmax" else n.args[2]) % len(shape)
            if dim != len(shape) - 1 or shape[-1] != ir.N or ir.N > ROW_EPILOGUE_MAX_N:
                raise NotImplementedError("a softmax fused into a GEMM must run over the whole last dim (<= 512 columns)")
            if name == "_softmax":
                if len(n.args) > 2 and n.args[2]:
                    raise NotImplementedError("half_to_float softmax is not fused into a GEMM")
                args = (self._operand(n.args[0], epi_set),)
            else:
                args = (self._operand(n.args[0], epi_set), self._operand(n.args[1], epi_set))
            ir.add(Node(n.name, "rowop", op=ROW_EPILOGUE_OPS[name], args=args))
        else:
            raise NotImplementedError(f"Doesn't support target {n.target}")
        self.value[n] = n.name

    def _emit_reduce(self, n: FxNode, op: str, epi_set):
        ir = self.ir
        src = n.args[0]
        dims = n.args[1] if len(n.args) > 1 else list(range(len(_shape(src))))
        keep = bool(n.args[2]) if len(n.args) > 2 else bool(n.kwargs.get("keepdim", False))
        if isinstance(dims, int):
            dims = [dims]
        sshape = _shape(src)
        dims = sorted(int(d) % len(sshape) for d in dims)
        cm = self.cmap.get(src)
        if cm is None:
            raise NotImplementedError(f"reduction source {src.name} has no canonical map")
        L, M, N = ir.L, ir.M, ir.N
        red_f: List[Factor] = []
        kept_dims = []
        for i, sub in enumerate(cm.dims):
            if i in dims:
                for sz, cs in sub:
                    red_f.extend(_split_dim(int(sz), int(cs), 0, L, M, N))
                if keep:
                    kept_dims.append([])
            else:
                kept_dims.append(list(sub))
        axes = set()
        for axis, extent in (("m", M), ("n", N)):
            covered = math.prod(f.size for f in red_f if f.axis == axis)
            if covered == 1:
                continue
            if covered != extent:
                raise NotImplementedError(f"partial reduction over axis {axis} ({covered} of {extent})")
            axes.add(axis)
        # the batch axis may be reduced fully, partly or not at all: the result simply has
        # no index factor for the reduced part and the atomics of different batches meet
        if any(f.axis == "l" for f in red_f):
            axes.add("l")
        if not (axes & {"m", "n"}):
            raise NotImplementedError("reduction over the batch axis only")
        if "n" in axes and "m" in axes:
            raise NotImplementedError("full-tensor reductions are not lowered")
        oshape = _shape(n)
        kept_map = Layout(kept_dims)
        assert tuple(kept_map.shape) == tuple(oshape), (kept_map.shape, oshape)
        tref = TensorRef(n.name, _dtype(n), oshape, _factors(kept_map, _contig_strides(oshape), L, M, N))
        ir.add(Node(n.name, "reduce", op=op, args=(self._operand(src, epi_set),), tensor=tref,
                    attrs={"axes": frozenset(axes)}))
        self.value[n] = n.name
        # downstream layout ops on a reduction output are views of the stored vector
        self.cmap[n] = kept_map


def trace_partition(gm: GraphModule, partition: Optional[Sequence[str]] = None) -> PartitionTrace:
    """Lower one partition.  With `partition=None` every call_function node of the graph
    belongs to it (the shape of the reference's per-node unit tests)."""
    if partition is None:
        # everything except (a) what consumes a finished reduction (the partitioner keeps
        # reductions as leaves of their partition, pass_fusion.py:817-842) and (b) what
        # feeds the heavy op, apart from layout nodes folded into a GEMM operand (a fusible
        # node may not share a partition with a nucleus it feeds, pass_fusion.py:760-815)
        anchors = [n for n in gm.graph.nodes if n.op == "call_function" and op_name(n.target) in ANCHOR_OPS]
        mains = [n for n in anchors if ANCHOR_OPS[op_name(n.target)] in ("gemm", "bmm")]
        if len(anchors) == 2 and len(mains) == 1:
            anchors = mains          # GEMM + softmax: the softmax rides in the GEMM's epilogue
        feeds = set()
        if len(anchors) == 1:
            is_mm = ANCHOR_OPS[op_name(anchors[0].target)] in ("gemm", "bmm")
            stack = [(x, True) for x in anchors[0].all_input_nodes]
            while stack:
                x, chain = stack.pop()
                if x.op != "call_function":
                    continue
                foldable = is_mm and chain and op_name(x.target) in ("permute", "view", "_unsafe_view", "clone", "expand")
                if not foldable:
                    feeds.add(x)
                for y in x.all_input_nodes:
                    stack.append((y, foldable))
        after_reduce = set()
        partition = []
        for n in gm.graph.nodes:
            if n.op != "call_function" or n in feeds:
                continue
            if any(x in after_reduce for x in n.all_input_nodes):
                after_reduce.add(n)
                continue
            partition.append(n.name)
            if op_name(n.target) in ("sum", "amax"):
                after_reduce.add(n)
    tr = _Tracer(gm, partition)
    return tr.run()
