"""The reference's own graph front end on top of this back end.

The reference compiles a model by tracing its joint forward + backward graph with AOT autograd
and running, in order, `GTLFrontend`, `pass_loss_elimination`, `pass_decomposition`, `pass_cse`,
`pass_constant_propagation`, `pass_fusion` and `pass_clean_up` on it (benchmark/bert/bert.py:35-47;
the passes live in python/gtl/compiler/passes/).  `pass_fusion` solves the partitioning MILP and
hands every partition to `EVTFuser` (pass_fusion.py:1356-1374).  All of that is kept: this module
only makes the reference's package importable next to this one and puts
`evt_ae_b200.fuser.EVTFuser` where `gtl.compiler.passes.evt_fuser.EVTFuser` is looked up, so the
partitions the reference finds are lowered to the sm_100a kernels instead of CUTLASS.

The reference is not part of this repository: `install(ref_root)` needs a checkout of it (or
`EVT_REFERENCE_ROOT`).  What is stood in for, and why:
  * `cutlass` (its fork of the CUTLASS Python package, only `CACHE_FILE` is read by pass_fusion),
    `pydot`, `seaborn`, `matplotlib` (graph drawing), `nvtx`: not installed, not needed to partition;
  * `gtl.compiler.passes.evt_fuser` -> this package's fuser; `gtl.compiler.passes.nv_fuser`
    (TorchScript fusion of elementwise-only partitions) -> a fuser that declines, those partitions
    stay eager;
  * `torch._functorch.partitioners._extract_graph_with_inputs_outputs` gained a required argument
    after the reference was written; a wrapper restores the three-argument form for its passes;
  * tensors the passes create on "cuda" are created on the CPU when no GPU is present
    (`cpu_constants()`), so the compile step also runs on a build machine.
"""
from __future__ import annotations

import contextlib
import importlib
import os
import sys
import types
from typing import Callable, Optional

import torch

_installed: Optional[str] = None


def _stub(name: str, **attrs):
    if name in sys.modules and not isinstance(sys.modules[name], _Stub):
        return sys.modules[name]            # the real package is installed: use it
    m = _Stub(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


class _Stub(types.ModuleType):
    pass


class _DecliningFuser:
    """Stands where the reference's TorchScript fuser is looked up: fuses nothing."""

    @staticmethod
    def fusible(partition) -> bool:
        return False

    def trace(self, graph_module, partition):
        raise RuntimeError("the TorchScript fuser of the reference is not part of this back end")


def install(ref_root: Optional[str] = None) -> str:
    """Makes `gtl.compiler.passes.*` of the reference checkout at `ref_root` importable with this
    package's fuser in place of the reference's.  Idempotent; returns the root used."""
    global _installed
    ref_root = ref_root or _installed or os.environ.get("EVT_REFERENCE_ROOT")
    if not ref_root or not os.path.isdir(os.path.join(ref_root, "python", "gtl", "compiler", "passes")):
        raise FileNotFoundError("a checkout of the reference (python/gtl/compiler/passes) is needed: pass its root "
                                "or set EVT_REFERENCE_ROOT")
    if _installed == ref_root:
        return ref_root
    _stub("pydot")
    _stub("seaborn")
    mpl = _stub("matplotlib")
    mpl.pyplot = _stub("matplotlib.pyplot")
    _stub("nvtx")
    _stub("cutlass", CACHE_FILE=os.path.join(os.environ.get("TMPDIR", "/tmp"), "evt_b200_partition_cache.db"))
    base = os.path.join(ref_root, "python", "gtl")
    # the package __init__ files import the CUTLASS-based fuser: empty packages with the real
    # directories as search path let the import system find the pass modules without running them
    for name, path in (("gtl", base), ("gtl.compiler", os.path.join(base, "compiler")),
                       ("gtl.compiler.passes", os.path.join(base, "compiler", "passes"))):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = [path]
            sys.modules[name] = m
    from . import fuser
    _stub("gtl.compiler.passes.evt_fuser", EVTFuser=fuser.EVTFuser)
    _stub("gtl.compiler.passes.nv_fuser", NVFuser=_DecliningFuser)
    from torch._functorch import partitioners as tp
    import inspect
    if "outputs_descs" in inspect.signature(tp._extract_graph_with_inputs_outputs).parameters:
        new = tp._extract_graph_with_inputs_outputs

        def three_argument_form(joint_graph, inputs, outputs, *unused, **unused_kw):
            return new(joint_graph, inputs, outputs, [None] * len(outputs), None, True)
        tp._extract_graph_with_inputs_outputs = three_argument_form
    _installed = ref_root
    return ref_root


@contextlib.contextmanager
def cpu_constants():
    """Inside this context every tensor asked for on "cuda" is made on the CPU.  The reference's
    passes build a handful of scalar constants that way; with a GPU present nothing is changed."""
    if torch.cuda.is_available():
        yield
        return
    from torch.overrides import TorchFunctionMode

    def is_cuda(x):
        return (isinstance(x, str) and x.startswith("cuda")) or (isinstance(x, torch.device) and x.type == "cuda")

    class OnCpu(TorchFunctionMode):
        def __torch_function__(self, func, types_, args=(), kwargs=None):
            kwargs = dict(kwargs or {})
            if is_cuda(kwargs.get("device")):
                kwargs["device"] = "cpu"
            return func(*tuple("cpu" if is_cuda(x) else x for x in args), **kwargs)
    with OnCpu():
        yield


def passes():
    """The reference's pass pipeline as (name, callable(joint_module) -> joint_module), in the order
    of benchmark/bert/bert.py:35-47."""
    install()
    P = lambda n: importlib.import_module("gtl.compiler.passes." + n)
    in_place = lambda f: (lambda m: (f(m, m.graph), m)[1])
    return [("frontend", lambda m: P("pass_frontend").GTLFrontend()(m)[0]),
            ("loss_elimination", in_place(P("pass_eliminate_loss").pass_loss_elimination)),
            ("decomposition", in_place(P("pass_decomposition").pass_decomposition)),
            ("cse", in_place(P("pass_cse").pass_cse)),
            ("constant_propagation", in_place(P("pass_constant_propagation").pass_constant_propagation)),
            ("fusion", in_place(P("pass_fusion").pass_fusion)),
            ("clean_up", in_place(P("pass_clean_up").pass_clean_up))]


def joint_optimization(joint_module, log: Optional[Callable[[str], None]] = None):
    """What the reference's benchmarks pass as `joint_compiler` (benchmark/bert/bert.py:35-47), with
    the fused nodes built by this package.  Call it where the reference calls its own: inside the
    partition function of AOT autograd."""
    with cpu_constants():
        for name, run in passes():
            joint_module = run(joint_module)
            if log is not None:
                log(f"{name}: {len(list(joint_module.graph.nodes))} nodes")
    joint_module.recompile()
    return joint_module


def fused_nodes(joint_module):
    """The fused operators `joint_optimization` planted, in graph order."""
    from .fused_ops import FusedOpBase
    return [n.target for n in joint_module.graph.nodes if n.op == "call_function" and isinstance(n.target, FusedOpBase)]
