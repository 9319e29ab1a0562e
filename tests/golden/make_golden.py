"""Generates tests/golden/golden.npz by running the REFERENCE's own fused-node test modules.

Run where a checkout of the reference is available (it is not part of this repository):

    PYTHONPATH=. python tests/golden/make_golden.py <path to the reference checkout>

For every entry of `cases.CASES` the named test method of unittest/evt_fuser/<file> is
executed as written, with three substitutions: `torch.randn`, `torch.randn_like` and
`torch.rand_like` return seeded CPU tensors (`cases.Draws`), `device="cuda"` is ignored, and
`self.util_test_evt_fuser(cls, inputs)` -- which in the reference runs the fuser and compares
with the eager module -- only runs the eager module `cls()` on the inputs upcast to fp32
(the reference's own oracle, python/gtl/helper/test_helper.py:78-104).  The inputs the test
built are compared bit for bit with `cases.golden_inputs(name)`; the outputs are sampled at
`cases.sample_index` and stored with a few checksums.
"""
from __future__ import annotations

import ast
import os
import sys
import textwrap
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def _patched_torch(draws: cases.Draws):
    t = types.ModuleType("torch_patched")
    t.__dict__.update(torch.__dict__)

    def randn(*shape, dtype=torch.float32, device=None, **kw):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        return draws.randn(shape, dtype)
    t.randn = randn
    t.randn_like = lambda x, **kw: draws.randn_like(x)
    t.rand_like = lambda x, **kw: draws.rand_like(x)
    return t


class _FakeSelf:
    def __init__(self):
        self.inputs = None
        self.outputs = None

    def util_test_evt_fuser(self, cls, inputs):
        self.inputs = list(inputs)
        mod = cls()
        up = [x.to(torch.float32) if x.dtype in (torch.float16, torch.bfloat16) else x for x in inputs]
        with torch.no_grad():
            out = mod(*up)
        self.outputs = [out] if isinstance(out, torch.Tensor) else list(out)


def run_reference_test(ref_root: str, fname: str, method: str, draws: cases.Draws):
    path = os.path.join(ref_root, "unittest", "evt_fuser", fname)
    tree = ast.parse(open(path).read())
    src = open(path).read()
    fn = None
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == method:
            fn = node
    if fn is None:
        raise KeyError(f"{method} not found in {path}")
    code = textwrap.dedent(ast.get_source_segment(src, fn))
    # the softmax-backward module names torch.float16 as the storage dtype; inputs are upcast
    code = code.replace("-1, torch.float16)", "-1, torch.float32)")
    import operator
    ns = {"torch": _patched_torch(draws), "operator": operator}
    exec(compile(code, path, "exec"), ns)
    fake = _FakeSelf()
    ns[method](fake)
    return fake.inputs, fake.outputs


def load_reference_leaves(ref_root: str):
    """Imports the reference's python/gtl/compiler/passes/pass_decomposition.py as it lies in the
    checkout, without running the package __init__ files above it (they import the fuser, which
    needs a CUTLASS fork that is not installable here): empty stand-in packages with the real
    directories as their __path__ let the normal import machinery find the submodules."""
    import importlib
    base = os.path.join(ref_root, "python", "gtl")
    for name, path in (("gtl", base), ("gtl.compiler", os.path.join(base, "compiler")),
                       ("gtl.compiler.passes", os.path.join(base, "compiler", "passes"))):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = [path]
            sys.modules[name] = m
    return importlib.import_module("gtl.compiler.passes.pass_decomposition")


def _store_outputs(store, key, outs):
    store[f"{key}/n_out"] = np.array(len(outs))
    for j, o in enumerate(outs):
        flat = o.detach().to(torch.float64).reshape(-1).numpy() if o.dtype != torch.bool else o.reshape(-1).numpy().astype(np.float64)
        idx = cases.sample_index(flat.size)
        store[f"{key}/{j}/shape"] = np.array(o.shape, dtype=np.int64)
        store[f"{key}/{j}/sample"] = flat[idx].astype(np.float32)
        store[f"{key}/{j}/sum"] = np.array(flat.sum())
        store[f"{key}/{j}/abs_sum"] = np.array(np.abs(flat).sum())


def reference_dropout_module(ref_root: str):
    """class Dropout1 as written inside unittest/evt_fuser/dropout.py:test_dropout."""
    import operator
    path = os.path.join(ref_root, "unittest", "evt_fuser", "dropout.py")
    src = open(path).read()
    for node in ast.walk(ast.parse(src)):
        if isinstance(node, ast.ClassDef) and node.name == "Dropout1":
            ns = {"torch": torch, "operator": operator}
            exec(compile(textwrap.dedent(ast.get_source_segment(src, node)), path, "exec"), ns)
            return ns["Dropout1"]()
    raise KeyError("Dropout1 not found")


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("EVT_REFERENCE_ROOT", "reference")
    store = {}
    # wrapped leaf functions of the reference's decomposition pass
    ref_leaves = load_reference_leaves(ref_root)
    for leaf in cases.LEAVES:
        with torch.no_grad():
            outs = cases.leaf_call(ref_leaves, leaf, cases.leaf_inputs(leaf))
        _store_outputs(store, f"leaf/{leaf}", list(outs))
        print("leaf", leaf, "ok:", [tuple(o.shape) for o in outs])
    # dropout: the reference module with the mask it drew
    mod = reference_dropout_module(ref_root)
    ins = cases.dropout_inputs()
    torch.manual_seed(cases.DROPOUT_SEED)
    with torch.no_grad():
        out, keep = mod(*[x.to(torch.float32) for x in ins])
    assert keep.dtype == torch.bool and abs(keep.float().mean().item() - (1 - cases.DROPOUT_P)) < 1e-2
    store["dropout/keep_bits"] = np.packbits(keep.reshape(-1).numpy())
    _store_outputs(store, "dropout", [out])
    print("dropout ok:", tuple(out.shape), "kept", keep.float().mean().item())
    for name, (fname, method, _, make_case) in cases.CASES.items():
        ref_in, ref_out = run_reference_test(ref_root, fname, method, cases.Draws(cases.SEED_BASE[name]))
        mine = cases.golden_inputs(name)
        assert len(mine) == len(ref_in), (name, len(mine), len(ref_in))
        for i, (a, b) in enumerate(zip(mine, ref_in)):
            assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b), f"{name}: input {i} differs"
        _store_outputs(store, name, ref_out)
        for j in cases.RANDOM_MASK_OUTPUTS.get(name, []):
            assert bool(ref_out[j].all()), f"{name}: the generated keep mask is not all ones"
        print(name, "ok:", [tuple(o.shape) for o in ref_out])
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **store)
    print("wrote", os.path.join(HERE, "golden.npz"))


if __name__ == "__main__":
    main()
