"""The C-ABI library builds, loads without a GPU and exports what include/evt_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from evt_ae_b200.build import build_library
    from evt_ae_b200 import runtime
    build_library()
    return runtime.load_library()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "evt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(evtb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_functions()
    assert "evtb_plan_create" in names and "evtb_launch" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/evt_b200.h but not exported"


def test_python_binding_lists_the_same_symbols(lib):
    from evt_ae_b200 import runtime
    assert sorted(runtime.EXPORTED_SYMBOLS) == _declared_functions()


def test_status_strings_and_argument_validation(lib):
    from evt_ae_b200 import runtime
    assert lib.evtb_version() >= 1
    assert lib.evtb_status_string(0) == b"ok"
    d = runtime.evtb_desc()
    d.kind = 99
    h = ctypes.c_void_p()
    st = lib.evtb_plan_create(ctypes.byref(d), ctypes.byref(h))
    assert st == 1 and not h.value          # EVTB_EINVAL, before any CUDA call
    d.kind = runtime.EVTB_GEMM
    d.M, d.N, d.K, d.L = 128, 128, 64, 1
    d.tile_n, d.stages = 48, 4               # not a multiple of 32
    d.image_path, d.entry = b"/nonexistent.cubin", b"k"
    d.threads, d.smem_bytes = 192, 1024
    st = lib.evtb_plan_create(ctypes.byref(d), ctypes.byref(h))
    assert st == 1
    assert b"tile_n" in lib.evtb_last_error()


def test_fused_op_refuses_cpu_tensors():
    import torch
    import partitions as P
    from evt_ae_b200.fuser import fuse_module
    if torch.cuda.is_available():
        pytest.skip("checks the no-GPU behaviour")
    case = P.mm_plain(128, 256, 64, False, True)
    gm, fused = fuse_module(case.module, case.inputs)
    with pytest.raises(RuntimeError):
        gm(*case.inputs)


def test_reduction_arena_hands_out_disjoint_zeroed_views():
    """One memset per step instead of one fill kernel per reduction target (host logic only)."""
    import torch
    from evt_ae_b200.fused_ops import ReductionArena
    arena = ReductionArena("cpu", floats=1024)
    a = arena.take((10, 3), "cpu")
    b = arena.take((70,), "cpu")
    assert a.shape == (10, 3) and b.shape == (70,) and a.dtype == torch.float32
    assert a.data_ptr() % 256 == arena.buf.data_ptr() % 256 and b.data_ptr() - a.data_ptr() == 64 * 4
    a.fill_(1.0)
    b.fill_(2.0)
    assert arena.take((2000,), "cpu") is None            # exhausted: callers fall back to their own fill
    arena.reset()
    assert float(arena.buf.abs().sum()) == 0.0 and arena.off == 0
    with arena:
        from evt_ae_b200 import fused_ops
        assert fused_ops._ACTIVE_ARENA is arena
    assert fused_ops._ACTIVE_ARENA is None


def test_integration_note_shows_the_current_descriptor():
    """The ctypes mirror of evtb_desc printed in INTEGRATION.md is what a maintainer copies: it
    must list the fields of the binding this package uses, in order, and the header must declare
    them in the same order."""
    from evt_ae_b200 import runtime
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    block = text[text.index("class evtb_desc(ctypes.Structure):"):]
    block = block[: block.index("\n\n")]
    doc_fields = re.findall(r'\("(\w+)",', block)
    mine = [f[0] for f in runtime.evtb_desc._fields_]
    assert doc_fields == mine, (doc_fields, mine)
    header = open(os.path.join(ROOT, "include", "evt_b200.h")).read()
    body = header[header.index("typedef struct evtb_desc {") + len("typedef struct evtb_desc {"): header.index("} evtb_desc;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    header_fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if decl:
            names = decl.split(None, 1)[1] if not decl.startswith("const") else decl.split(None, 2)[2]
            header_fields += [re.sub(r"[\*\s]|\[\d+\]", "", n) for n in names.split(",")]
    assert header_fields == mine, (header_fields, mine)
