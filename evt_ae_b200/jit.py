"""Generated CUDA source -> cubin, cached in-tree.

The reference JIT-compiles every fused kernel through the CUTLASS Python compiler and keeps
the binaries in `compiled_cache.db` (python/gtl/compiler/passes/evt_fuser.py:738-746;
python/gtl/ops/reduce_apply_operation.py:120-136).  Here each translation unit is compiled
by nvcc for sm_100a into `evt_ae_b200/_kcache/<hash>.cubin`; the hash covers the generated
source and the hand-written headers it includes, so editing a kernel invalidates the cache
(images built from older headers are never picked up again; `prune()` removes them, least
recently used first, when the directory outgrows a budget).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import tempfile
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
CACHE_DIR = os.environ.get("EVT_B200_CACHE", os.path.join(HERE, "_kcache"))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]

_lock = threading.Lock()
_header_digest = None
_pending: "List[str] | None" = None


class deferred:
    """`with jit.deferred() as d:` — compile_cubin() only records the sources it is asked for
    (returning the path the image will have); `d.flush()` then builds the missing ones in
    parallel.  Used to build many kernel variants on a box without a GPU."""

    def __enter__(self):
        global _pending
        _pending = []
        return self

    def __exit__(self, *exc):
        global _pending
        self.sources = _pending or []
        _pending = None
        return False

    def flush(self, workers: int = 8) -> int:
        todo = [s for s in dict.fromkeys(self.sources) if not os.path.exists(cubin_path_for(s))]
        compile_many(todo, workers)
        return len(todo)



def _headers_digest() -> str:
    global _header_digest
    if _header_digest is None:
        h = hashlib.sha256()
        for f in sorted(os.listdir(CSRC)):
            if f.endswith(".cuh"):
                with open(os.path.join(CSRC, f), "rb") as fh:
                    h.update(f.encode())
                    h.update(fh.read())
        _header_digest = h.hexdigest()
    return _header_digest


def cubin_path_for(source: str) -> str:
    key = hashlib.sha256((_headers_digest() + source).encode()).hexdigest()[:24]
    return os.path.join(CACHE_DIR, key + ".cubin")


def compile_cubin(source: str, verbose: bool = False) -> str:
    """Returns the path of the cubin for `source`, compiling it if it is not cached."""
    path = cubin_path_for(source)
    if os.path.exists(path):
        try:
            os.utime(path)          # marks the image as recently used for prune()
        except OSError:
            pass
        return path
    if _pending is not None:
        _pending.append(source)
        return path
    os.makedirs(CACHE_DIR, exist_ok=True)
    with tempfile.TemporaryDirectory() as td:
        cu = os.path.join(td, "kernel.cu")
        with open(cu, "w") as f:
            f.write(source)
        tmp_out = os.path.join(td, "kernel.cubin")
        cmd = [NVCC, "-cubin", "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS, "-I", CSRC,
               "-Xptxas", "-v", "-o", tmp_out, cu]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            keep = path + ".failed.cu"
            with open(keep, "w") as f:
                f.write(source)
            raise RuntimeError(f"nvcc failed (source kept at {keep}):\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        with open(path + ".log", "w") as f:
            f.write(r.stderr)
        with open(path + ".cu", "w") as f:
            f.write(source)
        with _lock:
            os.replace(tmp_out, path)
    return path


def compile_many(sources: Iterable[str], workers: int = 8) -> List[str]:
    sources = list(sources)
    with ThreadPoolExecutor(max_workers=workers) as ex:
        return list(ex.map(compile_cubin, sources))


def cache_entries() -> List[Tuple[str, float, int]]:
    """(key, last use, bytes incl. the kept source and compiler log) of every cached image."""
    out = []
    if not os.path.isdir(CACHE_DIR):
        return out
    for f in os.listdir(CACHE_DIR):
        if f.endswith(".cubin"):
            p = os.path.join(CACHE_DIR, f)
            size = sum(os.path.getsize(q) for q in (p, p + ".cu", p + ".log") if os.path.exists(q))
            out.append((f[:-6], os.path.getmtime(p), size))
    return out


def prune(max_bytes: int) -> int:
    """Removes least recently used images (with their sources and logs) until the cache holds at
    most `max_bytes`; returns the number of images removed.  Anything removed is rebuilt on its
    next use."""
    entries = sorted(cache_entries(), key=lambda e: e[1])
    total = sum(e[2] for e in entries)
    removed = 0
    with _lock:
        for key, _, size in entries:
            if total <= max_bytes:
                break
            base = os.path.join(CACHE_DIR, key + ".cubin")
            for q in (base, base + ".cu", base + ".log"):
                if os.path.exists(q):
                    os.remove(q)
            total -= size
            removed += 1
    return removed
