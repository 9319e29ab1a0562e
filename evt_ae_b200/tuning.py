"""Measured kernel configurations for fused nodes.

The reference picks its CUTLASS tile descriptions with a profile-guided tuner whose results
live in a cache keyed by problem size and epilogue census
(python/gtl/compiler/autotuner/tuner_base.py:57-152, gemm_tuner.py:126-153).  Here the
candidates are few (tile width, ring depth, number of epilogue warps, K splits), so the tuner
is a plain sweep: `python -m evt_ae_b200.tune` times every candidate of every GEMM node of a
workload on the GPU and records the winner in `tuned_tiles.json` beside this file;
`lookup()` is consulted by the fused-op constructors before the closed-form choice of
`fused_ops.pick_gemm_tile`.  Keys hold the epilogue signature hash, the problem size, the
operand majors and the dtype, so a table entry can never be applied to a different kernel.

The other node kinds go through the same table with keys `row|...`, `conv|...`, `spmm|...`
(`key_for_node`): threads per row / CTA size of the softmax and LayerNorm kernels (the reference's
reduce-apply tuner, autotuner/reduce_apply_tuner.py:32-275), channel-tile width, ring depth and
epilogue warps of the convolutions (autotuner/conv_tuner.py:27-147), and the row-length threshold,
task length and unrolls of the SpMM.  `lookup_config` returns the stored fields as a dict.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

from .codegen import GemmTileConfig

TABLE_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuned_tiles.json")
_table: Optional[Dict[str, dict]] = None


def key_for(ir, M: int, N: int, K: int, L: int, a_major: str, b_major: str, dtype) -> str:
    sig = hashlib.sha256(ir.signature().encode()).hexdigest()[:16]
    return f"{sig}|{L}x{M}x{N}x{K}|{a_major}{b_major}|{str(dtype).replace('torch.', '')}"


def key_for_node(kind: str, ir, shape, dtype) -> str:
    """Key of a row-kernel / convolution / SpMM node: kind, epilogue signature, problem shape, dtype."""
    sig = hashlib.sha256(ir.signature().encode()).hexdigest()[:16]
    return f"{kind}|{sig}|{'x'.join(str(int(s)) for s in shape)}|{str(dtype).replace('torch.', '')}"


def lookup_config(key: str) -> Optional[dict]:
    e = _load().get(key)
    return dict(e) if e is not None else None


def _load() -> Dict[str, dict]:
    global _table
    if _table is None:
        if os.environ.get("EVT_B200_NO_TUNED", "0") == "1" or not os.path.exists(TABLE_PATH):
            _table = {}
        else:
            with open(TABLE_PATH) as f:
                _table = json.load(f)
    return _table


def lookup(key: str) -> Optional[GemmTileConfig]:
    e = _load().get(key)
    if e is None:
        return None
    return GemmTileConfig(bn=int(e["bn"]), stages=int(e["stages"]), epi_warps=int(e["epi_warps"]),
                          split_k=int(e["split_k"]), cta_pair=bool(e.get("cta_pair", 0)))


def save(entries: Dict[str, dict], path: str = TABLE_PATH) -> None:
    """Merge `entries` into the table at `path` (sorted keys, stable diffs)."""
    cur = {}
    if os.path.exists(path):
        with open(path) as f:
            cur = json.load(f)
    cur.update(entries)
    with open(path, "w") as f:
        json.dump(cur, f, indent=1, sort_keys=True)
        f.write("\n")
    global _table
    _table = None
