"""Data-parallel gradient exchange for the training workloads.

The reference is single-GPU (no NCCL, no torch.distributed anywhere in its tree); the
benchmark configuration asks for data parallelism over 2/4/8 GPUs of one box with an NCCL
all-reduce of the gradients over NVLink and nothing else partitioned.  One process per GPU;
gradients are packed into a few large flat buckets (NVSwitch gives every peer full bandwidth,
so bucket size is chosen for launch latency, not link count) and summed with
`torch.distributed.all_reduce`, then averaged and unpacked in place.  Every tensor starts on
a 256-byte boundary of its bucket and bucket lengths are multiples of 256 bytes, so the pack /
unpack kernels and the collective always take their vector paths.  Works on any backend:
`nccl` on GPUs, `gloo` on CPU for the host-logic tests.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist


class GradAllReducer:
    ALIGN_BYTES = 256

    def __init__(self, grads: Dict[str, torch.Tensor], bucket_bytes: int = 64 << 20, group=None, average: bool = True):
        """`grads`: name -> tensor (shapes / dtypes / device of what will be reduced every step;
        the same names in the same order on every rank)."""
        self.group = group
        self.average = average
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.names = sorted(grads)
        self.buckets: List[Tuple[torch.Tensor, List[Tuple[str, int, int]]]] = []
        by_dtype: Dict[torch.dtype, List[str]] = {}
        for n in self.names:
            by_dtype.setdefault(grads[n].dtype, []).append(n)
        for dt, names in by_dtype.items():
            cur: List[Tuple[str, int, int]] = []
            cur_elems = 0
            esize = torch.empty((), dtype=dt).element_size()
            limit = max(1, bucket_bytes // esize)
            gran = max(1, self.ALIGN_BYTES // esize)       # elements per 256-byte granule
            for n in names:
                k = grads[n].numel()
                if cur and cur_elems + k > limit:
                    self._close(cur, cur_elems, dt, grads[names[0]].device)
                    cur, cur_elems = [], 0
                cur.append((n, cur_elems, k))
                cur_elems += (k + gran - 1) // gran * gran
            if cur:
                self._close(cur, cur_elems, dt, grads[names[0]].device)

    def _close(self, entries, elems, dtype, device):
        # zero-filled once: the padding between tensors takes part in the sum on every rank
        self.buckets.append((torch.zeros(elems, dtype=dtype, device=device), list(entries)))

    @property
    def bytes_per_step(self) -> int:
        return sum(b.numel() * b.element_size() for b, _ in self.buckets)

    def allreduce(self, grads: Dict[str, torch.Tensor]) -> None:
        """Sum (or average) `grads` over all ranks, in place."""
        if self.world == 1:
            return
        for flat, entries in self.buckets:
            views = [flat[o:o + k].view(grads[n].shape) for n, o, k in entries]
            srcs = [grads[n] for n, _, _ in entries]
            torch._foreach_copy_(views, srcs)
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
            if self.average:
                flat.div_(self.world)
            torch._foreach_copy_(srcs, views)


class OverlappedStep:
    """A training step whose gradient exchange runs behind its backward pass.

    `make_parts()` returns a generator over the step: it yields a dict of the parameter gradients that
    became final since the last yield, any number of times, and last a tuple whose second element is the
    dict of the remaining gradients (the workloads' `step_parts`).  Every stretch between two yields is
    captured as its own CUDA graph (one memory pool, replayed in order); `replay()` replays them and,
    after each, all-reduces that stretch's gradients on a second stream while the next graph runs.  Only
    the last stretch's exchange is exposed.  `final` is the tuple the generator ended with."""

    def __init__(self, make_parts, group=None):
        pool = torch.cuda.graph_pool_handle()
        gen = make_parts()
        self.segments: List[list] = []      # [graph, gradients it finishes, their reducer]
        self.final = None
        while self.final is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool, capture_error_mode="thread_local"):
                part = next(gen)
            if isinstance(part, tuple):
                self.final = part
                part = part[1]
            self.segments.append([g, dict(part), None])
        gen.close()
        self.comm = torch.cuda.Stream()
        for seg in self.segments:
            if seg[1]:
                seg[2] = GradAllReducer(seg[1], group=group)

    @property
    def grads(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for _, part, _ in self.segments:
            out.update(part)
        return out

    @property
    def bytes_per_step(self) -> int:
        return sum(red.bytes_per_step for _, _, red in self.segments if red is not None)

    def replay(self) -> None:
        main = torch.cuda.current_stream()
        for g, part, red in self.segments:
            g.replay()
            if red is not None:
                self.comm.wait_stream(main)
                with torch.cuda.stream(self.comm):
                    red.allreduce(part)
        main.wait_stream(self.comm)
