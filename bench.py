#!/usr/bin/env python
"""Benchmark of the fused-operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" = one pass of the workload over one batch of seeded synthetic input.  Rank 0
prints ONE JSON line.  `value` is measured with inputs resident in HBM; `e2e` goes through
the same public call with pinned HOST buffers (host->device copy of every input and
device->host copy of every output inside the timed region).  `roofline` describes the
dominant kernel, timed with CUDA events on the launching stream; `cpu_baseline` is the CPU
oracle (the unfused fp32 graph) timed on the host cores of this box.

With --impl reference the reference's own CPU path for the workload (the unfused eager
graph, which is what the reference's tests and its `-mt torch` mode run) is timed on the
host cores; no kernel of this repository is involved.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"],
                    tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# ----------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------

class Config0Workload:
    """BASELINE configuration 0: one fused GEMM, D = GELU(A@B + bias) + C with column sums
    and row maxima in the epilogue; M=16384, N=4096, K=1024, fp16, seeded."""
    name = "config0_fused_gemm_16384x4096x1024"
    metric = "fused GEMM TFLOP/s (GELU(A@B+bias)+C, colsum, rowmax in the epilogue)"
    unit = "TFLOP/s"
    dtype = "f16"

    def __init__(self, M=16384, N=4096, K=1024):
        from evt_ae_b200.workloads import cases as P
        self.M, self.N, self.K = M, N, K
        self.case = P.config0(M, N, K)
        self.flops = 2.0 * M * N * K
        # compulsory bytes: A, B, C read, D written (2 bytes each), bias, colsum, rowmax
        self.bytes = 2.0 * (M * K + K * N + 2 * M * N) + 2 * N + 4 * N + 4 * M

    def setup(self, device):
        from evt_ae_b200.fuser import fuse_module
        self.device = device
        self.host_inputs = [t.pin_memory() for t in self.case.inputs]
        self.dev_inputs = [t.to(device) for t in self.case.inputs]
        self.gm, self.fused = fuse_module(self.case.module, self.dev_inputs)
        self.host_out = None
        self.launches_per_step = 1
        # device-resident step = one replay of a captured graph (the fused node plus the fills of
        # its reduction targets), so that host launch cost does not bound kernels of tens of µs
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.gm(*self.dev_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from evt_ae_b200 import runtime
        before = runtime.KERNELS_ENQUEUED
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.s_out = self.gm(*self.dev_inputs)
        self.launches_per_step = runtime.KERNELS_ENQUEUED - before    # this library's kernels in one step

    def step_device(self):
        self.graph.replay()
        return self.s_out

    def step_e2e(self):
        ins = [t.to(self.device, non_blocking=True) for t in self.host_inputs]
        outs = self.gm(*ins)
        if self.host_out is None:
            self.host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        for h, o in zip(self.host_out, outs):
            h.copy_(o, non_blocking=True)
        return outs

    def h2d_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.host_inputs)

    def d2h_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.host_out or []))

    def value_from_ms(self, ms, n_gpus):
        return n_gpus * self.flops / (ms * 1e-3) / 1e12

    def check(self):
        self.fused.check_status()

    # CPU side (oracle): the unfused graph in fp32 eager
    def cpu_step(self):
        from oracle import run_unfused_fp32
        return run_unfused_fp32(self.case.module, self.case.inputs)

    cpu_sample = "the full configuration-0 expression in fp32 eager PyTorch (1 warm-up, median of 3)"


class Ffn1Workload(Config0Workload):
    """The dominant kernel of the BERT-large step on its own: FFN1, x W^T + b with the
    pre-activation and its tanh-GELU both stored (16384 x 4096 x 1024, bf16).  This is the small
    case profiler captures are taken on; inputs + outputs are 310 MB, larger than L2."""
    name = "bert_ffn1_gemm_16384x4096x1024_bf16"
    metric = "fused GEMM TFLOP/s (x W^T + b, pre-activation and GELU stored)"
    unit = "TFLOP/s"
    dtype = "bf16"
    cpu_sample = "the same expression in fp32 eager PyTorch (1 warm-up, median of 3)"

    def __init__(self, M=16384, N=4096, K=1024):
        from evt_ae_b200.workloads import cases as P
        self.M, self.N, self.K = M, N, K
        self.case = P.mm_bias_gelu(M, N, K, 512, M // 512, torch.bfloat16, "tanh")
        self.flops = 2.0 * M * N * K
        self.bytes = 2.0 * (M * K + K * N + 2 * M * N) + 2 * N


class Conv3x3Workload(Config0Workload):
    """A ResNet-50 convolution of BASELINE configuration 2 on its own: 3x3, 256 -> 256 channels on
    14 x 14 (conv4_x), batch 128, fp16, with the batch-norm statistics (E[y], E[y^2] per channel)
    in the epilogue."""
    name = "resnet50_conv4x_3x3_256_n128_f16"
    metric = "fused implicit-GEMM convolution TFLOP/s (3x3 conv + batch-norm statistics)"
    unit = "TFLOP/s"
    dtype = "f16"
    cpu_sample = "the same convolution + statistics in fp32 eager PyTorch (1 warm-up, median of 3)"

    def __init__(self):
        from evt_ae_b200.workloads import cases as P
        N, H, C, K = 128, 14, 256, 256
        self.case = P.conv_fprop_bn_stat(N, H, H, C, K, 3, 1)
        self.flops = 2.0 * N * H * H * K * C * 9
        self.bytes = 2.0 * (N * H * H * C + K * 9 * C + N * H * H * K) + 8 * K


class SpmmWorkload(Config0Workload):
    """The aggregation of BASELINE configuration 4 on its own: Y = D^-1/2 A D^-1/2 X on the
    Chung-Lu stand-in for ogbn-mag's paper graph (169,343 nodes), X fp32 [n, 128], int32 CSR,
    normalisation fused.  HBM-bound: value = compulsory bytes / time."""
    name = "gcn_spmm_sym_169343_f128_fp32"
    metric = "fused CSR SpMM GB/s (compulsory bytes: CSR + normalisation vector + X once + Y once)"
    unit = "GB/s"
    dtype = "f32"
    bound = "hbm"
    cpu_sample = "the same aggregation with torch.sparse on the host cores (1 warm-up, median of 3)"

    def __init__(self):
        from evt_ae_b200.workloads import cases as P
        self.case = P.spmm_case(169343, 585000, 128, "sym")
        self.flops = 0.0
        self.bytes = 0.0          # known once the plan exists (depends on the sampled nnz)

    def setup(self, device):
        super().setup(device)
        # compulsory bytes: row pointers, column indices, the per-node normalisation vector (there is
        # no value array), X read once, Y written once.  The epilogue's second read of X (the self
        # term) is NOT counted: it can be served from cache.
        n, nnz, F = self.fused.rows, self.fused.nnz, self.fused.F
        self.bytes = 4.0 * (n + 1) + 4.0 * nnz + 4.0 * n + 2 * 4.0 * n * F
        self.bytes_with_epilogue_inputs = self.fused.bytes_moved
        self.flops = 2.0 * self.fused.nnz * 128

    def value_from_ms(self, ms, n_gpus):
        return n_gpus * self.bytes / (ms * 1e-3) / 1e9


class GcnWorkload:
    """BASELINE configuration 4: two-layer GCN (128 -> 256 -> 40) on the Chung-Lu stand-in for
    ogbn-mag's paper graph (169,343 nodes, 585,000 sampled edges, symmetrised, de-duplicated, self
    loops: 1,167,363 nonzeros), forward + backward, cross-entropy over all nodes.  On N GPUs the
    destination rows are partitioned (balanced by nonzeros and rows) and every aggregation is
    preceded by a gather of its operand into local memory: the total work is fixed, so the
    scaling is strong."""
    name = "gcn_2layer_train_step_169343_nodes_f128_h256_c40"
    metric = "2-layer GCN train-step steps/s on the 169,343-node power-law graph (whole graph per step)"
    unit = "steps/s"
    dtype = "f32 features and first aggregation; bf16 dense maps and 40-wide aggregations, f32 accumulate"
    scaling = "strong"
    bound = "hbm"
    cpu_sample = "the same step (fp32 autograd, torch.sparse) on the host cores, whole graph (1 warm-up, median of 3)"

    def __init__(self):
        from evt_ae_b200.workloads import cases as P, gcn as wg
        import numpy as np
        self.wg = wg
        self.cfg = wg.GcnConfig()
        n = self.cfg.nodes
        r, c = P.chung_lu_graph(n, 585000)
        self.crow, self.col = P.csr_reference(r, c, n)
        deg = (self.crow[1:] - self.crow[:-1]).to(torch.float32)
        self.dinv = (deg + 1.0) ** -0.5
        self.x = P.seeded((n, self.cfg.in_feats), 301, 1.0, torch.float32)
        self.labels = torch.from_numpy(np.random.default_rng(302).integers(0, self.cfg.classes, size=n))
        self.params = wg.init_params(self.cfg, dtype=torch.bfloat16)
        self.nnz = int(self.col.shape[0])
        self.flops = 0.0

    def setup(self, device):
        import torch.distributed as dist
        from evt_ae_b200 import runtime
        wg, cfg = self.wg, self.cfg
        self.device = device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.p = {k: v.to(device) for k, v in self.params.items()}
        if self.world == 1:
            self.step = wg.GcnStep(cfg, self.nnz)
            self.r0, self.r1 = 0, cfg.nodes
            self.csr = (self.crow.to(device), self.col.to(device), self.dinv.to(device))
            parts = lambda: self.step.step_parts(self.p, *self.csr, self.s_x, self.s_labels)
        else:
            shard = wg.partition_rows(self.crow, self.col, self.dinv, self.world)[rank]
            self.shard = wg.GcnShard(cfg, shard, self.world, device)
            self.step = self.shard.step_impl
            self.r0, self.r1 = shard["r0"], shard["r1"]
            parts = lambda: self.shard.step_parts(self.p, self.s_x, self.s_labels)
        self.host = [self.x[self.r0:self.r1].contiguous().pin_memory(), self.labels[self.r0:self.r1].contiguous().pin_memory()]
        self.s_x = self.host[0].to(device)
        self.s_labels = self.host[1].to(device)
        self.host_loss = torch.zeros((), dtype=torch.float32).pin_memory()
        # warm-up (eager), then one CUDA graph per part between two exchanges
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._drive(parts())
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.step.check_status()
        before = runtime.KERNELS_ENQUEUED
        self.plan = []            # [(graph, exchange or None)]
        pool = torch.cuda.graph_pool_handle()
        gen = parts()
        while True:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool, capture_error_mode="thread_local"):
                item = next(gen)
            if item[0] == "done":
                self.plan.append((g, None))
                self.s_loss, self.s_grads = item[1], item[2]
                break
            self.plan.append((g, item[2]))
        self.launches_per_step = runtime.KERNELS_ENQUEUED - before
        # bytes of the dominant kernel (first aggregation, fp32, 128 wide) on this rank's rows
        rows = self.r1 - self.r0
        nnz_loc = int(self.crow[self.r1] - self.crow[self.r0])
        F = cfg.in_feats
        self.agg_bytes = 4.0 * (rows + 1) + 4.0 * nnz_loc + (4.0 * nnz_loc if self.world > 1 else 4.0 * cfg.nodes) \
            + 4.0 * cfg.nodes * F + 2.0 * rows * F
        self.bytes = self.agg_bytes

    @staticmethod
    def _drive(gen):
        item = next(gen)
        while item[0] != "done":
            item[2]()
            item = next(gen)
        return item[1], item[2]

    def _run(self):
        for g, exchange in self.plan:
            g.replay()
            if exchange is not None:
                exchange()
        return self.s_loss

    def step_device(self):
        return self._run()

    def step_e2e(self):
        self.s_x.copy_(self.host[0], non_blocking=True)
        self.s_labels.copy_(self.host[1], non_blocking=True)
        loss = self._run()
        self.host_loss.copy_(loss, non_blocking=True)
        return loss

    def h2d_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.host)

    def d2h_bytes(self):
        return 4

    def value_from_ms(self, ms, n_gpus):
        return 1e3 / ms

    def check(self):
        self.step.check_status()
        if not torch.isfinite(self.s_loss).item():
            raise SystemExit("non-finite loss")

    @property
    def bytes_exchanged_per_step(self):
        """gathered operands of one step: X (fp32, in_feats wide), z and dlogits (bf16, classes wide)"""
        cfg = self.cfg
        return cfg.nodes * (4 * cfg.in_feats + 2 * 2 * cfg.classes) if self.world > 1 else 0

    def dominant_kernel_hbm(self):
        """(name, algorithmic bytes, launch times in ms) of the first aggregation on this rank."""
        op = self.step.ops["agg_in"]
        if self.world == 1:
            byname = dict(crow=self.csr[0], col=self.csr[1], dinv=self.csr[2], x=self.s_x)
        else:
            # the gathered operand of the last step is still in the shard's buffer (no collective here:
            # only rank 0 runs this)
            full = self.shard._bufs[(self.cfg.in_feats, torch.float32, 0)]
            byname = dict(crow=self.shard.crow, col=self.shard.col, val=self.shard.val, x=full, x_own=self.s_x)
        args = [byname[n] for n in op.input_names + [a.name for a in op.args]]
        return ("agg_in (CSR SpMM 128-wide fp32 + self term, bf16 store)", self.agg_bytes,
                op.time_kernel(args, iters=20, warmup=3))

    def cpu_step(self):
        from oracle import gcn_ref
        return gcn_ref.loss_and_grads(self.params, self.crow, self.col, self.dinv, self.x, self.labels)


class VitWorkload:
    """BASELINE configuration 3: ViT-Base/16 (12 layers, hidden 768, 12 heads, MLP 3072), 224 x 224
    images (196 patches + class token = 197 tokens, padded to 200 masked-token rows for 16-byte row
    pitches), batch 128, bf16, one forward + backward step, 1000 random labels, random init.
    Patch embedding, encoder and its backward run on fused nodes inside one CUDA graph; patch
    extraction, the head on the 128 class-token rows and the loss are eager PyTorch."""
    name = "vit_base16_train_step_b128_224px_bf16"
    metric = "ViT-Base/16 train-step samples/s per B200"
    unit = "samples/s"
    dtype = "bf16"
    cpu_sample = ("2 encoder layers + embedding + head of the same model, batch 8, fp32 eager PyTorch forward + "
                  "backward; samples/s scaled by (2-layer FLOPs)/(12-layer FLOPs)")
    config_notes = ("197 tokens padded to 200 rows, padded keys masked (results equal the unpadded model's); "
                    "no optimizer update; head (128 x 1000 x 768) and loss in eager PyTorch")

    def __init__(self, B=128):
        from evt_ae_b200.workloads import vit as wv
        self.wv, self.cfg, self.B = wv, wv.VIT_BASE_16, B

    def setup(self, device):
        import torch.distributed as dist
        from evt_ae_b200 import runtime
        wv, cfg, B, dt = self.wv, self.cfg, self.B, torch.bfloat16
        self.device = device
        self.step = wv.VitStep(cfg, B, dtype=dt)
        self.p = {k: v.to(device) for k, v in wv.init_params(cfg, dtype=dt).items()}
        images, labels = wv.synthetic_batch(cfg, B)
        self.host = [images.to(dt).pin_memory(), labels.pin_memory()]
        self.s_images, self.s_labels = self.host[0].to(device), self.host[1].to(device)
        self.flops = self.step.gemm_flops

        def whole():
            tok, pm = self.step.embed_tokens(self.p, self.s_images)
            loss, grads, dtok = self.step.step(self.p, tok, self.s_labels)
            grads.update(self.step.embed_backward(dtok, pm))
            return loss, grads
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                whole()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.step.check_status()
        before = runtime.KERNELS_ENQUEUED
        self.graph = self.overlapped = self.segments = None
        if dist.is_initialized() and dist.get_world_size() > 1:
            # data parallel: the backward pass is cut after layers 9, 6 and 3; the gradients a stretch
            # finished are all-reduced on a second stream while the next stretch computes
            from evt_ae_b200.dp import OverlappedStep
            cuts = {(3 * cfg.layers) // 4, cfg.layers // 2, cfg.layers // 4}

            def parts():
                tok, pm = self.step.embed_tokens(self.p, self.s_images)
                for part in self.step.step_parts(self.p, tok, self.s_labels, cuts=cuts):
                    if isinstance(part, tuple):
                        loss, rest, dtok = part
                        rest = dict(rest)
                        rest.update(self.step.embed_backward(dtok, pm))
                        yield loss, rest
                    else:
                        yield part
            self.overlapped = OverlappedStep(parts)
            self.segments = self.overlapped.segments
            self.s_loss, self.s_grads = self.overlapped.final[0], self.overlapped.grads
        else:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                self.s_loss, self.s_grads = whole()
        self.launches_per_step = runtime.KERNELS_ENQUEUED - before
        self.host_loss = torch.zeros((), dtype=torch.float32).pin_memory()

    @property
    def bytes_reduced_per_step(self):
        return self.overlapped.bytes_per_step if self.overlapped is not None else 0

    def _run(self):
        if self.overlapped is not None:
            self.overlapped.replay()
        else:
            self.graph.replay()
        return self.s_loss

    def step_device(self):
        return self._run()

    def step_e2e(self):
        self.s_images.copy_(self.host[0], non_blocking=True)
        self.s_labels.copy_(self.host[1], non_blocking=True)
        loss = self._run()
        self.host_loss.copy_(loss, non_blocking=True)
        return loss

    def h2d_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.host)

    def d2h_bytes(self):
        return 4

    def value_from_ms(self, ms, n_gpus):
        return n_gpus * self.B / (ms * 1e-3)

    def check(self):
        self.step.check_status()
        if not torch.isfinite(self.s_loss).item():
            raise SystemExit("non-finite loss")

    def dominant_kernel(self):
        """the MLP up-projection GEMM (25,600 x 3072 x 768, bias + erf GELU, two stores)"""
        cfg, dt = self.cfg, torch.bfloat16
        op = self.step.n.ops["lin_dm_gelu"]
        T = cfg.tokens_padded * self.B
        x = torch.randn(T, cfg.dim, device=self.device, dtype=dt)
        byname = {"b": self.p["l0.ff1.b"], "x": x, "w": self.p["l0.ff1.w"]}
        args = [byname[n] for n in op.input_names + [a.name for a in op.args]]
        return "lin_dm_gelu (MLP GEMM 25600x3072x768 + bias + GELU, 2 stores)", op.flops, op.time_kernel(args, iters=20, warmup=3)

    def eager_gpu_ms(self, steps=5, warmup=3):
        """The same model and batch as plain eager PyTorch bf16 autograd on this GPU (the oracle's module
        moved to the device): the comparison the reference publishes.  A baseline, timed after the main
        measurement; none of this library's kernels run in it."""
        from oracle import vit_ref
        dt, dev = torch.bfloat16, self.device
        prepared = {k: v.detach().clone().to(dt).to(dev).requires_grad_(True) for k, v in self.p.items()}
        images, labels = self.s_images, self.s_labels
        for i in range(warmup + steps):
            if i == warmup:
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            vit_ref.loss_and_grads(None, self.cfg, images, labels, dtype=dt, device=dev, prepared=prepared)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def cpu_step(self):
        from oracle import vit_ref
        wv = self.wv
        if not hasattr(self, "_cpu"):
            import dataclasses
            cfg = dataclasses.replace(self.cfg, layers=2)
            self._cpu = (cfg, wv.init_params(cfg, dtype=torch.float32), *wv.synthetic_batch(cfg, 8))
        cfg, p, images, labels = self._cpu
        return vit_ref.loss_and_grads(p, cfg, images, labels)

    def cpu_value(self, seconds):
        return 8 / seconds * (2.0 / self.cfg.layers)


class ResNetWorkload:
    """BASELINE configuration 4: ResNet-50 (bottlenecks 3-4-6-3, v1.5 strides), 224 x 224 images, batch
    128, fp16, channels-last, batch norm on batch statistics, summed cross-entropy over 1000 random
    labels, random init; one forward + backward step.  Every convolution runs as fused tcgen05 nodes
    (forward with the batch-norm statistics in the epilogue -- the 7x7 stem on a window view of the
    image --, data gradient, weight gradient), batch-norm apply / backward passes are one-pass kernels
    and the max-pool of this library; the stem's weight gradient, average-pool, classifier and loss are
    library / eager PyTorch."""
    name = "resnet50_train_step_b128_224px_fp16_nhwc"
    metric = "ResNet-50 train-step samples/s per B200"
    unit = "samples/s"
    dtype = "f16"
    cpu_sample = ("the same network with one bottleneck per stage, batch 4, 128 x 128 images, fp32 eager PyTorch forward + "
                  "backward; samples/s scaled by the ratio of convolution FLOPs per sample")
    config_notes = ("own kernels: all 53 forward convolutions with BN statistics (the 7x7 stem through a 64-wide window "
                    "view), 52 data gradients, 52 weight gradients, every batch-norm / ReLU / residual pass, max-pool; library "
                    "or eager PyTorch: stem weight gradient, average pool, classifier, loss; no optimizer update")

    def __init__(self, B=128):
        from evt_ae_b200.workloads import resnet as wr
        self.wr, self.cfg, self.B = wr, wr.RESNET50, B

    def setup(self, device):
        import torch.distributed as dist
        from evt_ae_b200 import runtime
        wr, cfg, B, dt = self.wr, self.cfg, self.B, torch.float16
        self.device = device
        self.step = wr.ResNetStep(cfg, B, dtype=dt)
        self.p = {k: v.to(device) for k, v in wr.init_params(cfg, dtype=dt).items()}
        images, labels = wr.synthetic_batch(cfg, B)
        self.host = [images.to(dt).pin_memory(), labels.pin_memory()]
        self.s_images, self.s_labels = self.host[0].to(device), self.host[1].to(device)
        self.flops = self.step.conv_flops
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.step.step(self.p, self.s_images, self.s_labels)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.step.check_status()
        before = runtime.KERNELS_ENQUEUED
        self.graph = self.overlapped = self.segments = None
        if dist.is_initialized() and dist.get_world_size() > 1:
            # data parallel: the backward pass is cut after three quarters, half and a quarter of the
            # bottleneck blocks; a stretch's gradients are all-reduced on a second stream while the next
            # stretch computes
            from evt_ae_b200.dp import OverlappedStep
            nb = len(self.step.plan)
            cuts = {(3 * nb) // 4, nb // 2, nb // 4}
            self.overlapped = OverlappedStep(lambda: self.step.step_parts(self.p, self.s_images, self.s_labels, cuts=cuts))
            self.segments = self.overlapped.segments
            self.s_loss, self.s_grads = self.overlapped.final[0], self.overlapped.grads
        else:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                self.s_loss, self.s_grads = self.step.step(self.p, self.s_images, self.s_labels)
        self.launches_per_step = runtime.KERNELS_ENQUEUED - before
        self.host_loss = torch.zeros((), dtype=torch.float32).pin_memory()

    @property
    def bytes_reduced_per_step(self):
        return self.overlapped.bytes_per_step if self.overlapped is not None else 0

    def _run(self):
        if self.overlapped is not None:
            self.overlapped.replay()
        else:
            self.graph.replay()
        return self.s_loss

    def step_device(self):
        return self._run()

    def step_e2e(self):
        self.s_images.copy_(self.host[0], non_blocking=True)
        self.s_labels.copy_(self.host[1], non_blocking=True)
        loss = self._run()
        self.host_loss.copy_(loss, non_blocking=True)
        return loss

    def h2d_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.host)

    def d2h_bytes(self):
        return 4

    def value_from_ms(self, ms, n_gpus):
        return n_gpus * self.B / (ms * 1e-3)

    def check(self):
        self.step.check_status()
        if not torch.isfinite(self.s_loss).item():
            raise SystemExit("non-finite loss")

    def dominant_kernel(self):
        """the 3x3 convolution of the second stage (128 x 28 x 28 x 128 -> 128 channels) with the
        batch-norm statistics in its epilogue"""
        B, dt = self.B, torch.float16
        geo = (B, 28, 28, 128, 128, 3, 1)
        op = self.step.ops["fprop_" + "x".join(map(str, geo))]
        x = torch.randn(B, 28, 28, 128, device=self.device, dtype=dt)
        w = (torch.randn(128, 3, 3, 128, device=self.device) * 0.03).to(dt)
        byname = {"x": x, "w": w}
        args = [byname[n] for n in op.input_names + [a.name for a in op.args]]
        return "conv 3x3 fprop 128x28x28x128->128 + BN statistics", op.flops, op.time_kernel(args, iters=20, warmup=3)

    def eager_gpu_ms(self, steps=5, warmup=3):
        """The same model and batch as plain eager PyTorch fp16 autograd on this GPU, activations and
        filters channels-last in memory, cuDNN with its benchmark mode on (the oracle's module moved to the
        device): the comparison the reference publishes.  A baseline, timed after the main measurement;
        none of this library's kernels run in it."""
        from oracle import resnet_ref
        dt, dev = torch.float16, self.device
        prepared = {k: v.detach().clone().to(dt).to(dev).requires_grad_(True) for k, v in self.p.items()}
        arch = self.wr._arch(self.cfg)
        torch.backends.cudnn.benchmark = True
        for i in range(warmup + steps):
            if i == warmup:
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            resnet_ref.loss_and_grads(None, self.cfg, arch, self.s_images, self.s_labels, dtype=dt, device=dev, prepared=prepared)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def _cpu_cfg(self):
        import dataclasses
        return dataclasses.replace(self.cfg, layers=(1, 1, 1, 1), image=128)

    def cpu_step(self):
        from oracle import resnet_ref
        wr = self.wr
        if not hasattr(self, "_cpu"):
            cfg = self._cpu_cfg()
            self._cpu = (cfg, wr.init_params(cfg, dtype=torch.float32), *wr.synthetic_batch(cfg, 4))
        cfg, p, images, labels = self._cpu
        return resnet_ref.loss_and_grads(p, cfg, wr._arch(cfg), images, labels)

    def cpu_value(self, seconds):
        wr = self.wr
        small = wr.conv_flops_per_sample(self._cpu_cfg())
        full = wr.conv_flops_per_sample(self.cfg)
        return 4 / seconds * (small / full)


class BertLargeWorkload:
    """BASELINE configuration 1: BERT-large (24 layers, hidden 1024, 16 heads, FFN 4096,
    vocabulary 30522), batch 32 x sequence 512, bf16, one forward + backward step with the
    masked-LM head; uniform synthetic token ids, 15 % labelled positions, random init.
    The encoder + head step runs as one CUDA graph of fused nodes; the embedding runs in eager
    PyTorch around it, as in the reference (python/model_zoo/bert/bert_modeling.py:184-193)."""
    name = "bert_large_train_step_b32_s512_bf16"
    metric = "BERT-large train-step samples/s per B200; fused GEMM TFLOP/s as % of tensor peak"
    unit = "samples/s"
    dtype = "bf16"
    config_notes = ("timed step = embedding (eager), encoder + masked-LM head forward and backward on fused nodes, "
                    "embedding backward; dropout is omitted (the reference's configuration sets p = 1e-19, "
                    "mask == 1; fused dropout is tested on its own), the pooler and the next-sentence head "
                    "(two M = 32 GEMMs) are outside the step, no optimizer update (the reference times zero_grad + "
                    "forward + backward only, python/gtl/helper/test_helper.py:39-42)")
    cpu_sample = ("2 encoder layers + masked-LM head of the same model, batch 4 x sequence 512, fp32 eager "
                  "PyTorch forward + backward; samples/s scaled by (2-layer+head FLOPs)/(24-layer+head FLOPs)")

    def __init__(self, layers=24, B=32, S=512):
        from evt_ae_b200.workloads import bert as wb
        self.wb = wb
        self.cfg = wb.BertConfig(layers=layers)
        self.B, self.S = B, S

    def setup(self, device):
        wb, cfg, B, S = self.wb, self.cfg, self.B, self.S
        dt = torch.bfloat16
        self.device = device
        self.step = wb.BertStep(cfg, B, S, dtype=dt)
        params = wb.init_params(cfg, seed=1235, dtype=dt)
        self.emb = {k: v.to(device).requires_grad_(True) for k, v in params.items() if k.startswith("emb.")}
        self.p = self.step.prepare_params({k: v.to(device) for k, v in params.items()})
        ids, labels, mask = wb.synthetic_batch(cfg, B, S, seed=1235)
        self.host = [ids.pin_memory(), labels.pin_memory(), mask.to(dt).pin_memory()]
        self.dev_in = [t.to(device) for t in self.host]
        self.flops = self.step.gemm_flops
        self.embed = lambda ids: wb.embeddings(self.emb, ids, cfg.eps)
        # static buffers of the captured graph
        self.s_x0 = torch.zeros(S, B, cfg.hidden, dtype=dt, device=device)
        self.s_mask = self.dev_in[2].clone()
        self.s_labels = self.dev_in[1].clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                out = self.step.step(self.p, self.s_x0, self.s_mask, self.s_labels)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.step.check_status()
        del out
        import torch.distributed as dist
        multi = dist.is_initialized() and dist.get_world_size() > 1
        self.graph = None
        self.segments = None        # data parallel: [(graph, gradients finished by it, their reducer)]
        from evt_ae_b200 import runtime
        launches_before = runtime.KERNELS_ENQUEUED
        if os.environ.get("MODE", "RUN") != "DEBUG":   # DEBUG synchronises per node: no capture
            if not multi:
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                    self.s_loss, self.s_grads, self.s_dx0 = self.step.step(self.p, self.s_x0, self.s_mask, self.s_labels)
            else:
                # the backward pass is cut into four graphs (one memory pool, replayed in order) so that
                # the all-reduce of the gradients a graph finished runs on a second stream while the
                # next graph computes
                Ln = cfg.layers
                cuts = sorted({(3 * Ln) // 4, Ln // 2, Ln // 4} - {0})
                pool = torch.cuda.graph_pool_handle()
                gen = self.step.step_parts(self.p, self.s_x0, self.s_mask, self.s_labels, cuts=cuts)
                self.segments, self.s_grads = [], {}
                while True:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=pool, capture_error_mode="thread_local"):
                        part = next(gen)
                    if isinstance(part, tuple):
                        self.s_loss, part, self.s_dx0 = part
                        self.segments.append([g, part, None])
                        self.s_grads.update(part)
                        break
                    self.segments.append([g, part, None])
                    self.s_grads.update(part)
                gen.close()
        # this library's kernels in one step, counted while the step was captured (torch's own small
        # kernels around them -- embedding, loss bookkeeping, the arena memset -- are not included)
        self.launches_per_step = (runtime.KERNELS_ENQUEUED - launches_before) or self._count_launches()
        self.host_loss = torch.zeros((), dtype=torch.float32).pin_memory()
        # data parallel: every rank is a replica; parameter gradients are all-reduced (NCCL)
        self.reducer = None
        if multi:
            from evt_ae_b200.dp import GradAllReducer
            self.comm = torch.cuda.Stream()
            if self.segments is not None:
                for seg in self.segments:
                    seg[2] = GradAllReducer(seg[1])
            self._run(*self.dev_in)              # materialise the embedding gradients once
            torch.cuda.synchronize()
            self.reducer = GradAllReducer(self._all_grads() if self.segments is None else self._emb_grads())

    def _emb_grads(self):
        return {"autograd." + k: v.grad for k, v in self.emb.items() if v.grad is not None}

    def _all_grads(self):
        g = dict(self.s_grads)
        g.update(self._emb_grads())
        return g

    @property
    def bytes_reduced_per_step(self):
        total = getattr(self.reducer, "bytes_per_step", 0) if self.reducer is not None else 0
        for seg in (self.segments or []):
            total += seg[2].bytes_per_step if seg[2] is not None else 0
        return total

    def _count_launches(self):
        cfg = self.cfg
        per_layer_fwd, per_layer_bwd = 10, 21          # fused nodes + column sums per layer
        if self.step.n.fuse_attention:                 # scores + softmax and dprobs + softmax backward are one node each
            per_layer_fwd, per_layer_bwd = 9, 20
        return cfg.layers * (per_layer_fwd + per_layer_bwd) + 12

    def _run(self, ids, labels, mask):
        x0 = self.embed(ids)
        with torch.no_grad():
            self.s_x0.copy_(x0)
            self.s_mask.copy_(mask)
            self.s_labels.copy_(labels)
        main = torch.cuda.current_stream()
        if self.segments is not None:
            for g, part, red in self.segments:
                g.replay()
                if red is not None:
                    self.comm.wait_stream(main)
                    with torch.cuda.stream(self.comm):
                        red.allreduce(part)
        elif self.graph is not None:
            self.graph.replay()
        else:
            self.s_loss, self.s_grads, self.s_dx0 = self.step.step(self.p, self.s_x0, self.s_mask, self.s_labels)
        for v in self.emb.values():
            v.grad = None
        x0.backward(self.s_dx0.to(x0.dtype))
        if getattr(self, "reducer", None) is not None:
            if self.segments is not None:
                self.comm.wait_stream(main)
                with torch.cuda.stream(self.comm):
                    self.reducer.allreduce(self._emb_grads())
            else:
                self.reducer.allreduce(self._all_grads())
        if self.segments is not None and getattr(self, "comm", None) is not None:
            main.wait_stream(self.comm)
        return self.s_loss

    def step_device(self):
        return self._run(*self.dev_in)

    def step_e2e(self):
        ins = [t.to(self.device, non_blocking=True) for t in self.host]
        loss = self._run(*ins)
        self.host_loss.copy_(loss, non_blocking=True)
        return loss

    def h2d_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.host)

    def d2h_bytes(self):
        return 4

    def value_from_ms(self, ms, n_gpus):
        return n_gpus * self.B / (ms * 1e-3)

    def check(self):
        self.step.check_status()
        if not torch.isfinite(self.s_loss).item():
            raise SystemExit("non-finite loss")

    def dominant_kernel(self):
        """(name, flops per launch, list of launch times in ms) of the FFN1 GEMM, the
        node with the largest share of the step's FLOPs."""
        cfg, B, S = self.cfg, self.B, self.S
        T = B * S
        dt = torch.bfloat16
        op = self.step.n.ops["lin_hf_gelu"]
        x = torch.randn(T, cfg.hidden, device=self.device, dtype=dt)
        args = [self.p["l0.ff1.b"], x, self.p["l0.ff1.w"]]
        names = op.input_names + [a.name for a in op.args]
        byname = {"b": self.p["l0.ff1.b"], "x": x, "w": self.p["l0.ff1.w"]}
        args = [byname[n] for n in names]
        return "lin_hf_gelu (FFN1 GEMM 16384x4096x1024 + bias + GELU, 2 stores)", op.flops, op.time_kernel(args, iters=20, warmup=3)

    def eager_gpu_ms(self, steps=5, warmup=2):
        """The same model and batch as plain eager PyTorch bf16 autograd on this GPU (the oracle's
        module moved to the device): the comparison the reference itself publishes (fused step
        against PyTorch eager, benchmark/bert/bert.py:56-112).  A baseline, timed after the
        main measurement; none of this library's kernels run in it."""
        from oracle import bert_ref
        cfg, dev, dt = self.cfg, self.device, torch.bfloat16
        p = {k: v.to(dt).to(dev).requires_grad_(True) for k, v in bert_ref.init_params(cfg, seed=1235).items()}
        ids, labels, mask = self.dev_in[0], self.dev_in[1], self.dev_in[2]

        def step():
            for v in p.values():
                v.grad = None
            x = bert_ref.embeddings(p, ids, cfg.eps)
            loss = bert_ref.encoder_and_head_loss(p, cfg, x, mask, labels)
            loss.backward()
            return loss
        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    # CPU side (oracle): a bounded slice of the same model
    def cpu_step(self):
        from oracle import bert_ref
        wb = self.wb
        if not hasattr(self, "_cpu"):
            cfg = wb.BertConfig(layers=2)
            p = bert_ref.init_params(cfg, seed=1235)
            ids, labels, mask = bert_ref.synthetic_batch(cfg, 4, self.S, seed=1235)
            self._cpu = (cfg, p, ids, labels, mask)
        cfg, p, ids, labels, mask = self._cpu
        return bert_ref.loss_and_grads(p, cfg, ids, labels, mask)

    def cpu_value(self, seconds):
        """samples/s of the full model implied by the timed slice (FLOP-proportional)."""
        H, FF, S, V = self.cfg.hidden, self.cfg.ffn, self.S, self.cfg.vocab
        layer = 2 * S * H * (4 * H + 2 * FF) + 4 * S * S * H
        head = 2 * S * H * (H + V)
        frac = (2 * layer + head) / (self.cfg.layers * layer + head)
        return 4 / seconds * frac


# dram__bytes_read.sum + dram__bytes_write.sum of one FFN1 launch, from the ncu capture summarised in
# profiles/bert_ffn1_gemm_ncu_metrics.md (same kernel image and shape as the step's node)
FFN1_DRAM_TRAFFIC_BYTES = 307.6e6
FFN1_ALGORITHMIC_BYTES = 2.0 * (16384 * 1024 + 4096 * 1024 + 2 * 16384 * 4096) + 2 * 4096

WORKLOADS = {"config0": Config0Workload, "ffn1": Ffn1Workload, "conv": Conv3x3Workload, "spmm": SpmmWorkload,
             "bert": BertLargeWorkload, "gcn": GcnWorkload, "vit": VitWorkload, "resnet": ResNetWorkload}


def time_cpu(workload, reps=3):
    torch.set_num_threads(os.cpu_count() or 1)
    workload.cpu_step()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        workload.cpu_step()
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="evt_b200", choices=["evt_b200", "reference"])
    ap.add_argument("--workload", default="bert", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-eager-baseline", action="store_true",
                    help="skip the eager PyTorch bf16 step on the same GPU (an extra, labelled field)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "evt_b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS[args.workload]()

    if args.impl == "reference":
        if rank != 0:
            return
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        for _ in range(min(args.warmup, 1)):
            wl.cpu_step()
        ts = []
        for _ in range(args.steps):
            t0 = time.perf_counter()
            wl.cpu_step()
            ts.append(time.perf_counter() - t0)
        ms = 1e3 * sum(ts) / len(ts)
        val = wl.cpu_value(ms * 1e-3) if hasattr(wl, "cpu_value") else wl.value_from_ms(ms, 1)
        line = dict(metric=wl.metric, value=val, unit=wl.unit, n_gpus=args.gpus, steps=args.steps,
                    warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak",
                    vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                    config=dict(workload=wl.name, note="unfused fx graph, fp32 eager PyTorch on host cores"),
                    cpu_baseline=dict(value=val, unit=wl.unit, cores=cores, kind="port", sample=wl.cpu_sample),
                    e2e=dict(value=val, unit=wl.unit, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                    gpu_launches=0)
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused operators have no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        # a collective that one rank never joins ends the run after two minutes, not ten
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=120))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    wl.setup(device)
    peaks = load_peaks()

    def timed(step_fn, steps, warmup):
        for _ in range(warmup):
            step_fn()
        barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for i in range(steps):
            step_fn()
            ev[i + 1].record()
        barrier()
        per = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
        total = ev[0].elapsed_time(ev[-1])
        if dist is not None:
            t = torch.tensor([total], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total = float(t.item())
        return total / steps, per

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, per = timed(wl.step_device, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    wl.check()
    ms_e2e, _ = timed(wl.step_e2e, max(3, min(args.steps, 10)), 3)
    wl.check()

    if rank == 0:
        value = wl.value_from_ms(ms, world)
        e2e_val = wl.value_from_ms(ms_e2e, world)
        # dominant kernel = the fused GEMM; the step holds one launch of it plus torch fills
        # of the reduction targets, so the per-step event time bounds the kernel time from above
        total_s = ms * args.steps / 1e3
        if hasattr(wl, "dominant_kernel"):
            kname, kflops, ktimes = wl.dominant_kernel()
            kernel_ms = statistics.mean(ktimes)
            peak = peaks["tflops_burst"]
            achieved = kflops / (kernel_ms * 1e-3) / 1e12
            step_tflops = wl.flops / (ms * 1e-3) / 1e12
            is_ffn1 = isinstance(wl, BertLargeWorkload)
            roofline = dict(bound="tensor", achieved=achieved, peak=peak, unit="TFLOP/s", frac=achieved / peak,
                            traffic=FFN1_DRAM_TRAFFIC_BYTES if is_ffn1 else None,
                            traffic_unit=("bytes per launch (dram read + write), from the ncu capture summarised in "
                                          "profiles/bert_ffn1_gemm_ncu_metrics.md, not measured in this run") if is_ffn1 else None,
                            algorithmic_bytes=FFN1_ALGORITHMIC_BYTES if is_ffn1 else None, kernel=kname, kernel_ms=kernel_ms,
                            peak_source=f"{peaks['source']} (burst: kernel timed alone)",
                            step_gemm_tflops=step_tflops, step_gemm_flops=wl.flops,
                            step_gemm_frac_of_sustained_peak=step_tflops / peaks["tflops_sustained"])
        elif hasattr(wl, "dominant_kernel_hbm"):
            kname, kbytes, ktimes = wl.dominant_kernel_hbm()
            kernel_ms = statistics.mean(ktimes)
            achieved = kbytes / (kernel_ms * 1e-3) / 1e9
            roofline = dict(bound="hbm", achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s",
                            frac=achieved / peaks["hbm_gbs"], traffic=None, peak_source=peaks["source"],
                            algorithmic_bytes=kbytes, kernel=kname, kernel_ms=kernel_ms)
        else:
            kernel_ms = statistics.median(per)
            if getattr(wl, "bound", "tensor") == "hbm":
                achieved = wl.bytes / (kernel_ms * 1e-3) / 1e9
                roofline = dict(bound="hbm", achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s",
                                frac=achieved / peaks["hbm_gbs"], traffic=None, peak_source=peaks["source"],
                                algorithmic_bytes=wl.bytes)
            else:
                peak = peaks["tflops_burst"] if total_s < 1.0 else peaks["tflops_sustained"]
                achieved = wl.flops / (kernel_ms * 1e-3) / 1e12
                roofline = dict(bound="tensor", achieved=achieved, peak=peak, unit="TFLOP/s", frac=achieved / peak,
                                traffic=None, peak_source=f"{peaks['source']} ({'burst' if total_s < 1.0 else 'sustained'})",
                                hbm_gbs_at_this_rate=wl.bytes / (kernel_ms * 1e-3) / 1e9, hbm_peak_gbs=peaks["hbm_gbs"])
        cpu = None
        if not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            cpu_s = time_cpu(wl)
            cpu = dict(value=(wl.cpu_value(cpu_s) if hasattr(wl, "cpu_value") else wl.value_from_ms(cpu_s * 1e3, 1)),
                       unit=wl.unit, cores=cores, kind="port",
                       sample=wl.cpu_sample, seconds=cpu_s)
        eager = None
        if world == 1 and hasattr(wl, "eager_gpu_ms") and not args.no_eager_baseline:
            try:
                eager_ms = wl.eager_gpu_ms()
                eager = dict(ms_per_step=eager_ms, value=wl.value_from_ms(eager_ms, 1), unit=wl.unit,
                             speedup_of_fused_step=eager_ms / ms,
                             what=f"the same model and batch, eager PyTorch {wl.dtype} autograd on this GPU (baseline)")
            except Exception as e:   # the baseline must not take the measurement down
                eager = dict(error=repr(e)[:200])
        notes = getattr(wl, "config_notes", None)
        if world == 1:
            parallelism = "single GPU"
        elif hasattr(wl, "bytes_exchanged_per_step"):
            parallelism = (f"rows{world}: destination rows of the graph partitioned over the GPUs (balanced by nonzeros and rows), "
                           f"operand gathered into local memory before every aggregation "
                           f"({wl.bytes_exchanged_per_step / 1e6:.0f} MB of gathered operands per rank and step, NCCL), "
                           f"weight gradients all-reduced")
        else:
            how = ("overlapped with the backward pass in four segments" if getattr(wl, "segments", None)
                   else "after the step's single graph")
            parallelism = (f"dp{world}: one replica per GPU, per-GPU batch fixed, NCCL gradient all-reduce "
                           f"({getattr(wl, 'bytes_reduced_per_step', 0) / 1e6:.0f} MB per step, {how})")
        line = dict(metric=wl.metric, value=value, unit=wl.unit, n_gpus=world, steps=args.steps,
                    warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling=getattr(wl, "scaling", "weak"),
                    vs_baseline=None, dtype=wl.dtype, data="synthetic",
                    config=dict(workload=wl.name, l2="working set per step far exceeds the 126 MB L2",
                                **({"notes": notes} if notes else {}),
                                parallelism=parallelism),
                    roofline=roofline, cpu_baseline=cpu,
                    e2e=dict(value=e2e_val, unit=wl.unit, ms_per_step=ms_e2e,
                             h2d_bytes_per_step=wl.h2d_bytes(), d2h_bytes_per_step=wl.d2h_bytes()),
                    gpu_launches=wl.launches_per_step * args.steps, clocks=clocks,
                    **({"eager_torch_gpu": eager} if eager is not None else {}))
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
