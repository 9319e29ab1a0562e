"""The fused kernels next to other kernels of the same process.

In a data-parallel step the gradient exchange (pack / unpack copies and the collective's own
kernels) runs on a second stream while the next segment of the backward pass computes, so CTAs
of other kernels share SMs with the tcgen05 kernels and delay their memory traffic.  The
kernels' results must not depend on that: the segmented BERT step, replayed from its CUDA graphs
with a busy second stream working on the finished gradients, has to reproduce the quiet run."""
import pytest
import torch

from evt_ae_b200.dp import GradAllReducer
from evt_ae_b200.workloads import bert as wb

pytestmark = pytest.mark.gpu


def _same(a, b):      # atomically accumulated reductions differ in summation order between runs
    a, b = a.float(), b.float()
    return (a - b).norm().item() <= 2e-3 * b.norm().item() + 1e-6


def test_segment_graphs_next_to_a_busy_second_stream(cuda_device):
    cfg = wb.BertConfig(layers=4, hidden=256, heads=4, ffn=1024, vocab=1000, max_pos=128)
    B, S, dt, dev = 8, 128, torch.bfloat16, cuda_device
    step = wb.BertStep(cfg, B, S, dtype=dt)
    p = step.prepare_params(wb.init_params(cfg, seed=5, dtype=dt, device=dev))
    ids, labels, mask = wb.synthetic_batch(cfg, B, S, seed=5)
    x0 = (torch.randn(S, B, cfg.hidden, generator=torch.Generator().manual_seed(6)) * 0.5).to(dt).to(dev)
    args = (p, x0, mask.to(dt).to(dev), labels.to(dev))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        loss, grads, dx0 = step.step(*args)
        want = {k: v.clone() for k, v in grads.items()}
        want_dx0, want_loss = dx0.clone(), loss.clone()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    step.check_status()

    pool = torch.cuda.graph_pool_handle()
    gen = step.step_parts(*args, cuts=(3, 2, 1))
    segments, captured = [], {}
    while True:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=pool, capture_error_mode="thread_local"):
            part = next(gen)
        if isinstance(part, tuple):
            g_loss, part, g_dx0 = part
            segments.append((g, part))
            captured.update(part)
            break
        segments.append((g, part))
        captured.update(part)
    gen.close()
    assert len(segments) == 4

    # the second stream: pack the finished gradients, a stand-in for the collective (a long train
    # of memory-bound kernels whose CTAs fill every free slot of every SM), unpack
    comm = torch.cuda.Stream()
    reducers = [GradAllReducer(part) for _, part in segments]
    for r in reducers:
        r.world = 1          # single process: `busy_exchange` below stands where allreduce() would
    filler = torch.zeros(8 << 20, dtype=torch.float32, device=dev)
    other = torch.zeros_like(filler)

    def busy_exchange(red, part):
        for flat, entries in red.buckets:
            views = [flat[o:o + k].view(part[n].shape) for n, o, k in entries]
            srcs = [part[n] for n, _, _ in entries]
            torch._foreach_copy_(views, srcs)
            for _ in range(6):
                filler.add_(other)          # 96 MB of traffic per pass, adds zeros
            flat.add_(0.0)
            torch._foreach_copy_(srcs, views)

    main = torch.cuda.current_stream()
    for it in range(25):
        for (g, part), red in zip(segments, reducers):
            g.replay()
            comm.wait_stream(main)
            with torch.cuda.stream(comm):
                busy_exchange(red, part)
        main.wait_stream(comm)
        if it % 8 == 7:
            torch.cuda.synchronize()
            step.check_status()
    torch.cuda.synchronize()
    step.check_status()
    for k in want:
        assert _same(captured[k], want[k]), k
    assert _same(g_dx0, want_dx0) and _same(g_loss, want_loss)
