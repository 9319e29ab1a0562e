"""The allocation-free column sum (`evtb_colsum_static`) against the ordinary entry point.

Some programs that embed this library have no way to give it scratch memory -- for instance a
serving process that reserved all device memory for its own pool when it started, or a plugin
slot where a cudaMalloc (a device-wide synchronisation) is forbidden.  For them the partial
sums live in a fixed array inside the library image.  This test calls that entry point
through the C-ABI with caller-owned input and output buffers only, twice in a row with
different shapes (the second call inherits whatever the first left in the shared array), and
checks both results against `evtb_colsum`, which uses a caller-provided workspace.  Both run
the same kernel in the same summation order, so the results must agree exactly; the
assertion allows the usual tolerance of the other GPU tests (1e-2 relative + 1e-3).  Sizes
beyond the built-in limit must be refused without launching anything.

Collected last on purpose (file name): a failure here cannot hide the other tests' results.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

F16, BF16, F32 = 0, 1, 2


def _lib():
    from evt_ae_b200.build import build_library
    from evt_ae_b200 import runtime
    build_library()
    return runtime.load_library()


def _reference_colsum(lib, x, out_dtype_code, out_dtype):
    rows, cols = x.shape
    nbytes = ctypes.c_size_t()
    assert lib.evtb_colsum_workspace_bytes(rows, cols, ctypes.byref(nbytes)) == 0
    ws = torch.zeros((nbytes.value + 3) // 4, dtype=torch.int32, device=x.device)
    y = torch.empty(cols, dtype=out_dtype, device=x.device)
    code = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}[x.dtype]
    st = lib.evtb_colsum(x.data_ptr(), code, rows, cols, y.data_ptr(), out_dtype_code, ws.data_ptr(), ws.numel() * 4,
                         torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.evtb_last_error()
    return y


def test_static_scratch_colsum_matches_workspace_colsum(cuda_device):
    lib = _lib()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    # calls in a row, different geometry: each sees the previous one's leftovers.  The last two are
    # shapes where the built-in array, not the shape, sets the number of row chunks (16384 x 8192:
    # the widest accepted matrix, 64 chunks instead of 296; 20000 x 1024: 512 instead of 625) --
    # there the summation order differs from evtb_colsum's, so only the tolerance holds, not equality
    for rows, cols, dt, code in [(4096, 1024, torch.bfloat16, BF16), (777, 4104, torch.float16, F16),
                                 (4096, 1024, torch.bfloat16, BF16), (16384, 8192, torch.bfloat16, BF16),
                                 (20000, 1024, torch.float16, F16), (333, 1001, torch.float16, F16)]:
        x = torch.randn(rows, cols, device=cuda_device, dtype=torch.float32).to(dt)
        want = _reference_colsum(lib, x, F32, torch.float32)
        got = torch.empty(cols, dtype=torch.float32, device=cuda_device)   # caller-owned output
        st = lib.evtb_colsum_static(x.data_ptr(), code, rows, cols, got.data_ptr(), F32, stream)
        assert st == 0, lib.evtb_status_string(st)
        torch.cuda.synchronize()
        assert torch.allclose(got, want, rtol=1e-2, atol=1e-3), (rows, cols, (got - want).abs().max().item())
        # and against plain PyTorch, so that both entry points cannot be wrong together
        ref = x.float().sum(0)
        assert torch.allclose(got, ref, rtol=1e-2, atol=1e-2 * ref.pow(2).mean().sqrt().item())


def test_static_scratch_colsum_accepts_unaligned_rows_when_it_reads_scalars(cuda_device):
    """With a column count that is not a multiple of 8 the kernel reads element by element, so an
    input that starts on an odd element is fine; with a multiple of 8 it is refused."""
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    base = torch.randn(64 * 1001 + 8, device=cuda_device).to(torch.float16)
    x = base[1:1 + 64 * 1001].view(64, 1001)
    assert x.data_ptr() % 16 != 0
    got = torch.empty(1001, dtype=torch.float32, device=cuda_device)
    assert lib.evtb_colsum_static(x.data_ptr(), F16, 64, 1001, got.data_ptr(), F32, stream) == 0, lib.evtb_last_error()
    torch.cuda.synchronize()
    ref = x.float().sum(0)
    assert torch.allclose(got, ref, rtol=1e-2, atol=1e-2 * ref.pow(2).mean().sqrt().item())
    x8 = base[1:1 + 64 * 1000].view(64, 1000)
    st = lib.evtb_colsum_static(x8.data_ptr(), F16, 64, 1000, got.data_ptr(), F32, stream)
    assert st == 1 and b"16-byte" in lib.evtb_last_error()          # EVTB_EINVAL


def test_static_scratch_colsum_refuses_oversize(cuda_device):
    lib = _lib()
    limit = lib.evtb_colsum_static_max_cols()
    x = torch.zeros(8, limit + 8, device=cuda_device, dtype=torch.float16)
    y = torch.full((limit + 8,), 7.0, device=cuda_device, dtype=torch.float32)
    st = lib.evtb_colsum_static(x.data_ptr(), F16, 8, limit + 8, y.data_ptr(), F32,
                                torch.cuda.current_stream().cuda_stream)
    assert st == 6                                   # EVTB_ETOOLARGE
    assert b"limit" in lib.evtb_status_string(st)
    torch.cuda.synchronize()
    assert bool((y == 7.0).all())                    # nothing was launched


@pytest.mark.gpu
def test_colsum_accumulate_matches_fixed_order_sum(cuda_device):
    """The one-pass atomic column sum (fp32 result) against the two-step fixed-order one, plain
    and through a reduction arena, ragged column count included."""
    from evt_ae_b200 import ops
    from evt_ae_b200.fused_ops import ReductionArena
    for rows, cols, dt in [(16384, 1024, torch.bfloat16), (5000, 40, torch.float16), (777, 1000, torch.float32)]:
        x = (torch.randn(rows, cols, generator=torch.Generator().manual_seed(rows)) * 0.5).to(dt).to(cuda_device)
        ref = x.double().sum(0)
        a = ops.colsum(x, torch.float32)
        arena = ReductionArena(cuda_device, 1 << 14)
        arena.reset()
        with arena:
            b = ops.colsum(x, torch.float32)
            c = ops.colsum(x, torch.float32)
        torch.cuda.synchronize()
        assert b.data_ptr() != c.data_ptr() and arena.off >= 2 * cols
        for y in (a, b, c):
            assert y.dtype == torch.float32 and y.shape == (cols,)
            assert (y.double() - ref).abs().max().item() <= 1e-3 * max(1.0, ref.abs().max().item())
