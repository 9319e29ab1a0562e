"""CSR SpMM (merge-path, generated epilogue), SDDMM and the CSR builder on the GPU through
the C-ABI.  fp32 results: |out - ref| <= 1e-5 |ref| + 1e-5 x RMS of the row -- hub rows add
thousands of terms of both signs in a different order than the CPU; fp16 features: 1e-2 / 1e-3;
CSR arrays bit-exact."""
import pytest
import torch

import partitions as P
from evt_ae_b200 import ops
from evt_ae_b200.fuser import fuse_module
from oracle import run_unfused_fp32

pytestmark = pytest.mark.gpu


def _check(out, ref, half):
    out, ref = out.detach().cpu().double(), ref.detach().cpu().double()
    rowmag = ref.pow(2).mean(dim=-1, keepdim=True).sqrt()
    tol = (1e-2 * ref.abs() + 1e-3 * rowmag) if half else (1e-5 * ref.abs() + 1e-5 * rowmag)
    bad = (out - ref).abs() > tol
    assert not bad.any(), ((out - ref).abs().max().item(), int(bad.sum()))


@pytest.mark.parametrize("case", P.small_spmm_cases(), ids=lambda c: c.name)
def test_spmm_small(case, cuda_device):
    inputs = [t.to(cuda_device) for t in case.inputs]
    gm, fused = fuse_module(case.module, inputs)
    ref = run_unfused_fp32(case.module, case.inputs)[0]
    for _ in range(2):                     # second call: the scratch must have been left clean
        out = gm(*inputs)
        torch.cuda.synchronize()
        fused.check_status()
        _check(out, ref, case.inputs[3].dtype != torch.float32)


def test_spmm_gcn_size(cuda_device):
    """The GCN configuration: 169,343 nodes, ~1.17 M sampled edges (power-law, hubs with
    tens of thousands of neighbours), 128 features, normalisation fused, self term added."""
    case = P.spmm_case(169343, 585000, 128, "sym")
    inputs = [t.to(cuda_device) for t in case.inputs]
    gm, fused = fuse_module(case.module, inputs)
    out = gm(*inputs)
    torch.cuda.synchronize()
    fused.check_status()
    _check(out, run_unfused_fp32(case.module, case.inputs)[0], False)
    # linearity, independent of the oracle: A(2x) = 2 A(x)
    out2 = gm(inputs[0], inputs[1], inputs[2], inputs[3] * 2)
    assert torch.allclose(out2, out * 2, rtol=1e-5, atol=1e-5)


def test_sddmm(cuda_device):
    r, c = P.chung_lu_graph(4000, 30000)
    crow, col = P.csr_reference(r, c, 4000)
    u = P.seeded((4000, 128), 95, 1.0, torch.float32)
    v = P.seeded((4000, 128), 96, 1.0, torch.float32)
    out = ops.sddmm(crow.to(cuda_device), col.to(cuda_device), u.to(cuda_device), v.to(cuda_device)).cpu()
    rows = torch.repeat_interleave(torch.arange(4000), (crow[1:] - crow[:-1]).long())
    ref = (u.double()[rows] * v.double()[col.long()]).sum(-1)
    assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-4)


def test_sddmm_gcn_size(cuda_device):
    """Edge scores on the GCN configuration's graph (169,343 nodes, 1.17 M stored entries, hub rows
    of tens of thousands of entries), 128 features: sampled entries against a float64 dot product,
    plus linearity in U as a check that does not depend on the oracle."""
    n = 169343
    r, c = P.chung_lu_graph(n, 585000)
    crow, col = P.csr_reference(r, c, n)
    u = P.seeded((n, 128), 95, 1.0, torch.float32)
    v = P.seeded((n, 128), 96, 1.0, torch.float32)
    dev = lambda t: t.to(cuda_device)
    out = ops.sddmm(dev(crow), dev(col), dev(u), dev(v))
    out2 = ops.sddmm(dev(crow), dev(col), dev(u) * 2, dev(v))
    assert torch.allclose(out2, out * 2, rtol=1e-6, atol=1e-6)
    out = out.cpu()
    rows = torch.repeat_interleave(torch.arange(n), (crow[1:] - crow[:-1]).long())
    pick = torch.cat([torch.arange(0, 30000), torch.arange(0, col.shape[0], 37)])      # hub rows and a spread
    ref = (u.double()[rows[pick]] * v.double()[col.long()[pick]]).sum(-1)
    assert torch.allclose(out[pick].double(), ref, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("n,edges", [(1000, 5000), (169343, 585000)])
def test_csr_build_bit_exact(n, edges, cuda_device):
    r, c = P.chung_lu_graph(n, edges)
    crow_ref, col_ref = P.csr_reference(r, c, n)
    crow, col = ops.csr_build(r.to(cuda_device), c.to(cuda_device), n)
    assert torch.equal(crow.cpu(), crow_ref)
    assert torch.equal(col.cpu(), col_ref)
