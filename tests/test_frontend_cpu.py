"""The reference's front end driving this back end (needs a checkout of the reference, as the
build container has; skipped elsewhere).

One BERT encoder layer (the structure of python/model_zoo/bert: [S, B, H] token order, post-LN,
tanh GELU) is traced by AOT autograd into its joint forward + backward graph; the reference's
passes -- frontend, loss elimination, decomposition, CSE, constant propagation and the MILP
partitioner (pass_fusion.py:1356-1374) -- run unchanged and hand their partitions to
`evt_ae_b200.fuser.EVTFuser`.  The fused nodes that come out must be the node set that
`workloads/bert.py` writes down by hand for one layer: same kinds, same GEMM shapes, same number
of results and of epilogue reductions."""
import collections
import contextlib
import io
import os

import pytest
import torch
import torch.nn.functional as F

# a checkout of the reference: named by EVT_REFERENCE_ROOT, else a directory `reference` beside this repository
REF = os.environ.get("EVT_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "python", "gtl", "compiler", "passes")),
                                reason="no checkout of the reference here")

S, B, H, NH, FF = 64, 2, 128, 2, 256


def _layer(x, wq, bq, wk, bk, wv, bv, wo, bo, g1, b1, w1, c1, w2, c2, g2, b2):
    d, T = H // NH, S * B
    x2 = x.view(T, H)
    q = F.linear(x2, wq, bq).view(S, B * NH, d).transpose(0, 1)
    k = F.linear(x2, wk, bk).view(S, B * NH, d).permute(1, 2, 0)
    v = F.linear(x2, wv, bv).view(S, B * NH, d).transpose(0, 1)
    p = torch.softmax(torch.bmm(q, k) / (d ** 0.5), -1)
    ctx = torch.bmm(p, v).transpose(0, 1).contiguous().view(T, H)
    a = F.layer_norm(F.linear(ctx, wo, bo) + x2, (H,), g1, b1, 1e-12)
    f = F.gelu(F.linear(a, w1, c1), approximate="tanh")
    h = F.layer_norm(F.linear(f, w2, c2) + a, (H,), g2, b2, 1e-12)
    return h.float().pow(2).mean()


def _signature(op):
    ir = op.ir
    kinds = collections.Counter(n.kind for n in ir.nodes)
    k = getattr(op, "K", 0)
    return (type(op).__name__, ir.L, ir.M, ir.N, k, len(op.outputs))


def _partitioned_layer():
    from torch._functorch.aot_autograd import aot_function
    from torch._functorch.partitioners import default_partition
    from evt_ae_b200 import frontend
    frontend.install(REF)
    got = {}

    def partition_fn(joint_module, joint_inputs, **kw):
        import copy
        with contextlib.redirect_stdout(io.StringIO()):        # the MILP solver and the passes print a lot
            got["module"] = frontend.joint_optimization(copy.deepcopy(joint_module))
        return default_partition(joint_module, joint_inputs, **kw)
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(torch.float16).requires_grad_(True)
    args = [mk(S, B, H), mk(H, H), mk(H), mk(H, H), mk(H), mk(H, H), mk(H), mk(H, H), mk(H), mk(H), mk(H),
            mk(FF, H), mk(FF), mk(H, FF), mk(H), mk(H), mk(H)]
    ident = lambda gm, inputs: gm
    aot_function(_layer, fw_compiler=ident, bw_compiler=ident, partition_fn=partition_fn)(*args).backward()
    return frontend.fused_nodes(got["module"])


def test_reference_partitions_are_the_hand_written_node_set(monkeypatch):
    ops = _partitioned_layer()
    kinds = collections.Counter(type(o).__name__ for o in ops)
    # forward: q, k, v, out-proj, FFN1, FFN2 GEMMs, scores and context BMMs, softmax, two LayerNorms;
    # backward: a data- and a weight-gradient GEMM per linear map, four BMMs, softmax and LayerNorm backward
    assert kinds == {"FusedGEMM": 18, "FusedBMM": 6, "FusedSoftmax": 1, "FusedSoftmaxBackward": 1,
                     "FusedLayerNorm": 2, "FusedLayerNormBackward": 2}, kinds
    # the same layer as written by hand (scores / softmax kept apart, as the reference partitions them)
    monkeypatch.setenv("EVT_B200_FUSE_ATTENTION", "0")
    from evt_ae_b200.workloads import bert as wb
    n = wb._Nodes(wb.BertConfig(layers=1, hidden=H, heads=NH, ffn=FF, vocab=64, max_pos=S), B, S, torch.float16)
    per_layer = {"lin_hh": 3, "scores": 1, "softmax": 1, "context": 1, "lin_hh_res": 1, "layernorm": 2, "lin_hf_gelu": 1,
                 "lin_fh_res": 1, "layernorm_bwd": 2, "wgrad_hf": 1, "dgrad_gelu": 1, "wgrad_fh": 1, "dgrad_f_res_ln": 1,
                 "wgrad_hh": 4, "dgrad_hh": 1, "bmm_tn": 2, "dprobs": 1, "softmax_bwd": 1, "bmm_nn": 1, "dgrad_hh_res": 2}
    mine = collections.Counter()
    for name, cnt in per_layer.items():
        op = n.ops[name]
        mine[(type(op).__name__, op.ir.L, op.ir.M, op.ir.N, getattr(op, "K", 0))] += cnt
    # the last data gradient of the layer: with a residual and LayerNorm gradients of the layer below in
    # the hand-written step (dgrad_h_res_ln); the single traced layer has nothing below it
    mine[("FusedGEMM", 1, S * B, H, H)] += 1
    theirs = collections.Counter((type(o).__name__, o.ir.L, o.ir.M, o.ir.N, getattr(o, "K", 0)) for o in ops)
    assert theirs == mine, (sorted((theirs - mine).items()), sorted((mine - theirs).items()))
