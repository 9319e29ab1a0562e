"""CPU oracle for the fused-operator path.  TEST INFRASTRUCTURE ONLY.

Only `tests/`, `__graft_entry__.smoke()` and the `cpu_baseline` / `--impl reference` legs of
`bench.py` may import this package, and only as the checker or as the timed CPU baseline --
never as part of the product path (`evt_ae_b200/` does not import it).

The oracle is the one the reference itself uses: the *unfused* fx graph / nn.Module run in
eager PyTorch (python/gtl/helper/test_helper.py:78-104, and the in-situ check in
python/gtl/compiler/passes/evt_fuser.py:106-141), here upcast to fp32 and run on CPU.
`refgraph.py` runs a module that way and holds the comparison rule; `bert_ref.py` and
`gcn_ref.py` are the whole-model oracles (plain autograd modules of the two training steps).

Pinning: the reference ships no golden vectors (its tests compare fused vs eager on
unseeded random inputs).  `tests/golden/golden.npz` holds outputs generated in the build
container by executing, on seeded inputs, the reference's own code: 26 test methods of
unittest/evt_fuser/{mm,bmm,softmax,softmax_backward,layernorm,layernorm_backward,conv}.py,
the module of unittest/evt_fuser/dropout.py with the mask it drew, and the wrapped leaf
functions of python/gtl/compiler/passes/pass_decomposition.py:61-189 (`spmm`, channels-last
convolution forward / data gradient, the four split batch-norm leaves).  The CPU test suite
checks the restated modules and this package's leaves against them; the GPU suite checks the
CUDA path against the same numbers.  Not pinned by reference-generated numbers: the two
whole-model oracles (the reference's BERT needs NVIDIA's DeepLearningExamples module, its GCN
needs DGL / OGB; both are absent) -- they are restated from the architecture files and checked
only against autograd of themselves.
"""
from .refgraph import run_unfused_fp32, compare, TOL  # noqa: F401
