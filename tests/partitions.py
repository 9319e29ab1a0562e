"""The fused-node cases live in the package (`evt_ae_b200.workloads.cases`): the benchmark and
the ahead-of-time build use them too.  Tests keep importing them under this name."""
from evt_ae_b200.workloads.cases import *  # noqa: F401,F403
