"""Seeded inputs for the oracle and the tests: the workload definitions live in the package
(``swamla_b200/workloads.py``) so that the benchmark and the tests draw identical tensors."""
from swamla_b200.workloads import *  # noqa: F401,F403
from swamla_b200.workloads import WORKLOADS, Workload, make_inputs, param_shapes, round_to_bf16  # noqa: F401
