"""Reference: search_algo/benchmark.py."""
from ultraattn_b200.drivers.benchmark import benchmark_ops, benchmark_orchestrate_bsa  # noqa: F401
from ultraattn_b200.drivers.task2 import prepare_inter_comp_plans  # noqa: F401
from ultraattn_b200.runtime.orchestrated import create_buf_dict  # noqa: F401
