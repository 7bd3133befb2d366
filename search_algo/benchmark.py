"""Reference: search_algo/benchmark.py."""
from ultraattn_b200.drivers.benchmark import benchmark_ops, benchmark_orchestrate_bsa  # noqa: F401
