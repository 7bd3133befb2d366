"""Reference: search_algo/workload_partition.py."""
from ultraattn_b200.planner.allocate import (Allocation, brute_force_allocate,  # noqa: F401
                                             naive_allocate_strategy, solve_sparse_from_bsa)
