"""Reference: search_algo/workload_partition.py."""
from ultraattn_b200.planner.allocate import (Allocation, brute_force_allocate,  # noqa: F401
                                             comp_balance_allocate_strategy, naive_allocate_strategy,
                                             solve_sparse_from_bsa)


def Quad_LP_GUROBI_from_block_config(block_config, fob, hierarchy=1, ParD=None, **kw):
    """The reference's name for ILP #1 (workload_partition.py:272-470); accepts a ``BSA_Config`` or
    the older ``Block_Attention_Config``. The solver is HiGHS unless another one is selected."""
    if hasattr(block_config, "to_bsa_config"):
        block_config = block_config.to_bsa_config()
    return solve_sparse_from_bsa(block_config, fob=fob, hierarchy=hierarchy, ParD=ParD, **kw)
