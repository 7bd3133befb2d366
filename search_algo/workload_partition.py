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


def _causal_config(N: int):
    from ultraattn_b200.patterns.blocks import BSA_Config
    from ultraattn_b200.patterns.named import causal
    return BSA_Config(None, None, {"bsa_repr": causal(1), "CP": (N, 1)})


def Quad_LP_GUROBI(N: int, fob: int = 0, **kw):
    """Dense causal attention on ``N`` ranks with ``N`` x ``N`` tiles (the reference's first,
    causal-only formulation, workload_partition.py:161-269)."""
    return solve_sparse_from_bsa(_causal_config(N), fob=fob, ParD=N, **kw)


ILP = Quad_LP_GUROBI            # the PuLP / CBC form of the same problem (workload_partition.py:87-159)


def solve_global_causal(Ns=(2, 4, 8), fob: int = 0, **kw) -> dict:
    """Allocations of dense causal attention for several rank counts (reference:
    workload_partition.py:474-499 prints them)."""
    return {N: Quad_LP_GUROBI(N, fob, **kw) for N in Ns}
