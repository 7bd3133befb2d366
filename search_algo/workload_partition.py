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


def convert_result_to_np(CP: int, ParD: int, Vars: dict, v_attr: str, cmap=None, diagonal_full: bool = True):
    """Allocation table from a solver's variable dictionary (reference: workload_partition.py:67-85).
    ``Vars['x_i_j_k']`` is the 0/1 variable "tile (i, j) runs on rank k" and ``v_attr`` names the
    attribute that holds its value (``X`` for Gurobi, ``varValue`` for PuLP); tiles without
    variables stay EMPTY (-1) and, with ``diagonal_full``, diagonal tiles go to their row owner."""
    import numpy as np
    table = np.full((ParD, ParD), -1, dtype=np.int32)
    for i in range(ParD):
        for j in range(ParD):
            if i == j and diagonal_full:
                table[i, j] = cmap[i]
            elif f"x_{i}_{j}_0" in Vars:
                vals = [getattr(Vars[f"x_{i}_{j}_{k}"], v_attr) for k in range(CP)]
                table[i, j] = max(range(CP), key=lambda k: vals[k]) if max(vals) > 0 else -1
    return table


def print_lp_result(CP: int, ParD: int, Vars: dict, v_attr: str, cmap=None, diagonal_full: bool = True) -> None:
    """Print the variables and the allocation matrix ('/' where a tile has no variables);
    reference: workload_partition.py:40-65."""
    print("LP result:", flush=True)
    for name, var in Vars.items():
        print(f"{name}: {getattr(var, v_attr)}")
    table = convert_result_to_np(CP, ParD, Vars, v_attr, cmap, diagonal_full)
    print("Allocation Matrix:")
    for i in range(ParD):
        cells = []
        for j in range(ParD):
            known = (i == j and diagonal_full) or f"x_{i}_{j}_0" in Vars
            cells.append(f"{table[i, j]:<2d}" if known else "/ ")
        print(" ".join(cells))


def solve_custom_sparse(CP: int = 4, Par_D: int = 8, pattern_type: str = "local_global",
                        pattern_sparsity: float = 1 / 4, local_blocks=3, global_blocks=0, replicate: int = 1,
                        fob: int = 0, **kw):
    """Allocation of one parametric pattern (reference: workload_partition.py:501-545, whose
    defaults these are); returns the ``Allocation``."""
    from ultraattn_b200.patterns.blocks import BSA_Config
    from ultraattn_b200.utils.bsa_helpers import create_block_sparse_pattern
    pair = lambda x: tuple(x) if isinstance(x, (tuple, list)) else (x, x)
    pattern = create_block_sparse_pattern(CP, Par_D, pattern_type, pattern_sparsity, pair(local_blocks),
                                          pair(global_blocks), replicate)
    cfg = BSA_Config(None, None, {"bsa_repr": pattern, "CP": (CP, 1)})
    return solve_sparse_from_bsa(cfg, fob=fob, ParD=Par_D, **kw)


def main() -> None:
    for N, al in solve_global_causal().items():
        print(f"causal, {N} ranks: comm volume {al.comm_volume} ({al.status})")
        print(al.table)


if __name__ == "__main__":
    main()
