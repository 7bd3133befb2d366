"""One-call planning: pattern + shape + CP degree -> allocation -> kernel graph -> launch plan."""
from __future__ import annotations

from typing import Optional

from ..patterns.blocks import BSA_Config, BSA_Repr
from .allocate import naive_allocate_strategy, solve_sparse_from_bsa
from .cost import Dist_Attn_Config, Machine_Config, get_cc_optimal_schedule_from_table
from .fuse import Graph_Transformation_Engine
from .graph import Dependent_Graph
from .schedule import Execution_Plan


def make_plan(pattern: BSA_Repr, cp: int, seq_len: int, n_heads: int, head_dim: int = 128,
              n_kv_heads: Optional[int] = None, batch: int = 1, fob: int = 0, *,
              allocation: str = "ilp", plan_type: str = "Flexflow", kernel_tile: bool = False,
              m_config: Optional[Machine_Config] = None, ParD: Optional[int] = None,
              objective: str = "comm", time_limit: float = 30.0, cmap=None,
              cp_inter: int = 1) -> Execution_Plan:
    """Plan one intra-node distributed attention call.

    ``allocation``: ``"ilp"`` (ILP #1) or ``"naive"`` (row owner). ``plan_type``: ``"ILP"`` or
    ``"Flexflow"``. ``kernel_tile``: try rectangle fusion and keep it if the makespan improves.
    ``cp_inter`` > 1 plans two levels (``cp`` ranks per node, ``cp_inter`` nodes) and flattens them
    into one plan over ``cp * cp_inter`` ranks (rank = node * cp + local rank).
    """
    if cp_inter > 1:
        from .hierarchy import flatten_two_level
        two = BSA_Config(None, None, {"bsa_repr": pattern, "CP": (cp, cp_inter)})
        alloc = flatten_two_level(two, fob=fob, time_limit=time_limit)
        m_config = m_config or Machine_Config.b200_default()
        flat = BSA_Config(None, None, {"bsa_repr": pattern, "CP": (cp * cp_inter, 1)})
        shape = {"S": (seq_len, seq_len), "Nh": (n_heads, n_kv_heads or n_heads), "bs": batch, "D": head_dim}
        da = Dist_Attn_Config.from_bsa_config(flat, shape, hierarchy=1)
        graph = Dependent_Graph(get_cc_optimal_schedule_from_table(da, m_config, alloc), fob)
        plan = Execution_Plan(graph, fob, plan_type, time_limit=time_limit)
        plan.allocation = alloc
        return plan
    m_config = m_config or Machine_Config.b200_default()
    cfg = BSA_Config(None, None, {"bsa_repr": pattern if cmap is None else BSA_Repr(pattern.block_table_int, cmap),
                                  "CP": (cp, 1)})
    shape = {"S": (seq_len, seq_len), "Nh": (n_heads, n_kv_heads or n_heads), "bs": batch, "D": head_dim}
    da = Dist_Attn_Config.from_bsa_config(cfg, shape, hierarchy=1)
    if allocation == "naive":
        alloc = naive_allocate_strategy(cfg, fob=fob, hierarchy=1, ParD=ParD)
    elif allocation == "lightseq":
        # LightSeq's balanced causal worker / helper schedule as a fixed table
        from .allocate import Allocation, comm_volumes, comp_volumes, tile_volumes
        from .dense import get_lightseq_schedule_table
        import numpy as np
        table = get_lightseq_schedule_table(cp)
        cm = np.arange(cp)
        cin, cout = comm_volumes(table, cm, cp, fob)
        alloc = Allocation(cp, cm, table, float(max(cin.max(), cout.max())),
                           float(comp_volumes(table, tile_volumes(pattern, cp), cp).max()), "lightseq")
    else:
        alloc = solve_sparse_from_bsa(cfg, fob=fob, ParD=ParD, hierarchy=1, objective=objective,
                                      time_limit=time_limit, cmap=cmap)
    schedule = get_cc_optimal_schedule_from_table(da, m_config, alloc)
    graph = Dependent_Graph(schedule, fob)
    if kernel_tile:
        plan = Graph_Transformation_Engine(None, da, m_config).transform(graph, "greedy", plan_type,
                                                                         time_limit=time_limit)
    else:
        plan = Execution_Plan(graph, fob, plan_type, time_limit=time_limit)
    plan.allocation = alloc
    return plan


def make_plan_collective(group=None, src: int = 0, **kwargs) -> Execution_Plan:
    """Plan on one rank and broadcast the result, so that every rank walks the *same* plan.
    (A time-limited solver may return different incumbents in different processes; the reference
    likewise plans on rank 0 only and shares plans through its database,
    search_algo/task1_bsa.py:917-938.)"""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return make_plan(**kwargs)
    rank = dist.get_rank(group)
    box = [make_plan(**kwargs) if rank == src else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, src) if group is not None else src,
                               group=group)
    return box[0]
