"""FULL / causal dense attention: Y x X grid tables, shape-free plans and schedule look-ups.

Reference: search_algo/dense_utils.py:12-103 (grid allocation ``table[k, l] = S_map[k // X * X +
l % X]``, shape-free "seqlen variable" graphs with a manual plan, ablation over every (Y, X) with
X * Y = CP) and search_algo/manual_schedules.py:8-597, whose literal tables are cached answers of
the allocation program; here they are computed (and memoised) instead of stored.
"""
from __future__ import annotations

import functools

import numpy as np

from ..patterns.blocks import BSA_Config
from ..patterns.named import causal as causal_pattern
from ..patterns.named import full as full_pattern
from .allocate import solve_sparse_from_bsa
from .cost import Dist_Attn_Config, Dist_Attn_Schedule, Machine_Config
from .graph import Dependent_Graph
from .schedule import Execution_Plan


def get_block_schedule_table_for_full(CP: int, X: int, S_map=None) -> np.ndarray:
    S_map = np.arange(CP) if S_map is None else np.asarray(S_map)
    t = np.empty((CP, CP), dtype=np.int64)
    for k in range(CP):
        for l in range(CP):
            t[k, l] = S_map[k // X * X + l % X]
    return t


def get_qo_schedule_table(n: int, causal: bool = False) -> np.ndarray:
    """Every tile runs where its keys live (queries move, outputs come back)."""
    t = np.tile(np.arange(n)[None, :], (n, 1))
    if causal:
        t[np.triu_indices(n, 1)] = -1
    return t


def get_kv_schedule_table(n: int, causal: bool = False) -> np.ndarray:
    """Every tile runs where its queries live (keys/values move: ring-like)."""
    t = np.tile(np.arange(n)[:, None], (1, n))
    if causal:
        t[np.triu_indices(n, 1)] = -1
    return t


def get_lightseq_schedule_table(n: int) -> np.ndarray:
    """Balanced causal allocation of LightSeq's DistAttn (reference:
    easy_context/dist_flash_attn/lightseq_async_attn.py:244-435, a vendored baseline that runs
    n/2 + 1 time steps). Tile (i, j), j <= i, at distance d = i - j runs on its query owner i
    ("worker": keys/values travel) when d <= n // 2 and on its key owner j ("helper": the query
    block travels, the partial (O, lse) comes back and is merged) otherwise. Every rank ends up with
    n // 2 or n // 2 + 1 tiles. Expressed as an allocation table, the schedule runs on any of this
    framework's executors; the time-step structure of the original (one send/recv pair per step)
    is what the launch-order scheduler recovers from the dependencies."""
    t = np.full((n, n), -1, dtype=np.int64)
    for i in range(n):
        for j in range(i + 1):
            t[i, j] = i if i - j <= n // 2 else j
    return t


@functools.lru_cache(maxsize=None)
def _cc_optimal(n: int, causal: bool, fob: int, time_limit: float):
    pat = causal_pattern(1) if causal else full_pattern(1)
    cfg = BSA_Config(None, None, {"bsa_repr": pat, "CP": (n, 1)})
    al = solve_sparse_from_bsa(cfg, fob=fob, time_limit=time_limit)
    return np.asarray(al.table)


def get_cc_optimal_schedule_table(n: int, causal: bool = False, fob: int = 0, time_limit: float = 30.0) -> np.ndarray:
    """Communication-optimal, compute-balanced allocation of an n x n dense problem on n ranks."""
    return _cc_optimal(n, causal, fob, time_limit).copy()


def get_full_ablation_suffix(Y: int, X: int, dim: int = 0) -> str:
    return f"_ablation=(Y={Y},X={X},dim={dim})"


def create_ablation_configs_for_full(CP: int) -> list:
    return [(CP // x, x) for x in range(1, CP + 1) if CP % x == 0]


def ablation_dicts_for_full(hierarchy_cp: int, KERNEL_TILE_TYPEs=None) -> list:
    """The (Y, X) grids of FULL attention in the record form of the reference's campaign
    (search_algo/dense_utils.py:77-98): one dict per kernel-tile setting and grid, X ascending."""
    kinds = ["w/o_kernel_tile"] if KERNEL_TILE_TYPEs is None else list(KERNEL_TILE_TYPEs)
    return [{"Y": y, "X": x, "first_dim": 0, "KERNEL_TILE_TYPE": kind}
            for kind in kinds for y, x in create_ablation_configs_for_full(hierarchy_cp)]


def create_plan_key_suffixes_for_full(hierarchy_cp: int) -> list:
    """Plan-key suffixes of those grids, in the same order (search_algo/dense_utils.py:100-103)."""
    return [get_full_ablation_suffix(ad["Y"], ad["X"], ad["first_dim"]) for ad in ablation_dicts_for_full(hierarchy_cp)]


def create_plan_for_full(CP: int, X: int, fob: int, m_config: Machine_Config = None, shape_config=None,
                         first_dim: int = 0, hierarchy: int = 1) -> Execution_Plan:
    """Manual plan of FULL attention on a Y x X grid. Without ``shape_config`` the graph is
    shape-free (placeholder kernel times) and can be materialised for a shape later.
    ``hierarchy``: 1 = the grid spans the ``CP`` ranks of a node, 0 = ``CP`` nodes."""
    cfg = BSA_Config.create_full((CP, 1) if hierarchy else (1, CP))
    m_config = m_config or Machine_Config.b200_default()
    svg = shape_config is None
    shape = shape_config or {"S": (CP * 1024, CP * 1024), "Nh": (1, 1), "bs": 1, "D": 128}
    da = Dist_Attn_Config.from_bsa_config(cfg, shape, hierarchy=hierarchy)
    table = get_block_schedule_table_for_full(CP, X)
    sched = Dist_Attn_Schedule(da, m_config, (CP, CP, 1, 1), np.arange(CP)[None, :], table[None, None])
    g = Dependent_Graph(sched, fob, seqlen_variable_graph=svg)
    return Execution_Plan(g, fob, "manual", X=X, first_dim=first_dim)


def write_plan(execute_plan: Execution_Plan, prefix: str) -> str:
    """Store a plan as ``<prefix>/<plan name>.pkl`` with its JSON side-car next to it and read it
    back as a check (reference: search_algo/dense_utils.py:53-62). Returns the pickle's path."""
    import os
    import pickle
    from . import bind_reference_class_paths
    bind_reference_class_paths()
    os.makedirs(prefix, exist_ok=True)
    path = os.path.join(prefix, execute_plan.get_plan_name() + ".pkl")
    with open(path, "wb") as f:
        pickle.dump(execute_plan, f)
    execute_plan.to_json(path[:-4] + ".json")
    with open(path, "rb") as f:
        assert pickle.load(f).get_plan_name() == execute_plan.get_plan_name()
    return path


def split_dense_configs(dense_configs: list) -> tuple:
    """(full configs, causal configs) of a list of dense one-block patterns."""
    full, causal = [], []
    for c in dense_configs:
        tab = c.bsa_repr.table
        assert tab.shape == (1, 1), "dense patterns coarsen to a single block"
        if tab[0, 0] == 1:
            full.append(c)
        elif tab[0, 0] == 2:
            causal.append(c)
        else:
            raise ValueError("an empty pattern is not a dense configuration")
    return full, causal
