"""Device-/node-level context tiling: which rank computes which (query block, key block) tile.

This is the first integer program of the planner ("ILP #1", reference:
search_algo/workload_partition.py:271-470). Decision: binary x[i,j,g] = tile (i,j) runs on rank g.
A rank that computes a tile needs the Q-side data of row i and the K/V-side data of column j; if it
does not own them they are sent once per (row-or-column, rank) — broadcast-once semantics — and
partial outputs flow back the same way. With a[g,i] / b[g,j] the indicators "rank g touches row
i / column j":

    A_g = # foreign rows g needs            C_g = # (row of g, foreign rank) pairs that need it
    B_g = # foreign columns g needs         D_g = # (column of g, foreign rank) pairs
    forward : Cin = A + C + 2B            Cout = A + C + 2D
    backward: Cin = 2A + 2B + C + 2D      Cout = A + 2B + 2C + 2D

and the objective is min max_g(Cin_g, Cout_g) under a per-rank compute bound. Diagonal tiles are
pinned to the owner of their row when every diagonal tile is non-empty.

Differences from the reference, on purpose:
  * the compute bound starts at ceil(total / CP) rounded to the 0.5-unit granularity of causal
    tiles and is relaxed in 0.5 steps until the program is feasible, instead of literal fudge
    factors keyed on (CP, total) (reference :424-436);
  * ``objective="time"`` minimises max(compute_g * t_comp, Cin_g * t_comm, Cout_g * t_comm) with
    the communication volume as tie-break — on an NVSwitch box communication is an order of
    magnitude cheaper relative to compute than on the clusters the reference was tuned for, so
    load balance has to be part of the objective;
  * ownership (``cmap``) may be any map, not only contiguous chunks, which is how a context remap
    enters the program.
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from ..patterns.blocks import BSA_Config, BSA_Repr, _VOLUME
from .solver import Model

EMPTY_TILE = -1       # schedule_table value for a tile nobody computes
UNSETTLED = -2


@dataclass
class Allocation:
    """Result of ILP #1. ``table[i, j]`` = rank that computes tile (i, j) (-1: empty)."""
    Par_D: int
    cmap: np.ndarray
    table: np.ndarray
    comm_volume: float = float("nan")     # max_g max(Cin_g, Cout_g), in Q-tile units
    comp_max: float = float("nan")        # max_g compute volume, in full-tile units
    status: str = "optimal"

    def as_dict(self) -> dict:
        return {"Par_D": self.Par_D, "cmap": self.cmap, "table": self.table}

    def __getitem__(self, k):
        return self.as_dict()[k]


def tile_volumes(pattern: BSA_Repr, par_d: int) -> np.ndarray:
    """Compute volume of each tile of the par_d x par_d partition, in units of one FULL tile at
    that granularity."""
    cur = pattern.table.shape[0]
    if par_d >= cur:
        return _VOLUME[pattern.refined(par_d)]
    assert cur % par_d == 0
    f = cur // par_d
    v = _VOLUME[pattern.table].reshape(par_d, f, par_d, f).sum(axis=(1, 3)) / (f * f)
    return v


def comm_volumes(table: np.ndarray, cmap: np.ndarray, cp: int, fob: int):
    """(Cin, Cout) per rank for a given allocation table, with the weights of the docstring."""
    n = table.shape[0]
    a = np.zeros((cp, n), dtype=bool)
    b = np.zeros((cp, n), dtype=bool)
    for i in range(n):
        for j in range(n):
            g = table[i, j]
            if g >= 0:
                a[g, i] = True
                b[g, j] = True
    A = np.array([sum(a[g, i] for i in range(n) if cmap[i] != g) for g in range(cp)], dtype=float)
    B = np.array([sum(b[g, j] for j in range(n) if cmap[j] != g) for g in range(cp)], dtype=float)
    C = np.array([sum(a[k, i] for i in range(n) if cmap[i] == g for k in range(cp) if k != g)
                  for g in range(cp)], dtype=float)
    D = np.array([sum(b[k, j] for j in range(n) if cmap[j] == g for k in range(cp) if k != g)
                  for g in range(cp)], dtype=float)
    if fob == 0:
        return A + C + 2 * B, A + C + 2 * D
    return 2 * A + 2 * B + C + 2 * D, A + 2 * B + 2 * C + 2 * D


def comp_volumes(table: np.ndarray, vol: np.ndarray, cp: int) -> np.ndarray:
    return np.array([vol[table == g].sum() for g in range(cp)])


def naive_allocate_strategy(bsa_config: BSA_Config, fob: int = 0, hierarchy: int = 1,
                            ParD: Optional[int] = None) -> Allocation:
    """Row-owner allocation (every tile runs where its queries live; K/V move, ring-like).
    The "without device tile" ablation of the reference (workload_partition.py:550-587)."""
    cp = bsa_config.CP[0] if hierarchy == 1 else bsa_config.CP[1]
    par_d = ParD or max(cp, bsa_config.table.shape[0])
    vol = tile_volumes(bsa_config.bsa_repr, par_d)
    cmap = _default_cmap(bsa_config, par_d, cp)
    table = np.full((par_d, par_d), EMPTY_TILE, dtype=np.int64)
    for i in range(par_d):
        table[i, vol[i] > 0] = cmap[i]
    cin, cout = comm_volumes(table, cmap, cp, fob)
    return Allocation(par_d, cmap, table, float(max(cin.max(), cout.max())),
                      float(comp_volumes(table, vol, cp).max()), "naive")


def comp_balance_allocate_strategy(bsa_config: BSA_Config, fob: int = 0, hierarchy: int = 1,
                                   ParD: Optional[int] = None) -> Allocation:
    """Compute-balanced allocation that ignores traffic ("like zigzag"; a stub that raises in the
    reference, workload_partition.py:589-591): diagonal tiles stay with their owners, the other
    tiles go, heaviest first, to the least loaded rank, preferring the owner of the tile's
    queries, then of its keys, on ties. An upper bound on what balancing alone can achieve; the
    ILP trades some of it for traffic."""
    cp = bsa_config.CP[0] if hierarchy == 1 else bsa_config.CP[1]
    par_d = ParD or max(2 * cp, bsa_config.table.shape[0])
    vol = tile_volumes(bsa_config.bsa_repr, par_d)
    cmap = _default_cmap(bsa_config, par_d, cp)
    table = np.full((par_d, par_d), EMPTY_TILE, dtype=np.int64)
    load = np.zeros(cp)
    rest = []
    for i in range(par_d):
        for j in range(par_d):
            if vol[i, j] <= 0:
                continue
            if i == j:
                table[i, j] = cmap[i]
                load[cmap[i]] += vol[i, j]
            else:
                rest.append((i, j))
    rest.sort(key=lambda t: (-vol[t], t))
    for i, j in rest:
        low = load.min()
        cands = [g for g in range(cp) if load[g] <= low + 1e-9]
        g = cmap[i] if cmap[i] in cands else cmap[j] if cmap[j] in cands else cands[0]
        table[i, j] = g
        load[g] += vol[i, j]
    cin, cout = comm_volumes(table, cmap, cp, fob)
    return Allocation(par_d, cmap, table, float(max(cin.max(), cout.max())), float(load.max()), "comp_balance")


def _default_cmap(bsa_config: BSA_Config, par_d: int, cp: int) -> np.ndarray:
    if bsa_config.cmap is not None and len(bsa_config.cmap) == par_d:
        return np.asarray(bsa_config.cmap)
    return np.arange(par_d) // (par_d // cp)


def _score(table, cmap, cp, fob, vol, objective, t_comp, t_comm, comp_ub, diag_pinned=None):
    """Lexicographic score of an allocation (smaller is better); None if it breaks the bound."""
    comp = comp_volumes(table, vol, cp)
    cin, cout = comm_volumes(table, cmap, cp, fob)
    cmax = float(max(cin.max(), cout.max()))
    if objective == "comm":
        if comp.max() > comp_ub + 1e-9:
            return None
        return (cmax, float(cin.sum() + cout.sum()), float(comp.max()))
    t = max(float(comp.max()) * t_comp, cmax * t_comm)
    return (t, cmax, float(cin.sum() + cout.sum()))


def grid_table(par_d: int, cp: int, cmap: np.ndarray, vol: np.ndarray, X: int) -> np.ndarray:
    """Y x X grid allocation (reference: search_algo/dense_utils.py:19-31): the rank that owns
    row-chunk k and column-chunk l of the CP x CP chunk grid is ``k // X * X + l % X``."""
    table = np.full((par_d, par_d), EMPTY_TILE, dtype=np.int64)
    for i in range(par_d):
        for j in range(par_d):
            if vol[i, j] > 0:
                table[i, j] = cmap[i] // X * X + cmap[j] % X
    return table


def heuristic_candidates(par_d, cp, cmap, vol, diagonal_full):
    """Cheap structured allocations: row owner, column owner, every Y x X grid, anti-diagonal."""
    cands = []
    rows = np.full((par_d, par_d), EMPTY_TILE, dtype=np.int64)
    cols = rows.copy()
    anti = rows.copy()
    for i in range(par_d):
        for j in range(par_d):
            if vol[i, j] > 0:
                rows[i, j] = cmap[i]
                cols[i, j] = cmap[j]
                anti[i, j] = cmap[i] if (i + j) % 2 == 0 else cmap[j]
    cands += [rows, cols, anti]
    for X in range(1, cp + 1):
        if cp % X == 0:
            cands.append(grid_table(par_d, cp, cmap, vol, X))
    if diagonal_full:
        for t in cands:
            for i in range(par_d):
                t[i, i] = cmap[i]
    return cands


def local_search(table, cmap, cp, fob, vol, objective, t_comp, t_comm, comp_ub, diagonal_full,
                 iters: int = 4000, seed: int = 0):
    """Single-tile reassignment hill climbing on the lexicographic score."""
    rng = np.random.default_rng(seed)
    par_d = table.shape[0]
    movable = [(i, j) for i in range(par_d) for j in range(par_d)
               if table[i, j] >= 0 and not (i == j and diagonal_full)]
    best = _score(table, cmap, cp, fob, vol, objective, t_comp, t_comm, comp_ub)
    if not movable:
        return table, best
    table = table.copy()
    for _ in range(iters):
        i, j = movable[rng.integers(len(movable))]
        old = table[i, j]
        # candidate ranks: owners of the row / column first (they add no new traffic), then any
        g = [cmap[i], cmap[j], int(rng.integers(cp))][int(rng.integers(3))]
        if g == old:
            continue
        table[i, j] = g
        sc = _score(table, cmap, cp, fob, vol, objective, t_comp, t_comm, comp_ub)
        if sc is not None and (best is None or sc <= best):
            best = sc
        else:
            table[i, j] = old
    return table, best


def solve_sparse_from_bsa(bsa_config: BSA_Config, fob: int = 0, ParD: Optional[int] = None,
                          hierarchy: int = 1, *, cmap: Optional[Sequence[int]] = None,
                          objective: str = "comm", t_comp: float = 1.0, t_comm: float = 0.05,
                          time_limit: float = 300.0, backend: Optional[str] = None,
                          max_slack_steps: int = 8, use_ilp: bool = True,
                          heuristic_iters: int = 3000) -> Allocation:
    """Solve ILP #1 for ``bsa_config`` at level ``hierarchy`` (1 = ranks inside a node,
    0 = nodes). Returns an :class:`Allocation` (dict-like: 'Par_D', 'cmap', 'table')."""
    cp = bsa_config.CP[0] if hierarchy == 1 else bsa_config.CP[1]
    par_d = ParD or max(cp, bsa_config.table.shape[0])
    assert par_d % cp == 0, f"ParD={par_d} must be a multiple of CP={cp}"
    vol = tile_volumes(bsa_config.bsa_repr, par_d)
    cm = np.asarray(cmap) if cmap is not None else _default_cmap(bsa_config, par_d, cp)
    if cp == 1:
        table = np.where(vol > 0, 0, EMPTY_TILE)
        return Allocation(par_d, cm, table, 0.0, float(vol.sum()), "optimal")
    key = None
    if use_ilp and objective == "comm" and hierarchy == 1:
        key = allocation_cache_key(bsa_config, fob, cp, par_d, cm)
        hit = _cache_lookup(key, par_d, cp, vol)
        if hit is not None:
            table = hit
            cin, cout = comm_volumes(table, cm, cp, fob)
            return Allocation(par_d, cm, table, float(max(cin.max(), cout.max())),
                              float(comp_volumes(table, vol, cp).max()), "cached")
    alloc = _solve_uncached(bsa_config, fob, par_d, cp, cm, vol, objective, t_comp, t_comm, time_limit, backend,
                            max_slack_steps, use_ilp, heuristic_iters)
    if key is not None:
        _cache_store(key, alloc)
    return alloc


# ---------------------------------------------------------------------------------------------
# Cached answers. The reference keeps the results of this program in
# ``{intra,inter}_bsa_allocation.json`` of its plan database ("Bypassed !!!",
# search_algo/task1_bsa.py:106-143) and as literal tables (search_algo/manual_schedules.py:36-597).
# Here: a read-only file shipped with the package (the named benchmark patterns on 2 / 4 / 8 ranks,
# solved with a long time limit) plus an optional writable directory ``UA_PLAN_CACHE``. A cached
# table is only used if it is a valid allocation of the present pattern. ``UA_PLAN_CACHE=0``
# switches both off.
# ---------------------------------------------------------------------------------------------
_SHIPPED = None


def allocation_cache_key(bsa_config: BSA_Config, fob: int, cp: int, par_d: int, cmap: np.ndarray) -> str:
    contiguous = np.array_equal(cmap, np.arange(par_d) // (par_d // cp))
    cm = "contiguous" if contiguous else "-".join(str(int(x)) for x in cmap)
    return f"fob={int(fob)}_CP={cp}_ParD={par_d}_cmap={cm}_repr={bsa_config.bsa_repr}"


def _cache_files():
    import os
    from pathlib import Path
    env = os.environ.get("UA_PLAN_CACHE")
    if env == "0":
        return None, None
    shipped = Path(__file__).resolve().parents[1] / "data" / "allocations.json"
    user = Path(env) / "allocations.json" if env else None
    return shipped, user


def _cache_lookup(key: str, par_d: int, cp: int, vol: np.ndarray):
    import json
    global _SHIPPED
    shipped, user = _cache_files()
    if shipped is None:
        return None
    if _SHIPPED is None:
        _SHIPPED = json.loads(shipped.read_text()) if shipped.exists() else {}
    entry = _SHIPPED.get(key)
    if entry is None and user is not None and user.exists():
        entry = json.loads(user.read_text()).get(key)
    if entry is None:
        return None
    table = np.asarray(entry["table"], dtype=np.int64)
    ok = (table.shape == (par_d, par_d) and ((table >= 0) == (vol > 0)).all() and table.max() < cp)
    return table if ok else None


def _cache_store(key: str, alloc: "Allocation") -> None:
    import json
    import os
    _, user = _cache_files()
    if user is None:
        return
    user.parent.mkdir(parents=True, exist_ok=True)
    data = json.loads(user.read_text()) if user.exists() else {}
    data[key] = {"table": np.asarray(alloc.table).tolist(), "comm_volume": alloc.comm_volume,
                 "comp_max": alloc.comp_max, "status": alloc.status}
    tmp = user.with_suffix(f".tmp{os.getpid()}")
    tmp.write_text(json.dumps(data))
    os.replace(tmp, user)


def _solve_uncached(bsa_config, fob, par_d, cp, cm, vol, objective, t_comp, t_comm, time_limit, backend,
                    max_slack_steps, use_ilp, heuristic_iters) -> Allocation:

    diagonal_full = bool((np.diag(vol) > 0).all())
    tiles = [(i, j) for i in range(par_d) for j in range(par_d)
             if vol[i, j] > 0 and not (i == j and diagonal_full)]
    diag_comp = np.array([sum(vol[i, i] for i in range(par_d) if cm[i] == g) if diagonal_full else 0.0
                          for g in range(cp)])
    total = float(vol.sum())
    base_ub = math.ceil(total / cp * 2) / 2.0           # 0.5-unit granularity
    base_ub = max(base_ub, float(diag_comp.max()))

    for step in range(max_slack_steps + 1):
        ub = base_ub + 0.5 * step
        # 1. structured candidates + hill climbing give an incumbent quickly
        inc, inc_score = None, None
        for cand in heuristic_candidates(par_d, cp, cm, vol, diagonal_full):
            t, sc = local_search(cand, cm, cp, fob, vol, objective, t_comp, t_comm, ub,
                                 diagonal_full, iters=heuristic_iters)
            if sc is not None and (inc_score is None or sc < inc_score):
                inc, inc_score = t, sc
        # 2. the integer program has to beat the incumbent (objective cut-off)
        cutoff = None if inc_score is None else inc_score[0]
        sol = None
        if use_ilp:
            sol = _solve_once(par_d, cp, cm, vol, tiles, diagonal_full, diag_comp, fob, ub,
                              objective, t_comp, t_comm, time_limit, backend, cutoff)
        if sol is not None:
            table, status = sol
        elif inc is not None:
            table, status = inc, "heuristic"
        else:
            if objective == "time":
                break
            continue
        cin, cout = comm_volumes(table, cm, cp, fob)
        return Allocation(par_d, cm, table, float(max(cin.max(), cout.max())),
                          float(comp_volumes(table, vol, cp).max()), status)
    raise RuntimeError(f"tile allocation infeasible for {bsa_config} (ParD={par_d})")


def _solve_once(par_d, cp, cmap, vol, tiles, diagonal_full, diag_comp, fob, comp_ub, objective,
                t_comp, t_comm, time_limit, backend, cutoff=None):
    m = Model("workload_allocation")
    x = {(i, j, g): m.add_binary(f"x_{i}_{j}_{g}") for (i, j) in tiles for g in range(cp)}
    a = {(g, i): m.add_var(f"a_{g}_{i}", 0, 1) for g in range(cp) for i in range(par_d)}
    b = {(g, j): m.add_var(f"b_{g}_{j}", 0, 1) for g in range(cp) for j in range(par_d)}
    cin = [m.add_var(f"Cin_{g}") for g in range(cp)]
    cout = [m.add_var(f"Cout_{g}") for g in range(cp)]
    comm = m.add_var("Comm_Volume")
    for (i, j) in tiles:
        m.add_constr({x[i, j, g]: 1.0 for g in range(cp)}, "==", 1.0)
    for (i, j) in tiles:
        for g in range(cp):
            m.add_constr({a[g, i]: 1.0, x[i, j, g]: -1.0}, ">=", 0.0)
            m.add_constr({b[g, j]: 1.0, x[i, j, g]: -1.0}, ">=", 0.0)
    if diagonal_full:
        for i in range(par_d):      # pinned diagonal tiles touch their own row and column
            m.add_constr({a[cmap[i], i]: 1.0}, ">=", 1.0)
            m.add_constr({b[cmap[i], i]: 1.0}, ">=", 1.0)

    def lin(weights):   # weights: list of (coef, dict var->1)
        out = {}
        for coef, vs in weights:
            for v in vs:
                out[v] = out.get(v, 0.0) + coef
        return out

    for g in range(cp):
        A = [a[g, i] for i in range(par_d) if cmap[i] != g]
        B = [b[g, j] for j in range(par_d) if cmap[j] != g]
        C = [a[k, i] for i in range(par_d) if cmap[i] == g for k in range(cp) if k != g]
        D = [b[k, j] for j in range(par_d) if cmap[j] == g for k in range(cp) if k != g]
        if fob == 0:
            e_in = lin([(1, A), (1, C), (2, B)])
            e_out = lin([(1, A), (1, C), (2, D)])
        else:
            e_in = lin([(2, A), (2, B), (1, C), (2, D)])
            e_out = lin([(1, A), (2, B), (2, C), (2, D)])
        e_in[cin[g]] = -1.0
        e_out[cout[g]] = -1.0
        m.add_constr(e_in, "==", 0.0)
        m.add_constr(e_out, "==", 0.0)
        m.add_constr({cin[g]: 1.0, comm: -1.0}, "<=", 0.0)
        m.add_constr({cout[g]: 1.0, comm: -1.0}, "<=", 0.0)

    comp_expr = [{x[i, j, g]: float(vol[i, j]) for (i, j) in tiles} for g in range(cp)]
    if objective == "comm":
        for g in range(cp):
            if comp_expr[g]:
                m.add_constr(comp_expr[g], "<=", comp_ub - float(diag_comp[g]))
        if cutoff is not None:      # volumes are integers: strictly better means at least one less
            m.add_constr({comm: 1.0}, "<=", cutoff - 1.0)
        m.minimize({comm: 1.0})
    elif objective == "time":
        T = m.add_var("T")
        for g in range(cp):
            e = {k: v * t_comp for k, v in comp_expr[g].items()}
            e[T] = -1.0
            m.add_constr(e, "<=", -float(diag_comp[g]) * t_comp)
            m.add_constr({cin[g]: t_comm, T: -1.0}, "<=", 0.0)
            m.add_constr({cout[g]: t_comm, T: -1.0}, "<=", 0.0)
        if cutoff is not None:
            m.add_constr({T: 1.0}, "<=", cutoff * (1.0 - 1e-6))
        m.minimize({T: 1.0, comm: 1e-3 * t_comm})
    else:
        raise ValueError(f"unknown objective {objective!r}")

    sol = m.solve(time_limit=time_limit, backend=backend)
    if not sol.ok:
        return None
    table = np.full((par_d, par_d), EMPTY_TILE, dtype=np.int64)
    if diagonal_full:
        for i in range(par_d):
            table[i, i] = cmap[i]
    for (i, j) in tiles:
        g = int(np.argmax([sol.value(x[i, j, g]) for g in range(cp)]))
        table[i, j] = g
    return table, sol.status


def brute_force_allocate(bsa_config: BSA_Config, fob: int = 0, ParD: Optional[int] = None,
                         hierarchy: int = 1, cmap=None, comp_ub: Optional[float] = None) -> Allocation:
    """Exhaustive search over tile -> rank maps (only for tiny cases; the optimality oracle of the
    ILP tests, and the spirit of the reference's disabled brute-force engine,
    search_algo/search_engine.py:793-884)."""
    cp = bsa_config.CP[0] if hierarchy == 1 else bsa_config.CP[1]
    par_d = ParD or max(cp, bsa_config.table.shape[0])
    vol = tile_volumes(bsa_config.bsa_repr, par_d)
    cm = np.asarray(cmap) if cmap is not None else _default_cmap(bsa_config, par_d, cp)
    diagonal_full = bool((np.diag(vol) > 0).all())
    tiles = [(i, j) for i in range(par_d) for j in range(par_d)
             if vol[i, j] > 0 and not (i == j and diagonal_full)]
    assert cp ** len(tiles) <= 5_000_000, "brute force is for tiny cases only"
    if comp_ub is None:
        diag_comp = max((sum(vol[i, i] for i in range(par_d) if cm[i] == g) if diagonal_full else 0.0)
                        for g in range(cp))
        comp_ub = max(math.ceil(vol.sum() / cp * 2) / 2.0, diag_comp)
    base = np.full((par_d, par_d), EMPTY_TILE, dtype=np.int64)
    if diagonal_full:
        for i in range(par_d):
            base[i, i] = cm[i]
    best = None
    while best is None:
        for assign in itertools.product(range(cp), repeat=len(tiles)):
            t = base.copy()
            for (i, j), g in zip(tiles, assign):
                t[i, j] = g
            if comp_volumes(t, vol, cp).max() > comp_ub + 1e-9:
                continue
            cin, cout = comm_volumes(t, cm, cp, fob)
            c = max(cin.max(), cout.max())
            if best is None or c < best[0]:
                best = (c, t)
        comp_ub += 0.5
    return Allocation(par_d, cm, best[1], float(best[0]), float(comp_volumes(best[1], vol, cp).max()),
                      "optimal")


def search_context_remap(bsa_config: BSA_Config, fob: int = 0, ParD: Optional[int] = None,
                         candidates=("contiguous", "strided", "zigzag"), time_limit: float = 10.0) -> dict:
    """Context remap as a planner stage: try a small set of ownership maps (which rank owns which
    block of the sequence) and keep the one whose best allocation is cheapest, i.e. lowest
    worst-rank traffic, ties broken by the busiest rank's compute.

    The reference draws this stage in its overview (strided attention -> remapped context -> node
    / device / kernel tiles) but only ships its hand-made result for one pattern and the hook
    (``cmap``; "[TODO]: Explore the best cmap", search_algo/bsa_config.py:417-418). Returns
    ``{"name", "cmap", "allocation", "permutation", "scores"}``; ``permutation`` (block order that
    makes every rank's blocks contiguous) is what the data loader applies to token / position ids
    (``apply_block_permutation``) so that rank r simply holds the r-th chunk of the permuted
    sequence."""
    from ..patterns.named import cmap_contiguous, cmap_strided, cmap_zigzag, remap_permutation
    cp = bsa_config.CP[0]
    par_d = ParD or max(cp, bsa_config.table.shape[0])
    makers = {"contiguous": cmap_contiguous, "strided": cmap_strided, "zigzag": cmap_zigzag}
    scores, best = {}, None
    for name in candidates:
        if name == "zigzag" and par_d % (2 * cp):
            continue
        if par_d % cp:
            continue
        cmap = makers[name](par_d, cp)
        al = solve_sparse_from_bsa(bsa_config, fob=fob, ParD=par_d, time_limit=time_limit, cmap=cmap)
        scores[name] = (float(al.comm_volume), float(al.comp_max))
        if best is None or scores[name] < scores[best[0]]:
            best = (name, cmap, al)
    if best is None:
        raise ValueError(f"no ownership map fits {par_d} blocks on {cp} ranks")
    name, cmap, al = best
    return {"name": name, "cmap": cmap, "allocation": al, "permutation": remap_permutation(cmap), "scores": scores}


def apply_block_permutation(x, permutation, dim: int = 1):
    """Reorder the blocks of a ``[..., tokens, ...]`` tensor along ``dim``: block ``permutation[i]``
    of the input becomes block i of the output (token ids, position ids, targets at data-loading
    time; the inverse permutation restores the order)."""
    import torch
    n = len(permutation)
    blk = x.shape[dim] // n
    assert blk * n == x.shape[dim], "the token count is not a multiple of the number of blocks"
    idx = torch.cat([torch.arange(int(p) * blk, (int(p) + 1) * blk) for p in permutation]).to(x.device)
    return x.index_select(dim, idx)
