"""Kernel-level tiling: fuse same-rank rectangles of compute tiles into one larger kernel.

A *combinatorial rectangle* is a set of query rows R and key columns C (not necessarily contiguous)
such that every tile (r, c), r in R, c in C, is a non-causal tile scheduled on the same rank. Fusing
it replaces |R|*|C| kernels by one whose inputs are the union of the inputs and whose outputs feed
the union of the outputs: fewer, larger launches (better tensor-core utilisation) that can only
start once every input has arrived. The trade-off is settled by re-lowering each candidate graph
and keeping the best makespan.

Reference: search_algo/graph_transformation_engine.py:30-287 (rectangle search by DFS over rows,
shapes enumerated largest area first up to ceil(tiles / CP), ``greedy`` = non-overlapping in that
order, ``bf`` = every subset).
"""
from __future__ import annotations

import copy
import itertools
import math

import numpy as np

from .graph import Comp_Kernel, Dependent_Graph
from .schedule import Execution_Plan


class Graph_Substitution:
    """A rule that finds every place of a graph where one kind of rewrite applies."""

    def findall(self, d_graph: Dependent_Graph) -> list:
        raise NotImplementedError

    def findall_trans_in_d_graph(self, d_graph: Dependent_Graph, hierarchy_sp: int = 0) -> list:
        """The reference's method name (search_algo/graph_transformation_engine.py:127); the rank
        count is read from the graph here, so the second argument is accepted and unused."""
        return self.findall(d_graph)


class Graph_Transformation:
    """One concrete rewrite of a graph, applied in place."""

    def apply_on_d_graph(self, d_graph: Dependent_Graph) -> None:
        raise NotImplementedError


class Comm_Rebuild_Engine:
    """Placeholder of the reference (search_algo/graph_transformation_engine.py:17-19, an empty
    class there too): rebuilding point-to-point transfers into row / column broadcasts and
    reductions is done by the plan lowering (``runtime.plan_ir``), not by a graph rewrite."""


class Comp_Fusion_Transformation(Graph_Transformation):
    """One rectangle: ``ids = (b, h, rows, cols, rank)``. The reference's constructor takes the
    substitution first (``(sub, ids_tuple)``); both argument lists are accepted."""

    def __init__(self, *args):
        assert 1 <= len(args) <= 2, "Comp_Fusion_Transformation(ids) or (sub, ids)"
        self.sub = args[0] if len(args) == 2 else None
        self.ids = tuple(args[-1])

    @property
    def tiles(self) -> set:
        b, h, rows, cols, g = self.ids
        return {(b, h, r, c, g) for r in rows for c in cols}

    def apply_on_d_graph(self, d_graph: Dependent_Graph) -> None:
        b, h, rows, cols, g = self.ids
        fob = d_graph.fob
        olds = [d_graph.kernel_dict[k] for k in sorted(self.tiles)]
        # cost of the fused tile: merged profile key when the shape is representable, else the sum
        # of the parts minus the per-launch overheads it saves
        t = None
        cm = d_graph.m_config.comp_profile_maps[d_graph.hierarchy] if d_graph.m_config else None
        key = olds[0].comp_map_key
        if cm is not None and hasattr(cm, "merge_comp_map_key") and isinstance(key, tuple):
            try:
                krow = key
                for _ in range(len(cols) - 1):
                    krow = cm.merge_comp_map_key(krow, key, 1)
                kall = krow
                for _ in range(len(rows) - 1):
                    kall = cm.merge_comp_map_key(kall, krow, 0)
                t = np.asarray(cm.get_comp_time_from_map_key(kall), dtype=float)
                key = kall
            except (AssertionError, KeyError, ValueError):
                t = None
        if t is None:
            t = sum(np.asarray(o.time, dtype=float) for o in olds)
        new_key = (b, h, tuple(rows), tuple(cols), g)
        new = Comp_Kernel(new_key, d_graph.m_config, key, d_graph.hierarchy, time=t)
        for o in olds:
            for p in list(o.precursors):
                p.remove_successor(o)
                p.add_successor(new)
                new.add_precursor(p)
            for s in list(o.successors):
                s.remove_precursor(o)
                s.add_precursor(new)
                new.add_successor(s)
            del d_graph.kernel_dict[o.key]
        d_graph.kernel_dict[new_key] = new


class Comp_Fusion_Substitution(Graph_Substitution):
    """All rectangles of a given shape (x rows by y columns) in a graph."""

    def __init__(self, shape: tuple):
        self.shape = shape

    def findall(self, d_graph: Dependent_Graph) -> list:
        x, y = self.shape
        out = []
        by_rank: dict = {}
        for k, v in d_graph.kernel_dict.items():
            if v.type != "comp" or isinstance(k[2], tuple):
                continue
            b, h, r, c, g = k
            if d_graph._tile_type(r, c) != 1:       # only FULL tiles fuse (causal diagonals excluded)
                continue
            by_rank.setdefault((b, h, g), {}).setdefault(r, set()).add(c)
        for (b, h, g), rows in by_rank.items():
            row_ids = sorted(rows)
            for rs in itertools.combinations(row_ids, x):
                common = set.intersection(*(rows[r] for r in rs))
                if len(common) < y:
                    continue
                for cs in itertools.combinations(sorted(common), y):
                    out.append(Comp_Fusion_Transformation((b, h, rs, cs, g)))
        return out


class Graph_Transformation_Engine:
    def __init__(self, exp_config=None, da_config=None, m_config=None, max_candidates: int = 64):
        self.exp_config = exp_config
        self.da_config = da_config
        self.m_config = m_config
        self.max_candidates = max_candidates

    def candidate_shapes(self, d_graph: Dependent_Graph) -> list:
        n_tiles = sum(1 for v in d_graph.kernel_dict.values() if v.type == "comp")
        ub = max(1, math.ceil(n_tiles / max(1, d_graph.hierarchy_sp)))
        n = d_graph.split_degrees[0]
        shapes = [(x, y) for x in range(1, n + 1) for y in range(1, n + 1) if 1 < x * y <= ub]
        shapes.sort(key=lambda s: (-s[0] * s[1], abs(s[0] - s[1])))
        return shapes

    def select_greedy(self, d_graph: Dependent_Graph) -> list:
        used: set = set()
        chosen = []
        for shape in self.candidate_shapes(d_graph):
            for tr in Comp_Fusion_Substitution(shape).findall(d_graph):
                if used.isdisjoint(tr.tiles):
                    used |= tr.tiles
                    chosen.append(tr)
        return chosen

    # ---- the reference's step-by-step interface (search_algo/graph_transformation_engine.py:176-263)
    def calc_subs_dict(self) -> dict:
        """``subs_dict['comp_fusion']``: one substitution per candidate shape, largest area first."""
        assert hasattr(self, "d_graph"), "assign d_graph first (transform() does)"
        self.comp_fusion_shapes = self.candidate_shapes(self.d_graph)
        self.subs_dict = {"comp_fusion": [Comp_Fusion_Substitution(s) for s in self.comp_fusion_shapes],
                          "comm_fusion": []}
        return self.subs_dict

    def get_all_transformations(self) -> list:
        """``trans_all``: every rectangle of every shape; ``trans_sp[rank]`` groups them by rank."""
        if not hasattr(self, "subs_dict"):
            self.calc_subs_dict()
        self.trans_all = [t for sub in self.subs_dict["comp_fusion"] for t in sub.findall(self.d_graph)]
        self.trans_sp = [[] for _ in range(max(1, self.d_graph.hierarchy_sp))]
        for t in self.trans_all:
            self.trans_sp[t.ids[4]].append(t)
        return self.trans_all

    def apply_transformations(self, selected_trans: list, plan_type: str = None,
                              time_limit: float = 20.0) -> Execution_Plan:
        """Lower a copy of the graph with ``selected_trans`` applied."""
        g = copy.deepcopy(self.d_graph)
        for tr in selected_trans:
            tr.apply_on_d_graph(g)
        return Execution_Plan(g, g.fob, plan_type or getattr(self, "plan_type", "Flexflow"),
                              time_limit=time_limit)

    def transform(self, d_graph: Dependent_Graph, transform_mode: str = "greedy",
                  plan_type: str = "Flexflow", time_limit: float = 20.0, mode: str = None) -> Execution_Plan:
        """Return the best plan among the untransformed graph and the fused candidates. ``mode`` is
        the reference's keyword for ``transform_mode``; its ``plan_type='automatic'`` is the list
        schedule here."""
        if mode is not None:
            transform_mode = mode
        if plan_type in ("automatic", "ablation1"):
            plan_type = "Flexflow"
        self.d_graph, self.plan_type = d_graph, plan_type
        base = Execution_Plan(copy.deepcopy(d_graph), d_graph.fob, plan_type, time_limit=time_limit)
        best = base
        if transform_mode == "greedy":
            chosen = self.select_greedy(d_graph)
            candidates = [chosen] if chosen else []
        elif transform_mode == "bf":
            allt = []
            for shape in self.candidate_shapes(d_graph):
                allt += Comp_Fusion_Substitution(shape).findall(d_graph)
            allt = allt[: 12]
            candidates = []
            for n in range(1, len(allt) + 1):
                for sub in itertools.combinations(allt, n):
                    tiles = [t.tiles for t in sub]
                    if sum(len(t) for t in tiles) == len(set().union(*tiles)):
                        candidates.append(list(sub))
                    if len(candidates) >= self.max_candidates:
                        break
                if len(candidates) >= self.max_candidates:
                    break
        else:
            raise ValueError(transform_mode)
        self.selected = []
        for cand in candidates:
            g = copy.deepcopy(d_graph)
            for tr in cand:
                tr.apply_on_d_graph(g)
            plan = Execution_Plan(g, d_graph.fob, plan_type, time_limit=time_limit)
            if plan.end_time < best.end_time:
                best = plan
                self.selected = cand
        return best
