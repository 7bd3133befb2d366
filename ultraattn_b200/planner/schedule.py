"""Lowering a dependent kernel graph to a launch order: the second integer program of the planner.

Every rank has three logical streams — 0 compute, 1 send, 2 receive. A message occupies the
sender's stream 1 *and* the receiver's stream 2 for its whole duration. The plan is the order in
which each rank launches its kernels (``gpu_kernel_lists[rank]``); ordering between streams is
enforced at run time by events on the graph's edges.

Plan types (reference: search_algo/execute_plan.py:111-747):
  * ``ILP``      — minimise the makespan: continuous ``start[v]``, one binary per same-stream pair
                   deciding their order (big-M disjunction), precedence along graph edges.
                   The list schedule below provides the incumbent, a valid big-M and the fallback
                   when the solver hits its time limit.
  * ``Flexflow`` — event-driven list scheduling: among ready kernels take the one that can start
                   earliest (ties: longest remaining path first).
  * ``manual``   — fixed ring-shifted order for FULL attention on a Y x X grid.
After any of them the per-stream orders are kept and start times are relaxed to the earliest
feasible ones (``fine_tune_kernel_time``), then stream exclusivity is checked.

``Fused_Execution_Plan`` is the kernel-tile extreme for FULL attention: all-gather inputs along the
row group (X ranks) and the column group (Y ranks), one compute kernel, reduce outputs.
"""
from __future__ import annotations

import heapq
import json
from typing import Optional

import numpy as np

from .graph import Comm_Kernel, Comp_Kernel, Cuda_Kernel, Dependent_Graph
from .solver import Model

STREAM_COMP, STREAM_SEND, STREAM_RECV = 0, 1, 2


class Execution_Plan:
    def __init__(self, d_graph: Optional[Dependent_Graph], fob: int, plan_type: Optional[str] = "ILP",
                 is_hack: bool = False, time_limit: float = 60.0, backend: Optional[str] = None,
                 X: Optional[int] = None, first_dim: int = 0):
        self.d_graph = d_graph
        self.fob = fob
        self.plan_type = plan_type if plan_type is not None else "manual"
        self.stream_num = 3
        self.valid_kernels: list = []
        self.stream_kernel_lists: dict = {}
        self.gpu_kernel_lists: list = []
        self.end_time = 0.0
        self.mylp_obj = None
        self.time_limit = time_limit
        self.backend = backend
        if d_graph is None:
            return
        if self.plan_type == "manual":
            self.X = X or 1
            self.Y = self.hierarchy_sp // self.X
            self.first_dim = first_dim
        self.generate()

    # deducible ---------------------------------------------------------------------------------
    @property
    def da_config(self): return self.d_graph.da_config
    @property
    def m_config(self): return self.d_graph.m_config
    @property
    def split_degrees(self): return self.d_graph.split_degrees
    @property
    def hierarchy(self): return self.d_graph.hierarchy
    @property
    def hierarchy_sp(self): return self.d_graph.hierarchy_sp
    @property
    def tot_sp(self): return self.d_graph.tot_sp

    def get_end_time(self) -> float:
        return self.end_time

    def get_plan_name(self) -> str:
        return f"{self.da_config}_fob={self.fob}_{self.plan_type}"

    # -------------------------------------------------------------------------------------------
    def _collect(self) -> None:
        fob = self.fob
        self.valid_kernels = []
        for v in self.d_graph.kernel_dict.values():
            if not v.is_empty(fob):
                v.id = len(self.valid_kernels)
                self.valid_kernels.append(v)
        self.stream_kernel_lists = {(g, s): [] for g in range(self.hierarchy_sp) for s in range(3)}
        for v in self.valid_kernels:
            for key in self._streams_of(v):
                self.stream_kernel_lists[key].append(v)

    @staticmethod
    def _streams_of(v: Cuda_Kernel):
        if v.type == "comp":
            return [(v.key[-1], STREAM_COMP)]
        return [(v.key[3], STREAM_SEND), (v.key[4], STREAM_RECV)]

    def generate(self) -> None:
        self._collect()
        if self.plan_type == "Flexflow":
            self._list_schedule()
        elif self.plan_type == "ILP":
            self._list_schedule()
            incumbent = {v: v._start_time for v in self.valid_kernels}
            ub = max((incumbent[v] + v.time[self.fob] for v in self.valid_kernels), default=0.0)
            if ub <= self._makespan_lower_bound() * (1.0 + 1e-9):
                self.mylp_obj = ub           # the list schedule is provably optimal
            elif not self._solve_ilp(ub):
                for v, t in incumbent.items():
                    v._start_time = t
        elif self.plan_type == "manual":
            if not self._manual_order():
                self._list_schedule()
        else:
            raise ValueError(f"unknown plan_type {self.plan_type!r}")
        self._finalize()

    generate_execution_plan = generate

    def _makespan_lower_bound(self) -> float:
        """max(critical path, busiest stream)."""
        fob = self.fob
        load = max((sum(k.time[fob] for k in lst) for lst in self.stream_kernel_lists.values()), default=0.0)
        return max(self.d_graph.critical_path(), load)

    # ------------------------------- list scheduling -------------------------------------------
    def _rank_to_sink(self) -> dict:
        fob = self.fob
        memo: dict = {}
        order = self._topological_order()
        for v in reversed(order):
            memo[v] = v.time[fob] + max((memo[s] for s in v.successors), default=0.0)
        return memo

    def _topological_order(self) -> list:
        indeg = {v: len(v.precursors) for v in self.valid_kernels}
        ready = [v for v in self.valid_kernels if indeg[v] == 0]
        out = []
        while ready:
            v = ready.pop()
            out.append(v)
            for s in v.successors:
                indeg[s] -= 1
                if indeg[s] == 0:
                    ready.append(s)
        assert len(out) == len(self.valid_kernels), "dependent graph has a cycle"
        return out

    def _list_schedule(self) -> None:
        fob = self.fob
        prio = self._rank_to_sink()
        free = {k: 0.0 for k in self.stream_kernel_lists}
        ready_at = {v: 0.0 for v in self.valid_kernels}
        left = {v: len(v.precursors) for v in self.valid_kernels}
        pq: list = []

        def est(v):
            return max([ready_at[v]] + [free[k] for k in self._streams_of(v)])

        for v in self.valid_kernels:
            if left[v] == 0:
                heapq.heappush(pq, (est(v), -prio[v], v.id, v))
        done = 0
        while pq:
            t, _, _, v = heapq.heappop(pq)
            cur = est(v)
            if cur > t + 1e-15:        # a stream got busier since the push: re-queue
                heapq.heappush(pq, (cur, -prio[v], v.id, v))
                continue
            v._start_time = cur
            end = cur + v.time[fob]
            for k in self._streams_of(v):
                free[k] = end
            done += 1
            for s in v.successors:
                ready_at[s] = max(ready_at[s], end)
                left[s] -= 1
                if left[s] == 0:
                    heapq.heappush(pq, (est(s), -prio[s], s.id, s))
        assert done == len(self.valid_kernels)

    generate_execution_plan_through_start_time = _list_schedule

    # ------------------------------- ILP --------------------------------------------------------
    def _solve_ilp(self, upper_bound: float) -> bool:
        fob = self.fob
        ks = self.valid_kernels
        if not ks:
            return True
        big_m = max(upper_bound, 1e-12)
        scale = 1.0 / big_m          # work in units of the incumbent makespan for conditioning
        m = Model("kernel_schedule")
        start = {v: m.add_var(f"s_{v.id}", 0.0, 1.0) for v in ks}
        T = m.add_var("end_time", 0.0, 1.0)
        dur = {v: v.time[fob] * scale for v in ks}
        n_bin = 0
        for lst in self.stream_kernel_lists.values():
            for a in range(len(lst)):
                for b in range(a + 1, len(lst)):
                    u, v = lst[a], lst[b]
                    if self._ordered(u, v) or self._ordered(v, u):
                        continue     # already ordered by the graph
                    o = m.add_binary(f"o_{u.id}_{v.id}")
                    n_bin += 1
                    # o = 0: u before v ; o = 1: v before u
                    m.add_constr({start[u]: 1.0, start[v]: -1.0, o: -1.0}, "<=", -dur[u])
                    m.add_constr({start[v]: 1.0, start[u]: -1.0, o: 1.0}, "<=", 1.0 - dur[v])
        for u in ks:
            for v in u.successors:
                m.add_constr({start[v]: 1.0, start[u]: -1.0}, ">=", dur[u])
            m.add_constr({T: 1.0, start[u]: -1.0}, ">=", dur[u])
        cp = self.d_graph.critical_path() * scale
        m.add_constr({T: 1.0}, ">=", min(cp, 1.0))
        m.minimize({T: 1.0})
        if n_bin > 6000:             # too many disjunctions for a useful solve: keep the incumbent
            return False
        sol = m.solve(time_limit=self.time_limit, backend=self.backend, mip_rel_gap=1e-3)
        if not sol.ok or sol.value(T) > 1.0 + 1e-9:
            return False
        self.mylp_obj = sol.value(T) * big_m
        for v in ks:
            v._start_time = sol.value(start[v]) * big_m
        return True

    def _ordered(self, u, v) -> bool:
        """True if the graph already forces u before v (direct edge; cheap test)."""
        return v in u.successors

    # ------------------------------- manual (FULL, Y x X grid) ----------------------------------
    def _manual_order(self) -> bool:
        """Ring-shifted compute order and inputs-before-outputs message order
        (reference: search_algo/execute_plan.py:510-626). Returns False if the fixed orders
        contradict the graph (then the caller falls back to list scheduling)."""
        X, Y, cp = self.X, self.Y, self.hierarchy_sp
        pos = {}
        for g in range(cp):
            base = g // X * X
            order = []
            for off0 in range(Y):
                for off1 in range(X):
                    order.append((base + (g % X + off1) % X, (g % X + (g // X + off0) % Y * X) % cp))
            pos[g] = {rc: i for i, rc in enumerate(order)}
        for v in self.valid_kernels:
            if v.type == "comp":
                b, h, r, c, g = v.key
                per = self.split_degrees[0] // cp
                rr = (r if not isinstance(r, tuple) else r[0]) // per
                cc = (c if not isinstance(c, tuple) else c[0]) // per
                v._start_time = float(pos[g].get((rr, cc), len(pos[g])))
            else:
                # inputs first (rows then columns), outputs last
                v._start_time = (0.0 if v.key[5] == "i" else 1e6) + (0.0 if v.key[6] == "r" else 0.5) \
                    + 1e-3 * ((v.key[4] - v.key[3]) % cp)
        for lst in self.stream_kernel_lists.values():
            lst.sort(key=lambda x: x._start_time)
        try:
            self._relax(check_only=True)
        except AssertionError:
            return False
        return True

    # ------------------------------- finalisation -----------------------------------------------
    def _finalize(self) -> None:
        for lst in self.stream_kernel_lists.values():
            lst.sort(key=lambda x: (x._start_time, x.id))
        self.fine_tune_kernel_time()
        self.stream_exclusive = self.sanity_check_stream_exclusive()
        self.gpu_kernel_lists = []
        for g in range(self.hierarchy_sp):
            seen, merged = set(), []
            for s in range(3):
                for k in self.stream_kernel_lists[(g, s)]:
                    if id(k) not in seen:
                        seen.add(id(k))
                        merged.append(k)
            merged.sort(key=lambda x: (x._start_time, isinstance(x, Comp_Kernel), x.id))
            self.gpu_kernel_lists.append(merged)

    def _relax(self, check_only: bool = False) -> None:
        """Earliest start times under graph edges + the current per-stream orders."""
        fob = self.fob
        extra_succ = {v: [] for v in self.valid_kernels}
        extra_pre = {v: 0 for v in self.valid_kernels}
        for lst in self.stream_kernel_lists.values():
            for a, b in zip(lst[:-1], lst[1:]):
                if b not in a.successors:
                    extra_succ[a].append(b)
                    extra_pre[b] += 1
        left = {v: len(v.precursors) + extra_pre[v] for v in self.valid_kernels}
        st = {v: 0.0 for v in self.valid_kernels}
        ready = [v for v in self.valid_kernels if left[v] == 0]
        seen = 0
        while ready:
            v = ready.pop()
            seen += 1
            end = st[v] + v.time[fob]
            for u in list(v.successors) + extra_succ[v]:
                st[u] = max(st[u], end)
                left[u] -= 1
                if left[u] == 0:
                    ready.append(u)
        assert seen == len(self.valid_kernels), "stream orders contradict the dependency graph"
        if not check_only:
            for v in self.valid_kernels:
                v._start_time = st[v]
            self.end_time = max((st[v] + v.time[fob] for v in self.valid_kernels), default=0.0)

    def fine_tune_kernel_time(self) -> None:
        self._relax()

    def sanity_check_stream_exclusive(self) -> bool:
        fob = self.fob
        for lst in self.stream_kernel_lists.values():
            for a, b in zip(lst[:-1], lst[1:]):
                if a._start_time + a.time[fob] - b._start_time > 1e-3 * max(a.time[fob], 1e-12):
                    return False
        return True

    # ------------------------------- pickling ----------------------------------------------------
    def __getstate__(self) -> dict:
        """Pickles name only classes the reference has too (``search_algo.*`` paths), so that it can
        load plans written here: the allocation record attached by ``make_plan`` goes in as a plain
        dict and comes back as an ``Allocation`` when this class loads it."""
        state = dict(self.__dict__)
        al = state.get("allocation")
        if al is not None and not isinstance(al, dict):
            state["allocation"] = {"Par_D": int(al.Par_D), "cmap": np.asarray(al.cmap), "table": np.asarray(al.table),
                                   "comm_volume": float(al.comm_volume), "comp_max": float(al.comp_max),
                                   "status": str(al.status)}
        return state

    def __setstate__(self, state: dict) -> None:
        self.__dict__.update(state)
        al = state.get("allocation")
        if isinstance(al, dict):
            from .allocate import Allocation
            self.allocation = Allocation(**al)

    # ------------------------------- verification ------------------------------------------------
    def verify(self) -> list:
        """Static checks of a finished plan; returns a list of problems (empty = fine)."""
        problems = []
        fob = self.fob
        if not self.d_graph.is_acyclic():
            problems.append("dependent graph has a cycle")
        if not self.sanity_check_stream_exclusive():
            problems.append("two kernels overlap on one stream")
        for v in self.valid_kernels:
            for u in v.precursors:
                if u._start_time + u.time[fob] > v._start_time + 1e-9 * max(1.0, self.end_time):
                    problems.append(f"{v.key} starts before its precursor {u.key} ends")
        # every scheduled tile is computed exactly once
        tab = self.d_graph.schedule.schedule_table
        covered = {}
        for v in self.valid_kernels:
            if v.type == "comp":
                for r in v.rows:
                    for c in v.cols:
                        covered[(v.key[0], v.key[1], r, c)] = covered.get((v.key[0], v.key[1], r, c), 0) + 1
        for idx in zip(*np.nonzero(tab >= 0)):
            if covered.get(tuple(int(i) for i in idx), 0) != 1:
                problems.append(f"tile {idx} computed {covered.get(tuple(int(i) for i in idx), 0)} times")
        # every message sits once on a send stream and once on a receive stream
        for v in self.valid_kernels:
            if v.type == "comm":
                ns = sum(v in self.stream_kernel_lists[(v.key[3], STREAM_SEND)] for _ in [0])
                nr = sum(v in self.stream_kernel_lists[(v.key[4], STREAM_RECV)] for _ in [0])
                if ns != 1 or nr != 1:
                    problems.append(f"message {v.key} not on exactly one send and one receive stream")
        # every foreign input of a compute kernel has a producer edge
        smap = self.d_graph.schedule.S_map
        for v in self.valid_kernels:
            if v.type != "comp":
                continue
            b, h, g = v.key[0], v.key[1], v.key[4]
            need = [("r", r) for r in v.rows if int(smap[b, r]) != g] + \
                   [("c", c) for c in v.cols if int(smap[b, c]) != g]
            for rc, x in need:
                if not any(p.type == "comm" and p.key[5] == "i" and p.key[6] == rc and p.key[2] == x
                           and p.key[4] == g for p in v.precursors):
                    problems.append(f"{v.key} lacks the input message for {rc}{x}")
        # launch order per rank respects start times
        for g, lst in enumerate(self.gpu_kernel_lists):
            for a, b in zip(lst[:-1], lst[1:]):
                if a._start_time > b._start_time + 1e-12:
                    problems.append(f"rank {g} launch list not sorted by start time")
                    break
        return problems

    # ------------------------------- plain-data form -------------------------------------------
    def to_plain(self) -> dict:
        """The same plan as lists and dicts of plain values (the JSON side-car of the pickle)."""
        fob = self.fob
        kern = []
        for v in self.valid_kernels:
            kern.append({
                "id": int(v.id), "key": _plain(v.key), "type": v.type,
                "time": [float(v.time[0]), float(v.time[1])], "start": float(v._start_time),
                "precursors": sorted(int(u.id) for u in v.precursors),
                "units": [float(x) for x in v.units] if v.type == "comm" else None,
            })
        sch = self.d_graph.schedule
        return {
            "format": "ultraattn-plan/1", "fob": fob, "plan_type": self.plan_type,
            "end_time": float(self.end_time), "stream_num": 3,
            "da_config": {"SP": _plain(self.da_config.SP), "S": _plain(self.da_config.S),
                          "Nh": _plain(self.da_config.Nh), "bs": int(self.da_config.bs), "D": int(self.da_config.D),
                          "hierarchy": int(self.da_config.hierarchy),
                          "bsa_config": str(self.da_config.bsa_config)},
            "split_degrees": _plain(sch.split_degrees),
            "S_map": np.asarray(sch.S_map).tolist(),
            "schedule_table": np.asarray(sch.schedule_table).tolist(),
            "kernels": kern,
            "gpu_kernel_lists": [[int(k.id) for k in lst] for lst in self.gpu_kernel_lists],
        }

    def to_json(self, path) -> None:
        with open(path, "w") as f:
            json.dump(self.to_plain(), f)

    @classmethod
    def from_plain(cls, d: dict) -> "Execution_Plan":
        """Rebuild an executable plan from its plain-data form (the JSON side-car), without
        unpickling anything: kernels with their keys, times, start times and precursor /
        successor links, the per-rank launch lists, the per-stream lists, and the problem
        description the executors read (shape, pattern, partition, ownership)."""
        import re
        from ..patterns.blocks import BSA_Config, BSA_Repr
        from .cost import Dist_Attn_Config
        assert d.get("format") == "ultraattn-plan/1", f"unknown plan format {d.get('format')!r}"
        dc = d["da_config"]
        m = re.match(r"CP=\((\d+), (\d+)\)_repr=(.*)$", dc["bsa_config"])
        bsa = BSA_Config(None, None, {"bsa_repr": BSA_Repr.from_string(m.group(3)),
                                      "CP": (int(m.group(1)), int(m.group(2)))})
        da = Dist_Attn_Config.from_bsa_config(bsa, {"S": tuple(dc["S"]), "Nh": tuple(dc["Nh"]), "bs": dc["bs"],
                                                    "D": dc["D"]}, dc["hierarchy"])
        plan = cls(None, d["fob"], d["plan_type"])
        kernels = {}
        for k in d["kernels"]:
            key = tuple(tuple(x) if isinstance(x, list) else x for x in k["key"])
            if k["type"] == "comp":
                v = Comp_Kernel(key, None, None, 0, time=np.array(k["time"]))
            else:
                v = Comm_Kernel(key, None, None, np.array(k["units"] or [0.0, 0.0]), 0, seqlen_variable_graph=True)
                v.time = np.array(k["time"], dtype=float)
                del v.is_empty_kernel               # emptiness follows from the stored times again
            v.id, v._start_time = k["id"], k["start"]
            kernels[k["id"]] = v
        for k in d["kernels"]:
            v = kernels[k["id"]]
            for pid in k["precursors"]:
                v.precursors.add(kernels[pid])
                kernels[pid].successors.add(v)
        plan.valid_kernels = [kernels[k["id"]] for k in d["kernels"]]
        plan.gpu_kernel_lists = [[kernels[i] for i in lst] for lst in d["gpu_kernel_lists"]]
        plan.stream_kernel_lists = {}
        for v in plan.valid_kernels:
            for slot in cls._streams_of(v):
                plan.stream_kernel_lists.setdefault(slot, []).append(v)
        for lst in plan.stream_kernel_lists.values():
            lst.sort(key=lambda v: v._start_time)
        plan.end_time = d["end_time"]

        class _Schedule:            # what executors and tools read from ``plan.d_graph.schedule``
            pass
        sch = _Schedule()
        sch.da_config, sch.m_config = da, None
        sch.split_degrees = tuple(d["split_degrees"])
        sch.S_map, sch.schedule_table = np.asarray(d["S_map"]), np.asarray(d["schedule_table"])

        from .graph import Dependent_Graph

        class _Graph:               # the graph as far as executors, the simulator and verify() use it
            def valid_kernels(self):
                return list(self.kernel_dict.values())
            is_acyclic = Dependent_Graph.is_acyclic
        g = _Graph()
        g.schedule, g.fob, g.da_config, g.m_config = sch, d["fob"], da, None
        g.split_degrees, g.hierarchy, g.hierarchy_sp, g.tot_sp = sch.split_degrees, da.hierarchy, da.hierarchy_sp, da.tot_sp
        g.kernel_dict = {v.key: v for v in plan.valid_kernels}
        g.seqlen_variable_graph = False
        plan.d_graph = g
        return plan

    @classmethod
    def from_json(cls, path) -> "Execution_Plan":
        with open(path) as f:
            return cls.from_plain(json.load(f))

    def print_lp_result(self) -> None:
        for (g, s), lst in self.stream_kernel_lists.items():
            print(f"rank {g} stream {s}: " + " ".join(
                f"{k.key}@{k._start_time:.3e}+{k.time[self.fob]:.3e}" for k in lst))


def _plain(key):
    """A kernel key as plain JSON values (keys built by the reference carry NumPy integers)."""
    def one(x):
        if isinstance(x, (tuple, list)):
            return [one(y) for y in x]
        if isinstance(x, np.generic):
            return x.item()
        return x
    return [one(x) for x in key]


def create_one_node_exe_plan(fob: int, comp_time: float = 1.0) -> Execution_Plan:
    """Trivial inter-level plan for a single node: one compute kernel, no messages (reference:
    search_algo/execute_plan.py:138-156)."""
    plan = Execution_Plan(None, fob, "manual")
    k = Comp_Kernel((0, 0, 0, 0, 0), None, None, 0, time=np.array([comp_time, comp_time]))
    k.id = 0
    plan.valid_kernels = [k]
    plan.stream_kernel_lists = {(0, 0): [k], (0, 1): [], (0, 2): []}
    plan.gpu_kernel_lists = [[k]]
    plan.end_time = comp_time
    plan.one_node = True
    return plan


# the reference reaches it through the class (search_algo/execute_plan.py:138)
Execution_Plan.create_one_node_exe_plan = staticmethod(create_one_node_exe_plan)


class Fused_Execution_Plan:
    """FULL attention with kernel tiling on a Y x X rank grid: rank g computes the X query chunks of
    its row group against the Y key chunks ``g % X, g % X + X, ...`` as ONE kernel; inputs arrive by
    all-gather along the row group (Q side, X ranks) and the column group (K/V side, Y ranks),
    outputs leave by reduction along the same groups (reference: search_algo/execute_plan.py:22-108).
    """

    def __init__(self, Y: int, X: int, time=None, fob: int = 0, m_config=None, causal: bool = False):
        self.Y, self.X = Y, X
        self.fob = fob
        self.causal = causal
        self.stream_num = 3
        self.m_config = m_config
        self.end_time = time
        self.da_config = None
        self.plan_type = "fused"

    @property
    def cp(self) -> int:
        return self.X * self.Y

    def row_group(self, g: int) -> list:
        return list(range(g // self.X * self.X, g // self.X * self.X + self.X))

    def col_group(self, g: int) -> list:
        return list(range(g % self.X, self.cp, self.X))

    def materialize(self, da_config, m_config=None) -> float:
        """Estimated time for a concrete shape (compute of the X x Y rectangle + exposed gathers)."""
        from .cost import analytic_tile_time
        self.da_config = da_config
        m = m_config or self.m_config
        sq = da_config.S[0] // self.cp * self.X
        skv = da_config.S[1] // self.cp * self.Y
        comp = analytic_tile_time(sq, skv, da_config.Nh[0], da_config.bs, da_config.D, False)[self.fob]
        unit = da_config.S[0] // self.cp * da_config.bs * da_config.Nh[0] * da_config.D * 2
        comm = 0.0
        if m is not None:
            cm = m.comm_profile_maps[1]
            vol = (self.X - 1) * (1 if self.fob == 0 else 2) + (self.Y - 1) * 2
            comm = cm.get_comm_time_from_map_key((unit * vol,))
        self.end_time = max(comp, comm) + 0.1 * min(comp, comm)
        return self.end_time

    def get_plan_name(self) -> str:
        return f"fused_Y={self.Y}_X={self.X}_fob={self.fob}"

    def to_plain(self) -> dict:
        return {"format": "ultraattn-fused-plan/1", "Y": self.Y, "X": self.X, "fob": self.fob,
                "causal": bool(self.causal), "end_time": None if self.end_time is None else float(self.end_time)}

    @classmethod
    def from_plain(cls, d: dict, m_config=None) -> "Fused_Execution_Plan":
        assert d.get("format") == "ultraattn-fused-plan/1", f"unknown plan format {d.get('format')!r}"
        return cls(d["Y"], d["X"], d.get("end_time"), d["fob"], m_config, d.get("causal", False))
