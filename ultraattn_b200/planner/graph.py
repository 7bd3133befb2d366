"""The parallel dependent kernel graph: compute tiles and the messages they need.

From a :class:`~ultraattn_b200.planner.cost.Dist_Attn_Schedule` this builds one compute kernel per
scheduled tile and, for every row (Q-side data) or column (K/V-side data) that a foreign rank
touches, one input message owner -> rank and one output message rank -> owner — star broadcast /
star reduce, de-duplicated per (row-or-column, peer). Edges are ``input message -> compute ->
output message``. Messages whose payload is empty for the pass at hand (e.g. the forward's
output-column message: there is no dK/dV) are "empty kernels" and never get edges.

Kernel keys (kept identical to the reference, search_algo/dependent_graph.py:15-92, 209-334):
  compute  ``(b, h, r, c, rank)`` or fused ``(b, h, (r...), (c...), rank)``
  message  ``(b, h, row_or_col_id, src, dst, 'i'|'o', 'r'|'c')``
"""
from __future__ import annotations

import copy
from typing import Optional

import numpy as np

from ..patterns.blocks import BSA_Config, CAUSAL, FULL
from .cost import (Dist_Attn_Config, Dist_Attn_Schedule, Machine_Config, analytic_tile_time,
                   convert_shape_config_to_str)


class Cuda_Kernel:
    def __init__(self, key: tuple, type: str):
        self.key = key
        self.type = type
        self.precursors: set = set()
        self.successors: set = set()
        self.time = np.zeros(2)
        self.id = -1
        self._start_time = 0.0

    # graph edits ----------------------------------------------------------------------------
    def add_precursor(self, k): self.precursors.add(k)
    def add_successor(self, k): self.successors.add(k)
    def remove_precursor(self, k): self.precursors.discard(k)
    def remove_successor(self, k): self.successors.discard(k)

    def is_empty(self, fob: int) -> bool:
        if hasattr(self, "is_empty_kernel"):
            return bool(self.is_empty_kernel[fob])
        return self.time[fob] <= 0

    def add_edge(self, v: "Cuda_Kernel", fob: int) -> None:
        if self.is_empty(fob) or v.is_empty(fob):
            return
        self.add_successor(v)
        v.add_precursor(self)

    def remove_edge(self, v: "Cuda_Kernel", fob: int) -> None:
        if self.is_empty(fob) or v.is_empty(fob):
            return
        self.remove_successor(v)
        v.remove_precursor(self)

    @property
    def start_time(self) -> float:
        return self._start_time

    @start_time.setter
    def start_time(self, v: float) -> None:
        self._start_time = float(v)

    # kernels are identified by key; hashing by identity keeps sets cheap
    def __repr__(self) -> str:
        return f"{self.type}{self.key}"

    def __lt__(self, other) -> bool:       # tie-break inside priority queues
        return str(self.key) < str(other.key)


class Comp_Kernel(Cuda_Kernel):
    def __init__(self, key: tuple, m_config: Optional[Machine_Config], comp_map_key, hierarchy: int,
                 time: Optional[np.ndarray] = None, seqlen_variable_graph: bool = False):
        super().__init__(key, "comp")
        self.hierarchy = hierarchy
        self.comp_map_key = comp_map_key
        if seqlen_variable_graph:
            self.is_empty_kernel = np.array([False, False])
            self.time = np.array([1e-3, 1e-2])       # placeholder durations of a shape-free graph
        elif time is not None:
            self.time = np.asarray(time, dtype=float)
        else:
            self.time = np.asarray(
                m_config.comp_profile_maps[hierarchy].get_comp_time_from_map_key(comp_map_key), dtype=float)

    @property
    def rank(self) -> int:
        return self.key[4]

    @property
    def rows(self) -> tuple:
        r = self.key[2]
        return r if isinstance(r, tuple) else (r,)

    @property
    def cols(self) -> tuple:
        c = self.key[3]
        return c if isinstance(c, tuple) else (c,)


class Comm_Kernel(Cuda_Kernel):
    def __init__(self, key: tuple, m_config: Optional[Machine_Config], comm_raw_map_key,
                 units: np.ndarray, hierarchy: int, seqlen_variable_graph: bool = False):
        super().__init__(key, "comm")
        units = np.asarray(units, dtype=float)
        assert units.shape == (2,)
        self.units = units
        self.hierarchy = hierarchy
        self.comm_raw_map_key = comm_raw_map_key
        if seqlen_variable_graph:
            self.is_empty_kernel = units == 0
            self.time = np.array([1e-3, 1e-2])
        else:
            cm = m_config.comm_profile_maps[hierarchy]
            self.time = np.array([cm.get_comm_time_from_map_key((comm_raw_map_key[0] * u,)) for u in units])

    @property
    def src(self) -> int:
        return self.key[3]

    @property
    def dst(self) -> int:
        return self.key[4]

    @property
    def io(self) -> str:
        return self.key[5]

    @property
    def rc(self) -> str:
        return self.key[6]

    def nbytes(self, fob: int) -> float:
        return 0.0 if self.comm_raw_map_key is None else self.comm_raw_map_key[0] * self.units[fob]


class Dependent_Graph:
    def __init__(self, schedule: Dist_Attn_Schedule, fob: int, kernel_dict: Optional[dict] = None,
                 is_inter_bsa: bool = False, bsa_comp_key_suffixes=None,
                 seqlen_variable_graph: bool = False):
        self.schedule = schedule
        self.fob = fob
        self.bsa_comp_key_suffixes = bsa_comp_key_suffixes
        self.seqlen_variable_graph = seqlen_variable_graph
        self.kernel_dict: dict = {}
        if kernel_dict:
            self.kernel_dict = kernel_dict
        else:
            self.create_raw_graph()

    # deducible attributes ---------------------------------------------------------------------
    @property
    def da_config(self) -> Dist_Attn_Config: return self.schedule.da_config
    @property
    def m_config(self) -> Machine_Config: return self.schedule.m_config
    @property
    def split_degrees(self): return self.schedule.split_degrees
    @property
    def tot_sp(self) -> int: return self.schedule.tot_sp
    @property
    def hierarchy(self) -> int: return self.schedule.da_config.hierarchy
    @property
    def hierarchy_sp(self) -> int: return self.schedule.da_config.hierarchy_sp

    def materialize(self, da_config: Dist_Attn_Config) -> None:
        """Turn a shape-free graph into a timed one for a concrete shape."""
        self.schedule.da_config = da_config
        self.seqlen_variable_graph = False
        self.create_raw_graph()

    # construction -----------------------------------------------------------------------------
    def _tile_type(self, r: int, c: int) -> int:
        """Block type of tile (r, c) at the schedule's granularity (2 causal, 1 full, 0 empty,
        -1 mixed)."""
        sub = self.da_config.bsa_config.bsa_repr.create_sub_bsa_repr(self.split_degrees[0:2], [[r], [c]])
        t = sub.table
        return int(t[0, 0]) if t.shape == (1, 1) else -1

    def _comp_time(self, r: int, c: int):
        sch, da = self.schedule, self.da_config
        if self.hierarchy == 1:
            cmap_ = sch.m_config.comp_profile_maps[1]
            tt = self._tile_type(r, c)
            if tt in (FULL, CAUSAL):
                key = cmap_.get_comp_map_key(da, [1, 1], sch.split_degrees, causal=(tt == CAUSAL))
                return key, None
            sub = da.bsa_config.bsa_repr.create_sub_bsa_repr(sch.split_degrees[0:2], [[r], [c]])
            key = cmap_.get_comp_map_key(da, [1, 1], sch.split_degrees, causal=False)
            return key, np.asarray(cmap_.get_comp_time_from_map_key(key)) * sub.sparsity
        # inter level: cost of a node-level tile = best measured intra plan for its sub-pattern
        intra_cp = (da.SP[1], 1)
        sub = da.bsa_config.bsa_repr.create_sub_bsa_repr(sch.split_degrees[0:2], [[r], [c]])
        unit_shape = dict(da.shape_config)
        unit_shape["S"] = (da.S[0] // sch.split_degrees[0], da.S[1] // sch.split_degrees[1])
        sub_cfg = BSA_Config(None, None, {"bsa_repr": sub, "CP": intra_cp})
        prefix = (f"fob={self.fob}_CP={intra_cp}_shape_config={{{convert_shape_config_to_str(unit_shape)}}}"
                  f"_bsa_config={{{sub_cfg}}}")
        inter_map = sch.m_config.comp_profile_maps[0]
        best_key, best_t = None, None
        for suf in (self.bsa_comp_key_suffixes or [""]):
            k = prefix + suf
            if k in inter_map.profile_map:
                t = inter_map.get_comp_time_from_map_key(k)
                if best_t is None or t[self.fob] < best_t[self.fob]:
                    best_key, best_t = k, t
        if best_t is None:      # nothing measured yet: analytic estimate of a perfectly split tile
            t = analytic_tile_time(unit_shape["S"][0], unit_shape["S"][1], da.Nh[0], da.bs, da.D, False)
            best_key, best_t = prefix, t * sub.sparsity / intra_cp[0]
        return best_key, best_t

    def create_raw_graph(self) -> None:
        self.kernel_dict = {}
        sch, fob, hier = self.schedule, self.fob, self.hierarchy
        sd = sch.split_degrees
        assert sd[0] == sd[1], "Sq and Skv must be split alike"
        svg = self.seqlen_variable_graph
        comm_key = None if svg else sch.m_config.comm_profile_maps[hier].get_comm_map_key(
            sch.da_config, [1, 1], sd)
        tab = sch.schedule_table
        for b in range(sd[2]):
            for h in range(sd[3]):
                # compute kernels
                for r in range(sd[0]):
                    for c in range(sd[1]):
                        g = int(tab[b, h, r, c])
                        if g < 0:
                            continue
                        key = (b, h, r, c, g)
                        if svg:
                            self.kernel_dict[key] = Comp_Kernel(key, None, None, hier, seqlen_variable_graph=True)
                        else:
                            mk, t = self._comp_time(r, c)
                            self.kernel_dict[key] = Comp_Kernel(key, sch.m_config, mk, hier, time=t)
                # messages: rows then columns, one per (row/col, peer)
                for kind, units_in, units_out in (("r", sch.u_inp_row, sch.u_out_row),
                                                  ("c", sch.u_inp_col, sch.u_out_col)):
                    for x in range(sd[0]):
                        owner = int(sch.S_map[b, x])
                        line = tab[b, h, x, :] if kind == "r" else tab[b, h, :, x]
                        for peer in sorted({int(g) for g in line if g >= 0 and g != owner}):
                            ki = (b, h, x, owner, peer, "i", kind)
                            ko = (b, h, x, peer, owner, "o", kind)
                            self.kernel_dict[ki] = Comm_Kernel(ki, sch.m_config, comm_key, units_in, hier, svg)
                            self.kernel_dict[ko] = Comm_Kernel(ko, sch.m_config, comm_key, units_out, hier, svg)
                # edges
                for r in range(sd[0]):
                    for c in range(sd[1]):
                        g = int(tab[b, h, r, c])
                        if g < 0:
                            continue
                        comp = self.kernel_dict[(b, h, r, c, g)]
                        ro = int(sch.S_map[b, r])
                        if g != ro:
                            self.kernel_dict[(b, h, r, ro, g, "i", "r")].add_edge(comp, fob)
                            comp.add_edge(self.kernel_dict[(b, h, r, g, ro, "o", "r")], fob)
                        co = int(sch.S_map[b, c])
                        if g != co:
                            self.kernel_dict[(b, h, c, co, g, "i", "c")].add_edge(comp, fob)
                            comp.add_edge(self.kernel_dict[(b, h, c, g, co, "o", "c")], fob)

    # queries ----------------------------------------------------------------------------------
    def valid_kernels(self) -> list:
        return [k for k in self.kernel_dict.values() if not k.is_empty(self.fob)]

    def comp_kernels(self) -> list:
        return [k for k in self.kernel_dict.values() if k.type == "comp"]

    def is_acyclic(self) -> bool:
        ks = self.valid_kernels()
        indeg = {k: len(k.precursors) for k in ks}
        ready = [k for k in ks if indeg[k] == 0]
        seen = 0
        while ready:
            k = ready.pop()
            seen += 1
            for s in k.successors:
                indeg[s] -= 1
                if indeg[s] == 0:
                    ready.append(s)
        return seen == len(ks)

    def critical_path(self) -> float:
        memo: dict = {}

        def longest(k):
            if k not in memo:
                memo[k] = k.time[self.fob] + max((longest(s) for s in k.successors), default=0.0)
            return memo[k]
        return max((longest(k) for k in self.valid_kernels() if not k.precursors), default=0.0)

    def __deepcopy__(self, memo):
        # the schedule (problem + machine description) is shared, kernels are copied
        new = Dependent_Graph.__new__(Dependent_Graph)
        memo[id(self)] = new
        new.schedule = self.schedule
        new.fob = self.fob
        new.bsa_comp_key_suffixes = copy.copy(self.bsa_comp_key_suffixes)
        new.seqlen_variable_graph = self.seqlen_variable_graph
        new.kernel_dict = copy.deepcopy(self.kernel_dict, memo)
        return new
