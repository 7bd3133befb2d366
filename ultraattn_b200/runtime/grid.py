"""Kernel-tile execution of dense attention on a Y x X rank grid with collectives (the NCCL form).

Reference: orchestrated_attn/orchestrated_attn_impl.py:222-298 (forward) and :433-552 (backward),
driven by ``Fused_Execution_Plan`` (search_algo/execute_plan.py:22-108). Rank g works on the X
query chunks of its row group (ranks sharing ``g // X``) against the Y key/value chunks of its
column group (ranks sharing ``g % X``) as ONE kernel launch:

  forward   all-gather Q along the row group and K | V along the column group -> one attention
            launch over X x Y chunks -> every member of a row group now holds a partial (O, lse)
            of each of the X rows -> exchange inside the row group and merge.
  backward  all-gather Q | dO | D | lse (rows) and K | V (columns) -> one backward launch ->
            reduce-scatter(SUM) dQ along the row group and dK | dV along the column group.

Differences from the reference, on purpose. (1) Its forward reduce-scatters O with SUM, which is
not the softmax merge; here the partial outputs are exchanged with an all-to-all and merged with
the log-sum-exp rule, so the result is exact. (2) It re-packs the gathered ``[Y, 2, bs, S, Nh, D]``
bundle with transposes and ``torch.cat`` (and supports only one head in the backward because of
that); the kernels here take a list of sources, so each gathered chunk is used where it landed.
(3) Causal attention is supported: chunk pairs above the diagonal are left out, diagonal pairs are
causal.

This is the baseline form of the kernel-tile idea: the product form is the fused runtime given a
grid allocation (``planner.allocate.grid_table``), where the gathers and reductions happen inside
the kernels.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import attention as A
from ..ops import elementwise as E
from ..parallel.comm import A2AComm
from ..parallel.communicator import CommRegistry, IntraComm_fused
from .orchestrated import (Input_Col_Bwd, Input_Col_Fwd, Input_Row_Bwd, Input_Row_Fwd, Output_Col_Bwd,
                           Output_Row_Bwd, Output_Row_Fwd)


class GridExecutor:
    """Collective over the default group at construction (row / column communicators are made
    with ``dist.new_group``)."""

    def __init__(self, Y: int, X: int, group=None, device: Optional[torch.device] = None,
                 causal: bool = False, registry: Optional[CommRegistry] = None):
        world = dist.get_world_size(group)
        assert X * Y == world, f"a {Y} x {X} grid needs {X * Y} ranks, the group has {world}"
        self.Y, self.X, self.causal = Y, X, causal
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        ranks = [dist.get_global_rank(group, r) if group is not None else r for r in range(world)]
        self.g = dist.get_rank(group)
        self.registry = (registry if registry is not None else CommRegistry()).for_grid(ranks, X)
        self.comm = IntraComm_fused(self.registry, ranks, X, rank=ranks[self.g])
        self.x_id, self.y_id = self.g % X, self.g // X
        # chunk ids = positions in the group: rows of my row group, columns of my column group
        self.row_chunks = list(range(self.g // X * X, self.g // X * X + X))
        self.col_chunks = list(range(self.g % X, world, X))
        row_key = self.comm.groups["r"]
        self.row_a2a = A2AComm(self.registry[row_key].group) if len(row_key) > 1 else None

    @classmethod
    def from_plan(cls, plan, group=None, device=None, registry=None) -> "GridExecutor":
        """From a ``Fused_Execution_Plan``."""
        return cls(plan.Y, plan.X, group, device, getattr(plan, "causal", False), registry)

    # ---- helpers -------------------------------------------------------------------------------
    def _visible(self, r: int, c: int):
        """None: chunk pair masked out; else whether it is a diagonal (causal) pair."""
        if not self.causal:
            return False
        return None if c > r else (c == r)

    def _gather(self, rc: str, carrier_cls, shapes, fill, n_slots: int):
        """All-gather one carrier along the row ('r') or column ('c') group; returns the carriers
        of all members, each a view of the gathered buffer."""
        mine = carrier_cls.from_shapes(*shapes, device=self.device)
        fill(mine)
        n = mine.nbytes()
        gathered = torch.empty(n_slots * n, dtype=torch.uint8, device=self.device)
        self.comm.all_gather(rc, gathered, mine.data)
        return [carrier_cls.from_shapes(*shapes, buf=gathered[s * n:(s + 1) * n]) for s in range(n_slots)]

    # ---- forward -------------------------------------------------------------------------------
    def forward(self, q, k, v, softmax_scale=None):
        B, S, H, D = q.shape
        Hk = k.shape[2]
        shapes = (B, S, S, H, Hk, D, q.dtype)
        rows_in = self._gather("r", Input_Row_Fwd, shapes, lambda c: c.Q.copy_(q), self.X)
        cols_in = self._gather("c", Input_Col_Fwd, shapes, lambda c: (c.K.copy_(k), c.V.copy_(v)), self.Y)
        probe = Output_Row_Fwd.from_shapes(*shapes, device="meta")
        n_o = probe.nbytes()
        part_buf = torch.zeros(self.X * n_o, dtype=torch.uint8, device=self.device)
        parts = [Output_Row_Fwd.from_shapes(*shapes, buf=part_buf[x * n_o:(x + 1) * n_o]) for x in range(self.X)]
        rows = []
        for xi, r in enumerate(self.row_chunks):
            parts[xi].lse.fill_(float("-inf"))
            segs = []
            for yi, c in enumerate(self.col_chunks):
                vis = self._visible(r, c)
                if vis is not None:
                    segs.append(A.Seg(yi, 0, S, vis, 0))
            if segs:
                rows.append(A.Row(xi, 0, S, tuple(segs), xi, 0, False))
        if rows:
            A.attn_fwd([c.Q for c in rows_in], [c.K for c in cols_in], [c.V for c in cols_in],
                       [(p.O, p.lse) for p in parts], A.FwdPlan(rows, self.device), softmax_scale)
        # partial x goes to member x of the row group; what arrives are the X partials of my row
        if self.row_a2a is not None:
            recv = self.row_a2a.all_to_all(part_buf, 0, 0)
            mine = [Output_Row_Fwd.from_shapes(*shapes, buf=recv[x * n_o:(x + 1) * n_o]) for x in range(self.X)]
        else:
            mine = parts
        o = torch.empty_like(q)
        lse = torch.empty(B, H, S, dtype=torch.float32, device=self.device)
        for b in range(B):
            E.lse_merge([(p.O[b], p.lse[b]) for p in mine], (o[b], lse[b]))
        return o, lse

    # ---- backward ------------------------------------------------------------------------------
    def backward(self, d_o, q, k, v, o, lse, softmax_scale=None):
        B, S, H, D = q.shape
        Hk = k.shape[2]
        shapes = (B, S, S, H, Hk, D, q.dtype)
        dvec = torch.empty(B, H, S, dtype=torch.float32, device=self.device)
        for b in range(B):
            E.rowdot(o[b], d_o[b], dvec[b])

        def fill_row(c):
            c.Q.copy_(q)
            c.dO.copy_(d_o)
            c.D.copy_(dvec)
            c.lse.copy_(lse)
        rows_in = self._gather("r", Input_Row_Bwd, shapes, fill_row, self.X)
        cols_in = self._gather("c", Input_Col_Bwd, shapes, lambda c: (c.K.copy_(k), c.V.copy_(v)), self.Y)
        n_r = Output_Row_Bwd.from_shapes(*shapes, device="meta").nbytes()
        n_c = Output_Col_Bwd.from_shapes(*shapes, device="meta").nbytes()
        row_buf = torch.zeros(self.X * n_r, dtype=torch.uint8, device=self.device)
        col_buf = torch.zeros(self.Y * n_c, dtype=torch.uint8, device=self.device)
        out_rows = [Output_Row_Bwd.from_shapes(*shapes, buf=row_buf[x * n_r:(x + 1) * n_r]) for x in range(self.X)]
        out_cols = [Output_Col_Bwd.from_shapes(*shapes, buf=col_buf[y * n_c:(y + 1) * n_c]) for y in range(self.Y)]
        cols = []
        for yi, c in enumerate(self.col_chunks):
            segs = []
            for xi, r in enumerate(self.row_chunks):
                vis = self._visible(r, c)
                if vis is not None:
                    segs.append(A.Seg(xi, 0, S, vis, 0))
            if segs:
                cols.append(A.Col(yi, 0, S, tuple(segs), yi, 0))
        if cols:
            sides = [A.BwdQSide(ci.Q, ci.dO, ci.lse, ci.D, oi.dQ) for ci, oi in zip(rows_in, out_rows)]
            A.attn_bwd(sides, [c.K for c in cols_in], [c.V for c in cols_in],
                       [A.BwdKvOut(oc.dK, oc.dV) for oc in out_cols], A.BwdPlan(cols, self.device), softmax_scale)
        my_row = Output_Row_Bwd.from_shapes(*shapes, device=self.device)
        my_col = Output_Col_Bwd.from_shapes(*shapes, device=self.device)
        f32 = torch.float32
        self.comm.reduce_scatter("r", my_row.data.view(f32), row_buf.view(f32))
        self.comm.reduce_scatter("c", my_col.data.view(f32), col_buf.view(f32))
        return my_row.dQ.to(q.dtype), my_col.dK.to(k.dtype), my_col.dV.to(v.dtype)
