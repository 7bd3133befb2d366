"""User-facing context-parallel attention: plans once, then runs forward / backward per step.

``path="fused"`` uses the peer-memory kernels of :mod:`ultraattn_b200.runtime.fused`;
``path="nccl"`` executes the planner's launch plan with NCCL point-to-point messages
(:mod:`ultraattn_b200.runtime.executor`) and is the baseline the fused path is measured against.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..patterns.blocks import BSA_Config, BSA_Repr
from ..planner.allocate import tile_volumes, naive_allocate_strategy, solve_sparse_from_bsa
from ..planner.pipeline import make_plan


def plan_allocation(pattern: BSA_Repr, cp: int, fob: int = 1, allocation: str = "ilp",
                    time_limit: float = 20.0, cmap=None, select: str = "balance", shape: Optional[dict] = None):
    """(table, cmap) of the tile allocation for ``cp`` ranks. ``cmap``: an ownership map (block ->
    rank), None for contiguous chunks, or ``"search"`` to let the planner pick among contiguous /
    residue-class / zigzag ownership (context remap; every rank then passes the blocks it owns
    under the returned map, in increasing block order).

    ``select``: how the partition granularity (1x, 2x, 4x the rank count) is chosen. ``"balance"``
    (default) takes the coarsest one whose busiest rank is within 3 % of the mean. ``"model"``
    solves all three and keeps the one for which the time model of the fused runtime
    (``planner.cost.fused_step_time`` on the machine profile: tile times at that granularity,
    staging, transfers, the passes around the kernels) predicts the shortest step; it needs
    ``shape = {"seq_len": S, "n_heads": H[, "head_dim", "n_kv_heads", "batch"]}``. A finer
    partition balances better but runs smaller tiles and moves more blocks; the model prices both."""
    cfg = BSA_Config(None, None, {"bsa_repr": pattern, "CP": (cp, 1)})
    if isinstance(cmap, str):
        assert cmap == "search", f"unknown cmap option {cmap!r}"
        from ..planner.allocate import search_context_remap
        import math
        n = cfg.table.shape[0]
        par_d = n if n % (2 * cp) == 0 else math.lcm(n, 2 * cp)      # every candidate map must fit
        res = search_context_remap(cfg, fob=fob, ParD=par_d, time_limit=time_limit)
        return np.asarray(res["allocation"].table), np.asarray(res["cmap"])
    if allocation == "naive":
        al = naive_allocate_strategy(cfg, fob=fob)
        return np.asarray(al.table), np.asarray(al.cmap)
    if allocation == "lightseq":
        # LightSeq's balanced causal schedule (worker / helper ranks) as a fixed table
        from ..planner.dense import get_lightseq_schedule_table
        from ..utils.bsa_helpers import bsa_repr_is_causal
        assert bsa_repr_is_causal(pattern.simplify() if hasattr(pattern, "simplify") else pattern), \
            "the LightSeq schedule is defined for dense causal attention"
        return get_lightseq_schedule_table(cp), np.arange(cp)
    # A pattern with few blocks (dense causal: one) cannot be balanced at one block per rank: the
    # diagonal tiles stay with their owners and the rest is too coarse. Refine the partition (each
    # rank then owns several consecutive blocks, so the caller's shards do not change) until the
    # busiest rank is within 3 % of the mean.
    base = max(cp, cfg.table.shape[0])
    best = None
    assert select in ("balance", "model"), f"unknown select option {select!r}"
    if select == "model":
        assert shape is not None and "seq_len" in shape and "n_heads" in shape, \
            "select='model' needs shape={'seq_len': ..., 'n_heads': ...}"
        from ..planner.cost import fused_step_time
    for mult in ((1, 2, 4) if cmap is None and cp > 1 else (1,)):
        if select == "model" and shape["seq_len"] % (base * mult * 256):
            continue                            # blocks must stay multiples of the kernels' 256-row tiles
        try:
            al = solve_sparse_from_bsa(cfg, fob=fob, ParD=base * mult, time_limit=time_limit, cmap=cmap)
        except RuntimeError:
            if best is None and mult == 1:
                raise
            continue                            # a finer partition the solver could not settle in time
        table = np.asarray(al.table)
        if select == "model":
            t = fused_step_time(table, np.asarray(al.cmap), pattern, shape["seq_len"], shape["n_heads"],
                                shape.get("head_dim", 128), n_kv_heads=shape.get("n_kv_heads"),
                                batch=shape.get("batch", 1))
            score = t["step_s"] if fob else t["fwd_s"]
            if best is None or score < best[0]:
                best = (score, al)
            continue
        vol = tile_volumes(pattern, table.shape[0])
        work = np.array([vol[table == r].sum() for r in range(cp)], dtype=float)
        imbalance = work.max() / max(work.mean(), 1e-9)
        if best is None or imbalance < best[0] - 1e-6:
            best = (imbalance, al)
        if imbalance <= 1.03:
            break
    al = best[1]
    return np.asarray(al.table), np.asarray(al.cmap)


class _CPFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, runtime, softmax_scale):
        o, lse = runtime.forward(q, k, v, softmax_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.runtime = runtime
        ctx.scale = softmax_scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ctx.runtime.backward(d_o.contiguous(), q, k, v, o, lse, ctx.scale)
        return dq, dk, dv, None, None


class ContextParallelAttention:
    """Context-parallel block-sparse attention over the ranks of ``group`` (one node).

    Each rank passes its shard ``[B, S/CP, H, D]`` (the blocks it owns under the plan's ``cmap``,
    in increasing block order; contiguous chunks by default) and receives the matching shard of
    the output / gradients.
    """

    def __init__(self, pattern: BSA_Repr, seq_len: int, n_heads: int, head_dim: int = 128, *,
                 group=None, device: Optional[torch.device] = None, path: str = "fused",
                 n_kv_heads: Optional[int] = None, batch: int = 1, allocation: str = "ilp",
                 plan_time_limit: float = 20.0, dtype=torch.bfloat16, cmap=None,
                 nvls_min_consumers: int = 2, plan=None, local_groups: bool = False,
                 nvls_reduce: Optional[bool] = None, plan_type: str = "Flexflow", select: str = "balance"):
        """``select``: how the partition granularity is chosen, ``"balance"`` or ``"model"`` (see
        :func:`plan_allocation`).
        ``plan_type`` (NCCL path): how the launch order on the compute / send / receive streams
        is chosen, ``"Flexflow"`` (list scheduling) or ``"ILP"`` (the kernel-schedule integer
        program, reference search_algo/execute_plan.py:209-275).
        ``plan``: an earlier runtime's ``(table, cmap)`` to reuse instead of solving the
        allocation again (fused path; e.g. a second runtime for a different number of heads).
        ``local_groups``: create the internal process groups with only the members of ``group``
        taking part (needed when ``group`` is a strict subset of the job, as after a rank left)."""
        self._ctor = dict(seq_len=seq_len, n_heads=n_heads, head_dim=head_dim, device=device, path=path,
                          n_kv_heads=n_kv_heads, batch=batch, allocation=allocation,
                          plan_time_limit=plan_time_limit, dtype=dtype, nvls_min_consumers=nvls_min_consumers,
                          nvls_reduce=nvls_reduce, plan_type=plan_type, select=select)
        shape = {"seq_len": seq_len, "n_heads": n_heads, "head_dim": head_dim, "n_kv_heads": n_kv_heads, "batch": batch}
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.path = path
        self.pattern = pattern
        if path == "fused":
            from .fused import FusedContextParallel, SymmMemSpace
            box = [(plan if plan is not None else
                    plan_allocation(pattern, self.world, 1, allocation, plan_time_limit, cmap, select, shape))
                   if self.rank == 0 else None]
            dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0), group=self.group)
            table, cm = box[0]
            self.table, self.cmap = table, cm
            space = SymmMemSpace(self.group, self.device)
            self.impl = FusedContextParallel(table, cm, pattern, seq_len, n_heads, head_dim, space,
                                             n_kv_heads, batch, dtype, self.device,
                                             nvls_min_consumers=nvls_min_consumers, nvls_reduce=nvls_reduce)
        elif path == "nccl":
            from .executor import PlanExecutor
            kw = dict(pattern=pattern, cp=self.world, seq_len=seq_len, n_heads=n_heads, head_dim=head_dim,
                      n_kv_heads=n_kv_heads, batch=batch, allocation=allocation, plan_type=plan_type,
                      time_limit=plan_time_limit, cmap=cmap)
            if self.rank == 0 and allocation not in ("naive", "lightseq"):
                # same partition granularity (and, with cmap="search", ownership) as the fused path
                table0, cmap0 = plan_allocation(pattern, self.world, 1, allocation, plan_time_limit, cmap, select, shape)
                kw["ParD"] = table0.shape[0]
                if isinstance(cmap, str):
                    kw["cmap"] = cmap0
            box = [(make_plan(fob=0, **kw), make_plan(fob=1, **kw)) if self.rank == 0 else None]
            dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0), group=self.group)
            pf, pb = box[0]
            ranks = [dist.get_global_rank(self.group, r) for r in range(self.world)]
            duplex = tuple(dist.new_group(ranks, use_local_synchronization=local_groups) for _ in range(2))
            self.impl = PlanExecutor(pf, pb, group=self.group, device=self.device, p2p_groups=duplex)
            self.table = np.asarray(pf.allocation.table)
            self.cmap = np.asarray(pf.allocation.cmap)
        else:
            raise ValueError(f"unknown path {path!r}")

    def replan(self, group, **overrides) -> "ContextParallelAttention":
        """A runtime for the same problem over another set of ranks, e.g. the survivors after a
        rank left between two steps: the allocation is solved again for the new world size (plans
        are cheap at these sizes) and every member then passes its new, larger shard. Collective
        over ``group`` only. The reference has no recovery path (a failed task ends the job,
        scripts/runtime/wrapper_bx.sh:19); this is the building block for one."""
        kw = dict(self._ctor, **overrides)
        return ContextParallelAttention(self.pattern, group=group, local_groups=True, **kw)

    def forward(self, q, k, v, softmax_scale=None):
        return self.impl.forward(q, k, v, softmax_scale)

    def backward(self, d_o, q, k, v, o, lse, softmax_scale=None):
        return self.impl.backward(d_o, q, k, v, o, lse, softmax_scale)

    def __call__(self, q, k, v, softmax_scale=None):
        return _CPFunction.apply(q, k, v, self, softmax_scale)
