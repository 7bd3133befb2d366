"""Two-level (node x device) attention baselines.

Reference: hierarchy_attn/hierarchy_attn_impl.py:14-277 — inside a node K/V travel a ring, across
nodes the queries visit the other nodes and (O, lse) come back; forward only in the reference
(its backward is ``pass``), with an ``overlapped`` variant that double-buffers the query / output
exchange (hierarchy_attn/utils.py:201-287). Two modes here, both with a backward:

``mode="kv"`` (default)  both levels move K/V: a block makes a full tour of the intra-node ring
    and then takes one hop on the inter-node ring, so only every ``tasks_per_node``-th hop crosses
    the slow links; queries and outputs never leave their rank; dK/dV travel with their block and
    go home with one exchange per level.
``mode="qo"``  the reference's scheme: K/V never leave their node. For every other node, the
    queries visit the rank with the same local index there, run that node's intra ring, and the
    partial (O, lse) comes back and is merged. The next visitor's queries are requested before the
    current visitor is computed (the overlapped form). Backward: Q, dO, O, lse visit the same way,
    the host node's ring yields the visitor's dQ (sent back and added) and adds to its own dK/dV.

On a single NVSwitch box the inter level has one node and both reduce to the ring strategy.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import elementwise as E
from .comm import count_comm
from .ring import _check_unsupported, _RingFunc, _Route, ring_backward, ring_forward

_group_cache: dict = {}


def create_hierarchy_groups(tasks_per_node: int, world_size: int | None = None) -> dict:
    """``{'intra': pg, 'inter': pg}`` for consecutive-rank nodes (reference:
    hierarchy_attn/utils.py:69-117 creates its intra / inter groups the same way, lazily). Every
    rank must call this (``dist.new_group`` is collective); the result is cached."""
    world = world_size or dist.get_world_size()
    key = (tasks_per_node, world)
    if key in _group_cache:
        return _group_cache[key]
    assert world % tasks_per_node == 0
    rank = dist.get_rank()
    groups = {}
    for n in range(world // tasks_per_node):
        ranks = list(range(n * tasks_per_node, (n + 1) * tasks_per_node))
        g = dist.new_group(ranks)
        if rank in ranks:
            groups["intra"] = g
    for loc in range(tasks_per_node):
        ranks = list(range(loc, world, tasks_per_node))
        g = dist.new_group(ranks)
        if rank in ranks:
            groups["inter"] = g
    _group_cache[key] = groups
    return groups


class InterExchange:
    """Exchange of whole tensors with the rank of the same local index on another node
    (reference: ``InterComm`` / ``OverlappedInterComm``, hierarchy_attn/utils.py:119-287):
    ``post`` starts sends to node ``me + shift`` and receives from node ``me - shift`` (or the
    reverse direction), ``wait`` completes them and returns the received tensors."""

    def __init__(self, inter_group):
        self.group = inter_group
        self.n = dist.get_world_size(inter_group)
        self.me = dist.get_rank(inter_group)

    def _glob(self, node: int) -> int:
        return dist.get_global_rank(self.group, node % self.n)

    def post(self, tensors, shift: int, like=None):
        """Send ``tensors`` ``shift`` nodes ahead (negative: back); receive the same shapes (or
        the shapes of ``like``) from ``shift`` nodes behind."""
        recv = [torch.empty_like(t) for t in (like if like is not None else tensors)]
        ops = []
        for t in tensors:
            t = t.contiguous()
            count_comm(send_bytes=t.numel() * t.element_size())
            ops.append(dist.P2POp(dist.isend, t, self._glob(self.me + shift), group=self.group))
        for r in recv:
            count_comm(recv_bytes=r.numel() * r.element_size())
            ops.append(dist.P2POp(dist.irecv, r, self._glob(self.me - shift), group=self.group))
        return dist.batch_isend_irecv(ops) if ops else [], recv

    @staticmethod
    def wait(handle):
        reqs, recv = handle
        for r in reqs:
            r.wait()
        return recv


def _qo_forward(q, k, v, groups, kind, causal, scale):
    intra, ex = groups["intra"], InterExchange(groups["inter"])
    P, local = dist.get_world_size(intra), dist.get_rank(intra)
    route = _Route(intra, offset=ex.me * P)
    o, lse = ring_forward(q, k, v, route, kind, causal, scale)
    pending = ex.post([q], 1) if ex.n > 1 else None
    for t in range(1, ex.n):
        (q_f,) = ex.wait(pending)
        # overlapped form: the next visitor is already on its way while this one is computed
        pending = ex.post([q], t + 1) if t + 1 < ex.n else None
        owner = ((ex.me - t) % ex.n) * P + local
        o_f, lse_f = ring_forward(q_f, k, v, route, kind, causal, scale, q_rank=owner)
        o_b, lse_b = ex.wait(ex.post([o_f, lse_f], -t))
        for b in range(q.shape[0]):
            E.lse_merge([(o[b], lse[b]), (o_b[b], lse_b[b])], (o[b], lse[b]))
    return o, lse


def _qo_backward(d_o, q, k, v, o, lse, groups, kind, causal, scale):
    intra, ex = groups["intra"], InterExchange(groups["inter"])
    P, local = dist.get_world_size(intra), dist.get_rank(intra)
    route = _Route(intra, offset=ex.me * P)
    dq, dk, dv = ring_backward(d_o, q, k, v, o, lse, route, kind, causal, scale, keep_f32=True)
    bundle = [q, d_o, o, lse]
    pending = ex.post(bundle, 1) if ex.n > 1 else None
    for t in range(1, ex.n):
        q_f, do_f, o_f, lse_f = ex.wait(pending)
        pending = ex.post(bundle, t + 1) if t + 1 < ex.n else None
        owner = ((ex.me - t) % ex.n) * P + local
        dq_f, dk_t, dv_t = ring_backward(do_f, q_f, k, v, o_f, lse_f, route, kind, causal, scale,
                                         q_rank=owner, keep_f32=True)
        dk += dk_t
        dv += dv_t
        (dq_b,) = ex.wait(ex.post([dq_f], -t))
        dq += dq_b
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


class _HierarchyQOFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, groups, kind):
        o, lse = _qo_forward(q, k.contiguous(), v.contiguous(), groups, kind, causal, softmax_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.args = (softmax_scale, causal, groups, kind)
        return o, lse

    @staticmethod
    def backward(ctx, d_o, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, groups, kind = ctx.args
        dq, dk, dv = _qo_backward(d_o.contiguous(), q, k.contiguous(), v.contiguous(), o, lse, groups, kind,
                                  causal, scale)
        return dq, dk, dv, None, None, None, None


def hierarchy_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                        alibi_slopes=None, deterministic=False, return_attn_probs=False, groups=None,
                        group=None, PROC_INFO=None, mode: str = "kv"):
    """``groups``: ``{'intra': pg, 'inter': pg}`` (the reference's convention; see
    :func:`create_hierarchy_groups`). Shards are ordered by ``node * tasks_per_node + local rank``;
    causal inputs use the zigzag layout over that order (``shard_sequence(..., 'zigzag')``).
    ``mode``: "kv" or "qo" (see the module text)."""
    _check_unsupported(dropout_p, alibi_slopes, window_size)
    route = group
    two_level = isinstance(groups, dict) and groups.get("inter") is not None \
        and dist.get_world_size(groups["inter"]) > 1
    if two_level and mode == "qo":
        o, lse = _HierarchyQOFunc.apply(q, k, v, softmax_scale, causal, groups, "zigzag" if causal else "ring")
        return (o, lse, None) if return_attn_probs else o
    if two_level:
        route = {"intra": groups["intra"], "inter": groups["inter"]}
    elif isinstance(groups, dict):
        route = groups.get("intra", group)
    o, lse = _RingFunc.apply(q, k, v, softmax_scale, causal, route, "zigzag" if causal else "ring")
    return (o, lse, None) if return_attn_probs else o
