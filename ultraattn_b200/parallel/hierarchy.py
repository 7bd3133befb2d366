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


# -------------------------------------------------------------------------------------------------
# The reference's function and class names (hierarchy_attn/hierarchy_attn_impl.py:14-445). Its
# backward functions are empty (``pass``); these work. ``process_groups`` = {'intra': pg, 'inter': pg}.
# -------------------------------------------------------------------------------------------------
def intra_attn_forward(process_groups, q, k, v, softmax_scale, out=None, lse=None, dropout_p=0, causal=True,
                       window_size=(-1, -1), alibi_slopes=None, deterministic=False, PROC_INFO=None):
    """One intra-node ring pass; a given running ``(out, lse)`` is merged into (the reference's
    resumable form, hierarchy_attn_impl.py:14-104)."""
    _check_unsupported(dropout_p, alibi_slopes, window_size)
    group = process_groups["intra"] if isinstance(process_groups, dict) else process_groups
    o, l = ring_forward(q, k.contiguous(), v.contiguous(), group, "zigzag" if causal else "ring", causal, softmax_scale)
    if out is not None and lse is not None:
        for b in range(q.shape[0]):
            E.lse_merge([(out[b], lse[b]), (o[b], l[b])], (out[b], lse[b]))
        return out, lse
    return o, l


def hierarchy_attn_forward(process_groups, q, k, v, softmax_scale, dropout_p=0, causal=True, window_size=(-1, -1),
                           alibi_slopes=None, deterministic=False, PROC_INFO=None):
    """(out, lse) of the two-level scheme in which queries visit the other nodes ("qo" mode)."""
    _check_unsupported(dropout_p, alibi_slopes, window_size)
    return _qo_forward(q, k.contiguous(), v.contiguous(), process_groups, "zigzag" if causal else "ring", causal,
                       softmax_scale)


def hierarchy_attn_backward(process_group, dout, q, k, v, out, softmax_lse, softmax_scale, dropout_p=0, causal=True,
                            window_size=(-1, -1), alibi_slopes=None, deterministic=False):
    """(dq, dk, dv) of the same scheme."""
    _check_unsupported(dropout_p, alibi_slopes, window_size)
    return _qo_backward(dout.contiguous(), q, k.contiguous(), v.contiguous(), out, softmax_lse, process_group,
                        "zigzag" if causal else "ring", causal, softmax_scale)


# the visitor for step t + 1 is always requested before step t is computed: the plain and the
# "overlapped" forms of the reference are one function here
overlapped_hierarchy_attn_forward = hierarchy_attn_forward
overlapped_hierarchy_attn_backward = hierarchy_attn_backward


class HierarchyAttnFunc(torch.autograd.Function):
    """``apply(q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes, deterministic,
    return_softmax, groups, PROC_INFO, overlapped)`` as in the reference (:313-412)."""

    @staticmethod
    def forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes, deterministic,
                return_softmax, groups, PROC_INFO=None, overlapped=False):
        o, lse = hierarchy_attn_forward(groups, q, k, v, softmax_scale, dropout_p, causal, window_size, alibi_slopes)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.args = (softmax_scale, causal, groups)
        return (o, lse, None) if return_softmax else o

    @staticmethod
    def backward(ctx, d_o, *rest):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, groups = ctx.args
        return tuple(hierarchy_attn_backward(groups, d_o, q, k, v, o, lse, scale, causal=causal)) + (None,) * 10


# -------------------------------------------------------------------------------------------------
# Communicator classes with the interface of the reference's hierarchy_attn/utils.py:69-287, for
# code written against it. (The functions above use ``RingComm`` and ``InterExchange`` instead.)
# -------------------------------------------------------------------------------------------------
def wait_recursively(reqs) -> None:
    """Wait for a request or any nesting of lists of requests (None: nothing to wait for)."""
    if reqs is None:
        return
    if isinstance(reqs, (list, tuple)):
        for r in reqs:
            wait_recursively(r)
        return
    reqs.wait()


class IntraComm:
    """Neighbour exchange on the intra-node ring of ``process_groups['intra']``: ``send_recv``
    queues a send to the next local rank and a receive from the previous one, ``commit`` starts
    the batch, ``wait`` completes it (reference: hierarchy_attn/utils.py:69-123)."""

    def __init__(self, process_groups, PROC_INFO: dict = None):
        from .comm import RingComm
        group = process_groups["intra"] if isinstance(process_groups, dict) else process_groups
        self._ring = RingComm(group)
        self.rank, self.world_size = self._ring.rank, self._ring.world

    def send_recv(self, to_send: torch.Tensor, recv_tensor=None) -> torch.Tensor:
        return self._ring.send_recv(to_send, recv_tensor)

    def commit(self) -> None:
        self._ring.commit()

    def wait(self) -> None:
        self._ring.wait()


class InterComm:
    """Exchange with the same local rank on other nodes, step by step, without wrap-around: in
    step s the offset is ``s // 2 + 1`` (even s) or ``nodes - (s // 2 + 1)`` (odd s); queries go
    to node ``me - offset`` and come from ``me + offset``, partial (O, lse) travel the other way;
    a partner outside ``[0, nodes)`` means nothing is sent / ``None`` is returned (reference:
    hierarchy_attn/utils.py:125-202). ``PROC_INFO`` needs ``nodeid`` and ``tasks_per_node`` when
    the inter group is not given as ``process_groups['inter']``."""

    def __init__(self, process_groups: dict, PROC_INFO: dict = None):
        self.process_groups = process_groups
        if process_groups.get("inter") is None:
            assert PROC_INFO is not None, "PROC_INFO (rank, world_size, tasks_per_node) is needed to build the inter groups"
            local, world, me = PROC_INFO["tasks_per_node"], PROC_INFO["world_size"], PROC_INFO["rank"]
            for i in range(local):                     # collective: every rank creates every group
                ranks = list(range(i, world, local))
                g = dist.new_group(ranks)
                if me in ranks:
                    process_groups["inter"] = g
        self.group = process_groups["inter"]
        self.node_num = dist.get_world_size(self.group)
        self.node_id = dist.get_rank(self.group)
        self._ops, self._reqs = [], None

    def _offset(self, step: int) -> int:
        return step // 2 + 1 if step % 2 == 0 else self.node_num - (step // 2 + 1)

    def _peer(self, node: int):
        return dist.get_global_rank(self.group, node) if 0 <= node < self.node_num else None

    def send_recv_q(self, step: int, q: torch.Tensor, _q=None):
        off = self._offset(step)
        dst, src = self._peer(self.node_id - off), self._peer(self.node_id + off)
        if dst is not None:
            self._ops.append(dist.P2POp(dist.isend, q.contiguous(), dst, group=self.group))
        if src is None:
            return None
        _q = torch.empty_like(q) if _q is None else _q
        self._ops.append(dist.P2POp(dist.irecv, _q, src, group=self.group))
        return _q

    def send_recv_o(self, step: int, o: torch.Tensor, lse: torch.Tensor, _o=None, _lse=None):
        off = self._offset(step)
        dst, src = self._peer(self.node_id + off), self._peer(self.node_id - off)
        if dst is not None:
            self._ops.append(dist.P2POp(dist.isend, o.contiguous(), dst, group=self.group))
            self._ops.append(dist.P2POp(dist.isend, lse.contiguous(), dst, group=self.group))
        if src is None:
            return None, None
        _o = torch.empty_like(o) if _o is None else _o
        _lse = torch.empty_like(lse) if _lse is None else _lse
        self._ops.append(dist.P2POp(dist.irecv, _o, src, group=self.group))
        self._ops.append(dist.P2POp(dist.irecv, _lse, src, group=self.group))
        return _o, _lse

    def commit(self) -> None:
        if self._reqs is not None:
            raise RuntimeError("commit called twice")
        if self._ops:
            self._reqs = dist.batch_isend_irecv(self._ops)
            self._ops = []

    def wait(self) -> None:
        wait_recursively(self._reqs)
        self._reqs = None


OverlappedInterComm = InterComm      # requests are always posted ahead of the compute they feed
