"""Context-parallel sliding-window attention by halo exchange.

With contiguous shards (rank g holds tokens ``[g * S_loc, (g + 1) * S_loc)``) and a causal
window of ``left`` tokens, the queries of a rank can only see their own keys and the last ``left``
keys in front of the shard. Those keys (the halo) are fetched from the one or few preceding ranks
that hold them, attention runs locally with the queries standing at the end of ``[halo | shard]``
(``ops/window.py``: band with the queries at an offset inside the keys), and in the backward pass
the halo's dK / dV travel back to their owners and are added there. A two-sided window
(``right`` > 0, encoder-style local attention) also fetches the first ``right`` keys behind the
shard from the following ranks. Per rank and pass this moves ``2 * left`` key/value rows
instead of the ``2 * (world - 1) * S_loc`` of a ring, and every rank does the same work, so there
is nothing to balance.

The reference has no strategy for token-exact windows (its flash-attention calls always pass
``window_size = (-1, -1)``, ring_flash_attn/ring_flash_attn.py:33-43); its "streaming" pattern is
the block-level counterpart, which the planner-driven runtimes execute.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops.window import window_backward, window_forward


def _halo_plan(rank: int, world: int, s_loc: int, left: int, right: int = 0) -> dict:
    """Routes of one exchange. ``recv_front`` / ``recv_back``: [(source rank, tokens)] in token
    order, the halo in front of the shard (from preceding ranks, their tails) and behind it (from
    following ranks, their heads). ``send_tail`` / ``send_head``: [(destination rank, tokens)], the
    tail of this shard that a following rank sees and the head that a preceding rank sees. A rank
    at distance d contributes ``window - (d - 1) * S_loc`` of its tokens, capped at its shard."""
    plan = {"recv_front": [], "recv_back": [], "send_tail": [], "send_head": []}
    d = 1
    while (d - 1) * s_loc < max(left, right):
        nl = min(s_loc, left - (d - 1) * s_loc)
        nr = min(s_loc, right - (d - 1) * s_loc)
        if nl > 0:
            if rank - d >= 0:
                plan["recv_front"].append((rank - d, nl))
            if rank + d < world:
                plan["send_tail"].append((rank + d, nl))
        if nr > 0:
            if rank + d < world:
                plan["recv_back"].append((rank + d, nr))
            if rank - d >= 0:
                plan["send_head"].append((rank - d, nr))
        d += 1
    plan["recv_front"].reverse()             # farthest rank first = token order
    return plan


def _exchange(send_bufs: list, recv_shapes: list, like: torch.Tensor, group) -> list:
    """Post all sends (``[(peer, tensor)]``) and receives (``[(peer, shape)]``) of one phase as one
    batch and wait; returns the received tensors in the order of ``recv_shapes``. Two messages
    between the same pair of ranks are matched in posting order, which both sides build alike
    (front / tail routes before back / head routes)."""
    ops, out = [], []
    to_global = (lambda p: dist.get_global_rank(group, p)) if group is not None else (lambda p: p)
    for peer, shape in recv_shapes:
        buf = torch.empty(shape, dtype=like.dtype, device=like.device)
        out.append(buf)
        ops.append(dist.P2POp(dist.irecv, buf, to_global(peer), group))
    for peer, t in send_bufs:
        ops.append(dist.P2POp(dist.isend, t.contiguous(), to_global(peer), group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return out


def halo_extend(group, k, v, left: int, right: int = 0):
    """``[front halo | shard | back halo]`` key and value rows of this rank and the number of front
    rows: the shard with the last ``left`` rows in front of it and the first ``right`` rows behind
    it, received from the ranks that hold them (every rank of the group calls this)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    s_loc = k.shape[1]
    plan = _halo_plan(rank, world, s_loc, left, right)
    kv = torch.stack([k, v])                                        # one message per peer, side and pass
    shape = lambda n: (2, k.shape[0], n) + tuple(k.shape[2:])
    got = _exchange([(peer, kv[:, :, s_loc - n:]) for peer, n in plan["send_tail"]]
                    + [(peer, kv[:, :, :n]) for peer, n in plan["send_head"]],
                    [(peer, shape(n)) for peer, n in plan["recv_front"] + plan["recv_back"]], k, group)
    nf = len(plan["recv_front"])
    parts = got[:nf] + [kv] + got[nf:]
    ext = torch.cat(parts, dim=2)
    return ext[0], ext[1], sum(n for _, n in plan["recv_front"])


def halo_window_attn_forward(group, q, k, v, left: int, softmax_scale: Optional[float] = None, right: int = 0):
    """``q`` ``[B, S_loc, H, D]``, ``k`` / ``v`` ``[B, S_loc, Hkv, D]`` (this rank's contiguous shard).
    Returns ``(o, lse, k_ext, v_ext)``: the output of the shard's queries and the key/value rows
    ``[front halo | shard | back halo]`` that the backward takes."""
    k_ext, v_ext, front = halo_extend(group, k, v, left, right)
    o, lse = window_forward(q, k_ext, v_ext, (left, right), False, softmax_scale, q_offset=front)
    return o, lse, k_ext, v_ext


def halo_window_attn_backward(group, d_o, q, k_ext, v_ext, o, lse, left: int, softmax_scale: Optional[float] = None,
                              right: int = 0):
    """Gradients of this rank's shard: dQ is local; dK / dV of the halo rows go back to the ranks
    that own them, and what the neighbours computed for this shard's tail and head is added here."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    s_loc = q.shape[1]
    plan = _halo_plan(rank, world, s_loc, left, right)              # the forward's routes, walked backwards
    front = sum(n for _, n in plan["recv_front"])
    dq, dk_ext, dv_ext = window_backward(d_o, q, k_ext, v_ext, o, lse, (left, right), False, softmax_scale,
                                         q_offset=front)
    dkv = torch.stack([dk_ext, dv_ext])
    back, a = [], 0
    for peer, n in plan["recv_front"]:
        back.append((peer, dkv[:, :, a:a + n]))
        a += n
    mine = dkv[:, :, a:a + s_loc].clone()
    a += s_loc
    for peer, n in plan["recv_back"]:
        back.append((peer, dkv[:, :, a:a + n]))
        a += n
    shape = lambda n: (2, q.shape[0], n) + tuple(k_ext.shape[2:])
    got = _exchange(back, [(peer, shape(n)) for peer, n in plan["send_tail"] + plan["send_head"]], dkv, group)
    nt = len(plan["send_tail"])
    for (peer, n), g in zip(plan["send_tail"], got[:nt]):
        mine[:, :, s_loc - n:] += g
    for (peer, n), g in zip(plan["send_head"], got[nt:]):
        mine[:, :, :n] += g
    return dq, mine[0], mine[1]


class HaloWindowAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, left, softmax_scale, group, right=0):
        o, lse, k_ext, v_ext = halo_window_attn_forward(group, q, k, v, int(left), softmax_scale, int(right))
        ctx.save_for_backward(q, k_ext, v_ext, o, lse)
        ctx.args = (int(left), softmax_scale, group, int(right))
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k_ext, v_ext, o, lse = ctx.saved_tensors
        left, scale, group, right = ctx.args
        dq, dk, dv = halo_window_attn_backward(group, d_o.contiguous(), q, k_ext, v_ext, o, lse, left, scale, right)
        return dq, dk, dv, None, None, None, None


def halo_window_attn_func(q, k, v, window_size, softmax_scale: Optional[float] = None, causal: bool = True,
                          group=None) -> torch.Tensor:
    """Sliding-window attention over a sequence sharded contiguously across ``group``; autograd.
    ``window_size = (left, right)`` as in flash-attention, both bounded; ``causal`` sets
    ``right = 0`` (the default: a causal window fetches nothing from the ranks behind)."""
    left, right = (int(x) for x in window_size)
    right = 0 if causal else right
    assert left >= 0 and right >= 0, \
        "an unbounded side is not a window: use the ring or the planner-driven runtime for causal / full attention"
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        from ..ops.window import sliding_window_attention
        return sliding_window_attention(q, k, v, (left, right), False, softmax_scale)
    return HaloWindowAttnFunc.apply(q, k, v, left, softmax_scale, group, right)
