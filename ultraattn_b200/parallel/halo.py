"""Context-parallel sliding-window attention by halo exchange.

With contiguous shards (rank g holds tokens ``[g * S_loc, (g + 1) * S_loc)``) and a causal
window of ``left`` tokens, the queries of a rank can only see their own keys and the last ``left``
keys in front of the shard. Those keys (the halo) are fetched from the one or few preceding ranks
that hold them, attention runs locally with the queries standing at the end of ``[halo | shard]``
(``ops/window.py``: bottom-right aligned band), and in the backward pass the halo's dK / dV travel
back to their owners and are added there. Per rank and pass this moves ``2 * left`` key/value rows
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


def _halo_plan(rank: int, world: int, s_loc: int, left: int) -> tuple[list, list]:
    """(receives, sends): ``receives`` = [(source rank, tokens)] nearest rank last, i.e. in token
    order; ``sends`` = [(destination rank, tokens)]: the tail of this shard that the destination
    sees. A rank at distance d in front of the reader contributes the last ``left - (d - 1) * S_loc``
    of its tokens, capped at its shard."""
    recv, send = [], []
    d = 1
    while (d - 1) * s_loc < left:
        n = min(s_loc, left - (d - 1) * s_loc)
        if rank - d >= 0:
            recv.append((rank - d, n))
        if rank + d < world:
            send.append((rank + d, n))
        d += 1
    return recv[::-1], send


def _exchange(send_bufs: list, recv_shapes: list, like: torch.Tensor, group) -> list:
    """Post all sends (``[(peer, tensor)]``) and receives (``[(peer, shape)]``) of one phase as one
    batch and wait; returns the received tensors in the order of ``recv_shapes``."""
    ops, out = [], []
    for peer, shape in recv_shapes:
        buf = torch.empty(shape, dtype=like.dtype, device=like.device)
        out.append(buf)
        ops.append(dist.P2POp(dist.irecv, buf, dist.get_global_rank(group, peer) if group is not None else peer, group))
    for peer, t in send_bufs:
        ops.append(dist.P2POp(dist.isend, t.contiguous(), dist.get_global_rank(group, peer) if group is not None else peer,
                              group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return out


def halo_extend(group, k, v, left: int):
    """``[halo | shard]`` key and value rows of this rank: the shard with the last ``left`` rows in
    front of it, received from the ranks that hold them (every rank of the group calls this)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    s_loc = k.shape[1]
    recv, send = _halo_plan(rank, world, s_loc, left)
    kv = torch.stack([k, v])                                        # one message per peer and pass
    got = _exchange([(peer, kv[:, :, s_loc - n:]) for peer, n in send],
                    [(peer, (2, k.shape[0], n) + tuple(k.shape[2:])) for peer, n in recv], k, group)
    return torch.cat([g[0] for g in got] + [k], dim=1), torch.cat([g[1] for g in got] + [v], dim=1)


def halo_window_attn_forward(group, q, k, v, left: int, softmax_scale: Optional[float] = None):
    """``q`` ``[B, S_loc, H, D]``, ``k`` / ``v`` ``[B, S_loc, Hkv, D]`` (this rank's contiguous shard).
    Returns ``(o, lse, k_ext, v_ext)``: the output of the shard's queries and the key/value rows
    ``[halo | shard]`` that the backward takes."""
    k_ext, v_ext = halo_extend(group, k, v, left)
    o, lse = window_forward(q, k_ext, v_ext, (left, 0), True, softmax_scale)
    return o, lse, k_ext, v_ext


def halo_window_attn_backward(group, d_o, q, k_ext, v_ext, o, lse, left: int, softmax_scale: Optional[float] = None):
    """Gradients of this rank's shard: dQ is local; dK / dV of the halo rows go back to the ranks
    that own them, and what the following ranks computed for this shard's tail is added here."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    s_loc = q.shape[1]
    recv, send = _halo_plan(rank, world, s_loc, left)               # the forward's routes, walked backwards
    dq, dk_ext, dv_ext = window_backward(d_o, q, k_ext, v_ext, o, lse, (left, 0), True, softmax_scale)
    dkv = torch.stack([dk_ext, dv_ext])
    back, a = [], 0
    for peer, n in recv:
        back.append((peer, dkv[:, :, a:a + n]))
        a += n
    mine = dkv[:, :, a:].clone()
    got = _exchange(back, [(peer, (2, q.shape[0], n) + tuple(k_ext.shape[2:])) for peer, n in send], dkv, group)
    for (peer, n), g in zip(send, got):
        mine[:, :, s_loc - n:] += g
    return dq, mine[0], mine[1]


class HaloWindowAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, left, softmax_scale, group):
        o, lse, k_ext, v_ext = halo_window_attn_forward(group, q, k, v, int(left), softmax_scale)
        ctx.save_for_backward(q, k_ext, v_ext, o, lse)
        ctx.args = (int(left), softmax_scale, group)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k_ext, v_ext, o, lse = ctx.saved_tensors
        left, scale, group = ctx.args
        dq, dk, dv = halo_window_attn_backward(group, d_o.contiguous(), q, k_ext, v_ext, o, lse, left, scale)
        return dq, dk, dv, None, None, None


def halo_window_attn_func(q, k, v, window_size, softmax_scale: Optional[float] = None, causal: bool = True,
                          group=None) -> torch.Tensor:
    """Causal sliding-window attention over a sequence sharded contiguously across ``group``;
    autograd. ``window_size = (left, right)`` as in flash-attention; the window has to be causal
    (``causal=True`` or ``right == 0``) and bounded to the left."""
    left, right = (int(x) for x in window_size)
    assert causal or right == 0, "the halo strategy takes causal windows (keys behind the query are not fetched)"
    assert left >= 0, "an unbounded window is plain causal attention: use the ring or the planner-driven runtime"
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        from ..ops.window import sliding_window_attention
        return sliding_window_attention(q, k, v, (left, 0), True, softmax_scale)
    return HaloWindowAttnFunc.apply(q, k, v, left, softmax_scale, group)
