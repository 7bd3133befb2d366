"""Sliding-window (local) attention on the block-sparse kernels, without a kernel of its own.

Query ``r`` sees the keys ``r - left <= c <= r + right`` (flash-attention's ``window_size =
(left, right)``, -1 = unbounded; ``causal`` sets ``right = 0``). The kernels mask one-sidedly: a
segment is either fully visible or bounded from above by ``c <= r + diag``. A band needs both
bounds, but never both inside one tile if the work is split in two:

* part A, in the usual token order: row block ``[r0, r1)`` against the keys from ``r0`` on. Only
  the upper bound can bind there (``c >= r0 >= r - left`` as long as the block is at most
  ``left + 1`` rows long), which is the kernels' causal mask with ``diag = right``;
* part B, in reversed token order (``r' = S - 1 - r``, ``c' = S - 1 - c``): the same row block
  against the keys before ``r0``. Only the lower bound ``c >= r - left`` can bind there, and
  reversed it reads ``c' <= r' + left``: again the kernels' causal mask.

Both parts go into one forward launch (two query sources, two key/value sources, two outputs) and
one backward launch; the partial results are merged by their log-sum-exps like the steps of a ring.
The reversed copies cost three passes over Q, K, V (and dO) - small beside the attention itself.

Attention sinks (the first ``sink_tokens`` keys stay visible to every later query: the exact,
token-level form of the "streaming" pattern) add a third part: a fully visible segment ``[0,
sink_tokens)`` for every row block behind the first, with the band clipped so that no key is
counted twice; its dK / dV go to a buffer of their own and are added afterwards.

The reference's flash-attention fork accepts ``window_size`` in every call
(ring_flash_attn/ring_flash_attn.py:33-43) and always passes ``(-1, -1)``.
"""
from __future__ import annotations

import functools
import math
from typing import Optional

import torch

from . import attention as A
from . import elementwise as E

ROW_BLOCK = 256         # rows of the kernels' forward tile


def _bounds(S: int, window_size, causal: bool) -> tuple[int, int]:
    left, right = (int(x) for x in window_size)
    left = S if left < 0 else min(left, S)
    right = S if right < 0 else min(right, S)
    if causal:
        right = 0
    return left, right


def _partition(S: int, left: int) -> list:
    """Row blocks [r0, r1): at most ``left + 1`` rows each, so that inside part A the lower bound
    and inside part B the upper bound never bind."""
    step = max(1, min(ROW_BLOCK, left + 1))
    return [(a, min(S, a + step)) for a in range(0, S, step)]


def window_rows_cols(S: int, left: int, right: int, base: int = 0, total: Optional[int] = None,
                     sink: int = 0) -> tuple[list, list]:
    """(forward rows, backward columns) of the plan for one sequence of ``S`` tokens that starts at
    token ``base`` of a buffer of ``total`` tokens (a packed batch; default: the sequence is the
    buffer). Source / output slot 0 is the usual token order, slot 1 the buffer reversed, where the
    sequence occupies ``[total - base - S, total - base)``. With ``sink`` > 0 the first ``sink``
    keys are visible to every query behind the first row block (which sees them through its
    causal part anyway); their gradients are collected in gradient slot 2 at rows ``base...``."""
    total = S if total is None else total
    rbase = total - base - S
    blocks = _partition(S, left)
    sink = min(sink, S)
    assert sink <= blocks[0][1], f"at most {blocks[0][1]} sink tokens fit the first row block of this window"
    rows, cols = [], []
    for r0, r1 in blocks:
        n = r1 - r0
        s_here = sink if r0 > 0 else 0              # sink keys this block sees as a segment of their own
        # part A (+ the sinks)
        a_len = min(S, r1 + right) - r0
        segs = (A.Seg(0, base + r0, a_len, right < S, right),)
        if s_here:
            segs = (A.Seg(0, base, s_here, False, 0),) + segs
        rows.append(A.Row(0, base + r0, n, segs, 0, base + r0, False))
        q0 = max(0, r0 - right)                      # key block [r0, r1): rows from q0 to r1 reach it
        cols.append(A.Col(0, base + r0, n, (A.Seg(0, base + q0, r1 - q0, right < S, q0 + right - r0),), 0, base + r0))
        # part B, reversed order: row block [S - r1, S - r0), its keys start right behind it and
        # stop before the sinks
        b_len = min(left, r0 - s_here)
        if b_len > 0:
            rows.append(A.Row(1, rbase + S - r1, n, (A.Seg(1, rbase + S - r0, b_len, left < S, left - n),), 1,
                              rbase + S - r1, False))
        c0 = S - r1                                  # the same block as a key block of the reversed order
        q0 = max(0, c0 - left)
        if c0 - q0 > 0 and not (sink and r1 <= sink):
            # as keys, the first `sink` tokens of the sequence belong to the sink part for every
            # later row block, so in the reversed order the key block loses them
            k_len = n if r0 >= sink else r1 - sink      # reversed, the sink keys are the tail of the first block
            cols.append(A.Col(1, rbase + c0, k_len, (A.Seg(1, rbase + q0, c0 - q0, left < S, q0 + left - c0),), 1,
                              rbase + c0))
    if sink and len(blocks) > 1:
        first = blocks[0][1]
        cols.append(A.Col(0, base, sink, (A.Seg(0, base + first, S - first, False, 0),), 2, base))
    return rows, cols


def window_rows_cols_offset(Sq: int, Skv: int, left: int, right: int, off: Optional[int] = None) -> tuple[list, list]:
    """The two-part plan when the ``Sq`` queries are a stretch of a longer sequence of ``Skv`` keys
    (a chunk behind cached context, or a shard between the halos received from its neighbours):
    query ``r`` stands at position ``p = r + off`` and sees ``p - left <= c <= p + right``. Default
    ``off = Skv - Sq``: the queries are the last tokens (the bottom-right alignment of
    flash-attention). Slot 0: usual order; slot 1: the query buffer and the key buffer each
    reversed. Of the keys in front of the first query only the last ``left`` can be seen, of those
    behind the last query only the first ``right``."""
    off = Skv - Sq if off is None else off
    tail = Skv - off - Sq                    # keys behind the last query
    assert off >= 0 and tail >= 0, "the queries must lie inside the key sequence"
    rows, cols = [], []
    for r0, r1 in _partition(Sq, left):
        n, p0, p1 = r1 - r0, r0 + off, r1 + off
        a_len = min(Skv, p1 + right) - p0
        rows.append(A.Row(0, r0, n, (A.Seg(0, p0, a_len, right < Skv, right),), 0, r0, False))
        q0 = max(0, r0 - right)
        cols.append(A.Col(0, p0, n, (A.Seg(0, q0, r1 - q0, right < Skv, q0 + right - r0),), 0, p0))
        b_len = min(left, p0)
        if b_len > 0:
            rows.append(A.Row(1, Sq - r1, n, (A.Seg(1, Skv - p0, b_len, left < Skv, left - n),), 1, Sq - r1, False))
        c0 = Sq - r1                     # the block's start among the reversed queries; among the reversed keys it is c0 + tail
        q0 = max(0, c0 - left)
        if c0 - q0 > 0:
            cols.append(A.Col(1, c0 + tail, n, (A.Seg(1, q0, c0 - q0, left < Skv, q0 + left - c0),), 1, c0 + tail))
    if Sq > 0:
        lo = max(0, off - left)          # keys in front, [lo, off): reversed they lie behind every query
        if off - lo > 0:
            q0 = max(0, Sq - left)
            cols.append(A.Col(1, Sq + tail, off - lo, (A.Seg(1, q0, Sq - q0, left < Skv, q0 + left - Sq),), 1, Sq + tail))
        hi = min(Skv, off + Sq + right)  # keys behind, [off + Sq, hi): seen by the last `right` queries
        if hi - (off + Sq) > 0:
            q0 = max(0, Sq - right)
            cols.append(A.Col(0, off + Sq, hi - (off + Sq), (A.Seg(0, q0, Sq - q0, right < Skv, q0 + right - Sq),), 0,
                              off + Sq))
    return rows, cols


def window_rows_cols_suffix(Sq: int, Skv: int, left: int, right: int) -> tuple[list, list]:
    """:func:`window_rows_cols_offset` with the queries at the end of the keys."""
    return window_rows_cols_offset(Sq, Skv, left, right, Skv - Sq)


@functools.lru_cache(maxsize=32)
def _plans_offset(Sq: int, Skv: int, off: int, window_size: tuple, causal: bool, device_str: str):
    left, right = _bounds(Skv, window_size, causal)
    rows, cols = window_rows_cols_offset(Sq, Skv, left, right, off)
    dev = torch.device(device_str)
    return A.FwdPlan(rows, dev), A.BwdPlan(cols, dev)


@functools.lru_cache(maxsize=32)
def _plans(bounds: tuple, total: int, window_size: tuple, causal: bool, device_str: str, sink: int = 0):
    """Plans of a buffer of ``total`` tokens holding the sequences ``bounds`` = ((start, end), ...)."""
    rows, cols = [], []
    for a, b in bounds:
        if b > a:
            left, right = _bounds(b - a, window_size, causal)
            r, c = window_rows_cols(b - a, left, right, a, total, sink)
            rows += r
            cols += c
    dev = torch.device(device_str)
    return A.FwdPlan(rows, dev), A.BwdPlan(cols, dev)


def _seq_bounds(cu_seqlens, S: int) -> tuple:
    if cu_seqlens is None:
        return ((0, S),)
    cu = [int(x) for x in cu_seqlens]
    assert cu[0] == 0 and cu[-1] <= S, "cu_seqlens must start at 0 and stay inside the buffer"
    return tuple(zip(cu[:-1], cu[1:]))


def _pick_plans(Sq: int, Skv: int, window_size, causal, device, cu_seqlens, sink_tokens, q_offset=None):
    window = tuple(int(x) for x in window_size)
    if Skv != Sq or q_offset:
        assert Skv >= Sq and cu_seqlens is None and not sink_tokens, \
            "with more keys than queries the queries are a stretch of one sequence (no packing, no sinks)"
        return _plans_offset(Sq, Skv, Skv - Sq if q_offset is None else int(q_offset), window, bool(causal), str(device))
    return _plans(_seq_bounds(cu_seqlens, Sq), Sq, window, bool(causal), str(device), int(sink_tokens))


def _whole_sequence_plans(Sq: int, Skv: int, window_size, causal, device, cu_seqlens, q_offset):
    """When the window reaches over every sequence (a 4096-token window on 2048-token documents)
    the band is plain causal or full attention: one work item per sequence in the usual order, no
    reversed copies, no merge. Returns (forward plan, backward plan) or None."""
    if Skv != Sq or q_offset:
        return None
    bounds = _seq_bounds(cu_seqlens, Sq)
    kinds = set()
    for a, b in bounds:
        if b > a:
            left, right = _bounds(b - a, window_size, causal)
            if left < b - a - 1 or 0 < right < b - a - 1:
                return None
            kinds.add(right == 0)
    if len(kinds) != 1:
        return None
    from ..api import varlen_plans
    cu = [bounds[0][0]] + [b for _, b in bounds]
    return varlen_plans(cu, kinds.pop(), device)


def _flip(t: torch.Tensor, dim: int = 1) -> torch.Tensor:
    return t.flip(dim).contiguous()


def window_forward(q, k, v, window_size, causal: bool = False, softmax_scale: Optional[float] = None,
                   out: Optional[torch.Tensor] = None, cu_seqlens=None, sink_tokens: int = 0,
                   q_offset: Optional[int] = None):
    """``q`` ``[B, S, H, D]``, ``k`` / ``v`` ``[B, Skv, Hkv, D]`` -> ``(o [B, S, H, D], lse [B, H, S] fp32)``.
    ``Skv > S``: the queries are the positions ``q_offset ... q_offset + S`` of the key sequence
    (default: the last ``S``).
    With ``cu_seqlens`` the token axis is a packed batch: sequence i spans ``cu_seqlens[i] :
    cu_seqlens[i + 1]``, attends only itself, and the window counts positions inside it.
    ``sink_tokens``: the first keys of every sequence that stay visible beyond the window."""
    B, S, H, D = q.shape
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    whole = _whole_sequence_plans(S, k.shape[1], window_size, causal, q.device, cu_seqlens, q_offset)
    if whole is not None:
        o = out if out is not None else torch.empty_like(q)
        o.zero_()
        lse = torch.full((B, H, S), float("-inf"), dtype=torch.float32, device=q.device)
        A.attn_fwd([q], [k], [v], [(o, lse)], whole[0], scale)
        return o, lse
    fplan, _ = _pick_plans(S, k.shape[1], window_size, causal, q.device, cu_seqlens, sink_tokens, q_offset)
    qr, kr, vr = _flip(q), _flip(k), _flip(v)
    o_a, o_b = torch.zeros_like(q), torch.zeros_like(q)
    lse_a = torch.full((B, H, S), float("-inf"), dtype=torch.float32, device=q.device)
    lse_b = torch.full_like(lse_a, float("-inf"))
    A.attn_fwd([q, qr], [k, kr], [v, vr], [(o_a, lse_a), (o_b, lse_b)], fplan, scale)
    o = out if out is not None else torch.empty_like(q)
    lse = torch.empty_like(lse_a)
    o_b, lse_b = _flip(o_b), _flip(lse_b, 2)
    for b in range(B):
        E.lse_merge([(o_a[b], lse_a[b]), (o_b[b], lse_b[b])], (o[b], lse[b]))
    return o, lse


def window_backward(d_o, q, k, v, o, lse, window_size, causal: bool = False,
                    softmax_scale: Optional[float] = None, softmax_d: Optional[torch.Tensor] = None,
                    cu_seqlens=None, sink_tokens: int = 0, q_offset: Optional[int] = None):
    """Gradients ``(dq, dk, dv)`` in the dtypes of ``q``, ``k``, ``v``. ``lse`` is the merged
    log-sum-exp the forward returned; with ``softmax_d`` (= rowsum(dO * O), ``[B, H, S]``) given,
    ``o`` is not read."""
    B, S, H, D = q.shape
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    q, k, v, d_o = q.contiguous(), k.contiguous(), v.contiguous(), d_o.contiguous()
    if softmax_d is None:
        softmax_d = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
        for b in range(B):
            E.rowdot(o[b], d_o[b], softmax_d[b])
    lse = lse.float().contiguous()
    softmax_d = softmax_d.float().contiguous()
    f32 = lambda t: torch.zeros(t.shape, dtype=torch.float32, device=t.device)
    whole = _whole_sequence_plans(S, k.shape[1], window_size, causal, q.device, cu_seqlens, q_offset)
    if whole is not None:
        dq32, kv = f32(q), A.BwdKvOut(f32(k), f32(v))
        A.attn_bwd([A.BwdQSide(q, d_o, lse, softmax_d, dq32)], [k], [v], [kv], whole[1], scale)
        return dq32.to(q.dtype), kv.dk.to(k.dtype), kv.dv.to(v.dtype)
    _, bplan = _pick_plans(S, k.shape[1], window_size, causal, q.device, cu_seqlens, sink_tokens, q_offset)
    dq_a, dq_b = f32(q), f32(q)
    kv_a, kv_b = A.BwdKvOut(f32(k), f32(v)), A.BwdKvOut(f32(k), f32(v))
    kv_outs = [kv_a, kv_b] + ([A.BwdKvOut(f32(k), f32(v))] if sink_tokens else [])     # slot 2: the sinks' share
    sides = [A.BwdQSide(q, d_o, lse, softmax_d, dq_a),
             A.BwdQSide(_flip(q), _flip(d_o), _flip(lse, 2), _flip(softmax_d, 2), dq_b)]
    A.attn_bwd(sides, [k, _flip(k)], [v, _flip(v)], kv_outs, bplan, scale)
    dq = (dq_a + dq_b.flip(1)).to(q.dtype)
    dk32, dv32 = kv_a.dk + kv_b.dk.flip(1), kv_a.dv + kv_b.dv.flip(1)
    if sink_tokens:
        dk32 += kv_outs[2].dk
        dv32 += kv_outs[2].dv
    return dq, dk32.to(k.dtype), dv32.to(v.dtype)


class _WindowFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, window_size, causal, softmax_scale, cu_seqlens=None, sink_tokens=0):
        cu = None if cu_seqlens is None else tuple(int(x) for x in cu_seqlens)
        o, lse = window_forward(q, k, v, window_size, causal, softmax_scale, cu_seqlens=cu, sink_tokens=sink_tokens)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.args = (tuple(window_size), bool(causal), softmax_scale, None, cu, int(sink_tokens))
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = window_backward(d_o, q, k, v, o, lse, *ctx.args)
        return dq, dk, dv, None, None, None, None, None


def sliding_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window_size=(-1, -1),
                             causal: bool = False, softmax_scale: Optional[float] = None,
                             cu_seqlens=None, sink_tokens: int = 0) -> torch.Tensor:
    """``softmax(mask(Q K^T) * scale) V`` with the band mask ``r - left <= c <= r + right``; autograd.
    ``cu_seqlens``: the token axis is a packed batch of sequences that attend only themselves.
    ``sink_tokens``: the first keys of every sequence stay visible to all later queries (attention
    sinks of streaming inference; at most one row block: ``min(256, left + 1)`` tokens).
    ``[batch, tokens, heads, head_dim]`` tensors (bf16 and head dim 128 on CUDA; any float type and
    head dim on CPU; a smaller head dim on CUDA runs zero-padded to 128 with the scale of the true
    head dim); grouped-query K / V allowed."""
    D = q.shape[-1]
    if q.is_cuda and D < A.KERNEL_HEAD_DIM:
        pad = A.KERNEL_HEAD_DIM - D
        scale = softmax_scale if softmax_scale is not None else D ** -0.5
        qp, kp, vp = (torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v))
        return _WindowFunction.apply(qp, kp, vp, tuple(window_size), causal, scale, cu_seqlens, sink_tokens)[..., :D]
    return _WindowFunction.apply(q, k, v, tuple(window_size), causal, softmax_scale, cu_seqlens, sink_tokens)
