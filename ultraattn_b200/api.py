"""The differentiable entry point: ``attention(q, k, v, pattern, ...)``.

On one GPU it runs the block-sparse forward / backward kernels directly. With a process group it
runs context-parallel: every rank passes its shard of the sequence and gets its shard of the
output, and gradients flow back the same way. The reference exposes ``orchestrated_attn_func``
with a forward that returns nothing and a backward that asserts
(orchestrated_attn/orchestrated_attn_impl.py:688-792); this is the operator it was meant to be.
"""
from __future__ import annotations

from typing import Optional

import torch

from .ops import attention as A
from .ops import elementwise as E
from .patterns.blocks import BSA_Repr

_plan_cache: dict = {}


def local_plans(pattern: BSA_Repr, seq_len: int, device) -> tuple:
    """(FwdPlan, BwdPlan) for the whole pattern on one device, cached."""
    key = (str(pattern), pattern.block_table_int.shape, seq_len, str(device))
    if key not in _plan_cache:
        tab = pattern.block_table_int
        n = tab.shape[0]
        assert seq_len % n == 0, f"sequence length {seq_len} is not a multiple of {n} blocks"
        blk = seq_len // n
        _plan_cache[key] = (A.FwdPlan(A.rows_from_block_table(tab, blk), device),
                            A.BwdPlan(A.cols_from_block_table(tab, blk), device))
    return _plan_cache[key]


class _LocalAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, pattern, softmax_scale):
        fplan, bplan = local_plans(pattern, q.shape[1], q.device)
        o = torch.empty_like(q)
        lse = torch.empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32, device=q.device)
        A.attn_fwd([q], [k], [v], [(o, lse)], fplan, softmax_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.bplan = bplan
        ctx.scale = softmax_scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = local_backward(q, k, v, o, lse, d_o.contiguous(), ctx.bplan, ctx.scale)
        return dq, dk, dv, None, None


def local_backward(q, k, v, o, lse, d_o, bplan, softmax_scale=None):
    """dQ, dK, dV of the single-device operator (bf16 on CUDA, input dtype on CPU)."""
    B, S, H, D = q.shape
    dvec = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    for b in range(B):
        E.rowdot(o[b], d_o[b], dvec[b])
    dq32 = torch.zeros(B, S, H, D, dtype=torch.float32, device=q.device)
    if q.is_cuda:
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
    else:
        dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
        dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    A.attn_bwd([A.BwdQSide(q, d_o, lse, dvec, dq32)], [k], [v], [A.BwdKvOut(dk, dv)], bplan, softmax_scale)
    if q.is_cuda:
        dq = torch.empty_like(q)
        E.cast_scale(dq32, dq)
        return dq, dk, dv
    return dq32.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pattern: BSA_Repr, *,
              softmax_scale: Optional[float] = None, runtime=None) -> torch.Tensor:
    """Block-sparse attention ``softmax(mask(Q K^T) * scale) V`` with autograd.

    ``q, k, v``: ``[batch, tokens, heads, head_dim]`` (bf16 on CUDA, head_dim 128 native and smaller
    head dims zero-padded to it; any float type and head dim on CPU). Without ``runtime`` the tensors hold the whole sequence and the call
    runs on this device alone. With a :class:`ultraattn_b200.runtime.ContextParallelAttention`
    (``runtime=``) they hold this rank's shard and the call is context-parallel over its group.
    """
    if runtime is not None:
        return runtime(q, k, v, softmax_scale)
    D = q.shape[-1]
    if q.is_cuda and D < A.KERNEL_HEAD_DIM:
        # The kernels are built for head dim 128. A smaller head dim runs zero-padded: the padding
        # adds nothing to Q K^T, the padded output columns are zero and are cut off again, and
        # autograd drops the padding's gradients (the scale stays that of the true head dim).
        # Correct, at the cost of the 128-wide tiles.
        pad = A.KERNEL_HEAD_DIM - D
        scale = softmax_scale if softmax_scale is not None else D ** -0.5
        qp, kp, vp = (torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v))
        return _LocalAttention.apply(qp, kp, vp, pattern, scale)[..., :D]
    return _LocalAttention.apply(q, k, v, pattern, softmax_scale)


# -------------------------------------------------------------------------------------------------
# variable-length (packed) sequences
# -------------------------------------------------------------------------------------------------
def varlen_plans(cu_seqlens, causal: bool, device):
    """Launch plans for a packed batch: sequence i occupies tokens cu_seqlens[i]..cu_seqlens[i+1]
    of the packed [1, T, H, D] tensors and attends only itself (the document mask). This is the
    role of the reference's ``_flash_attn_varlen_forward/backward`` call sites
    (ring_flash_attn/ring_flash_attn_varlen.py:50-64, 116-137); no separate kernel is needed because
    the kernels already take a list of (query block, key segments) work items."""
    cu = [int(x) for x in cu_seqlens]
    key = ("varlen", tuple(cu), causal, str(device))
    if key not in _plan_cache:
        rows, cols = [], []
        for a, b in zip(cu[:-1], cu[1:]):
            if b > a:
                rows.append(A.Row(0, a, b - a, (A.Seg(0, a, b - a, causal, 0),), 0, a, False))
                cols.append(A.Col(0, a, b - a, (A.Seg(0, a, b - a, causal, 0),), 0, a))
        _plan_cache[key] = (A.FwdPlan(rows, device), A.BwdPlan(cols, device))
    return _plan_cache[key]


class _VarlenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, causal, softmax_scale):
        fplan, bplan = varlen_plans(cu_seqlens, causal, q.device)
        o = torch.zeros_like(q)
        lse = torch.full((q.shape[0], q.shape[2], q.shape[1]), float("-inf"), dtype=torch.float32, device=q.device)
        A.attn_fwd([q], [k], [v], [(o, lse)], fplan, softmax_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.bplan, ctx.scale = bplan, softmax_scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = local_backward(q, k, v, o, lse, d_o.contiguous(), ctx.bplan, ctx.scale)
        return dq, dk, dv, None, None, None


class _PlannedAttention(torch.autograd.Function):
    """Attention under a token-level launch plan (forward rows, backward columns) on one buffer."""

    @staticmethod
    def forward(ctx, q, k, v, fplan, bplan, softmax_scale):
        o = torch.zeros_like(q)
        lse = torch.full((q.shape[0], q.shape[2], q.shape[1]), float("-inf"), dtype=torch.float32, device=q.device)
        A.attn_fwd([q], [k], [v], [(o, lse)], fplan, softmax_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.bplan, ctx.scale = bplan, softmax_scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = local_backward(q, k, v, o, lse, d_o.contiguous(), ctx.bplan, ctx.scale)
        return dq, dk, dv, None, None, None


def prefix_lm_plans(seq_len: int, prefix_length: int, device, cu_seqlens=None):
    """Launch plans of the prefix-LM mask: the first ``prefix_length`` tokens of a sequence attend
    each other in both directions, every later token attends causally (and so sees the whole
    prefix). Token-exact on the block-sparse kernels: the prefix is one fully visible work item, the
    rest one causal item whose diagonal is shifted by the prefix. With ``cu_seqlens`` every
    sequence of the packed buffer has its own prefix (clipped to its length)."""
    bounds = [(0, seq_len)] if cu_seqlens is None else list(zip([int(x) for x in cu_seqlens][:-1],
                                                                 [int(x) for x in cu_seqlens][1:]))
    key = ("prefix_lm", tuple(bounds), int(prefix_length), str(device))
    if key not in _plan_cache:
        rows, cols = [], []
        for a, b in bounds:
            n = b - a
            p = max(0, min(int(prefix_length), n))
            if p > 0:
                rows.append(A.Row(0, a, p, (A.Seg(0, a, p, False, 0),), 0, a, False))
                cols.append(A.Col(0, a, p, (A.Seg(0, a, n, False, 0),), 0, a))          # every token sees the prefix
            if n > p:
                rows.append(A.Row(0, a + p, n - p, (A.Seg(0, a, n, True, p),), 0, a + p, False))
                cols.append(A.Col(0, a + p, n - p, (A.Seg(0, a + p, n - p, True, 0),), 0, a + p))
        _plan_cache[key] = (A.FwdPlan(rows, device), A.BwdPlan(cols, device))
    return _plan_cache[key]


def prefix_lm_attention(q, k, v, prefix_length: int, softmax_scale: Optional[float] = None, cu_seqlens=None):
    """Attention under the prefix-LM mask, with autograd. ``[batch, tokens, heads, head_dim]`` (or
    packed ``[tokens, heads, head_dim]``); same dtype / head-dim rules as :func:`attention`."""
    squeeze = q.dim() == 3
    if squeeze:
        q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
    D = q.shape[-1]
    fplan, bplan = prefix_lm_plans(q.shape[1], prefix_length, q.device, cu_seqlens)
    if q.is_cuda and D < A.KERNEL_HEAD_DIM:
        pad = A.KERNEL_HEAD_DIM - D
        scale = softmax_scale if softmax_scale is not None else D ** -0.5
        qp, kp, vp = (torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v))
        o = _PlannedAttention.apply(qp, kp, vp, fplan, bplan, scale)[..., :D]
    else:
        o = _PlannedAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), fplan, bplan, softmax_scale)
    return o.squeeze(0) if squeeze else o


def varlen_attention(q, k, v, cu_seqlens, causal: bool = True, softmax_scale: Optional[float] = None,
                     window_size=(-1, -1)):
    """Attention over a packed batch ``[total_tokens, heads, head_dim]`` (or with a leading batch
    dimension of 1) where ``cu_seqlens`` gives the sequence boundaries. ``window_size = (left,
    right)`` restricts every query to a band of its own sequence (``ops/window.py``)."""
    squeeze = q.dim() == 3
    if squeeze:
        q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
    if tuple(int(x) for x in window_size) != (-1, -1):
        from .ops.window import sliding_window_attention
        o = sliding_window_attention(q, k, v, window_size, causal, softmax_scale, cu_seqlens=cu_seqlens)
    else:
        o = _VarlenAttention.apply(q, k, v, tuple(int(x) for x in cu_seqlens), causal, softmax_scale)
    return o.squeeze(0) if squeeze else o
