"""The kernel-level calling convention of the reference, on this framework's kernels.

The reference runtime and its ring baselines call a forked flash-attention through four private
functions (orchestrated_attn/orchestrated_attn_impl.py:326-337, 578-596;
ring_flash_attn/ring_flash_attn.py:33-43, 91-108; ring_flash_attn_varlen.py:50-64, 116-137):

    _flash_attn_forward(q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                        return_softmax, out=None) -> (out, q, k, v, out_padded, softmax_lse, S_dmask, rng_state)
    _flash_attn_backward(dout, q, k, v, out, softmax_lse, dq, dk, dv, dropout_p, softmax_scale,
                         causal, window_size, alibi_slopes, deterministic, rng_state=None, softmax_d=None)
    _flash_attn_varlen_forward / _flash_attn_varlen_backward  (packed batches with cu_seqlens)

The fork's two additions are kept: ``out=`` lets the caller name the output buffer, and
``softmax_d=`` passes a precomputed ``D = rowsum(dO * O)`` so that O itself need not be present
(``out`` may then be any tensor of the right shape, as in the reference, which passes Q).
Code written against those calls runs on the sm_100a kernels (CUDA tensors, bf16, head dim 128) or
on the fp32 restatement (CPU tensors) by importing them from here. Sliding windows
(``window_size = (left, right)``) run on the same kernels for ``Sq <= Skv`` (``ops/window.py``: the
band is split into a part in the usual token order and a part in reversed order, each of which
needs a one-sided mask only). Dropout and ALiBi are not supported (the reference never uses them:
``dropout_p = 0``, ``alibi_slopes = None`` at every call site, and ``window_size = (-1, -1)``).
With ``Sq != Skv`` a causal mask is aligned to the bottom-right corner, as in flash-attention 2.1
and later. The varlen calls take windows when every sequence has as many keys as queries.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import attention as A
from . import elementwise as E
from . import window as W


def _check(dropout_p, window_size, alibi_slopes, windows_ok: bool = False):
    assert dropout_p == 0.0, "dropout is not supported"
    assert alibi_slopes is None, "ALiBi is not supported"
    assert windows_ok or tuple(window_size) == (-1, -1), "sliding windows are not supported by this call"


def _windowed(window_size) -> bool:
    return tuple(int(x) for x in window_size) != (-1, -1)


def _scale(q, softmax_scale):
    return softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])


def _forward(q, k, v, rows, out, softmax_scale):
    o = out if out is not None else torch.empty_like(q)
    o.zero_()
    lse = torch.full((q.shape[0], q.shape[2], q.shape[1]), float("-inf"), dtype=torch.float32, device=q.device)
    A.attn_fwd([q], [k], [v], [(o, lse)], A.FwdPlan(rows, q.device), softmax_scale)
    return o, lse


def _backward(dout, q, k, v, out, lse, dq, dk, dv, cols, softmax_scale, softmax_d):
    B, S, H, D = q.shape
    if softmax_d is None:
        softmax_d = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
        for b in range(B):
            E.rowdot(out[b], dout[b], softmax_d[b])
    dq32 = torch.zeros(B, S, H, D, dtype=torch.float32, device=q.device)
    if q.is_cuda:
        dkv = A.BwdKvOut(dk, dv)                   # bf16 destinations are written directly
    else:
        dkv = A.BwdKvOut(torch.zeros(k.shape, dtype=torch.float32), torch.zeros(v.shape, dtype=torch.float32))
    A.attn_bwd([A.BwdQSide(q, dout.contiguous(), lse, softmax_d.float(), dq32)], [k], [v], [dkv],
               A.BwdPlan(cols, q.device), softmax_scale)
    if q.is_cuda:
        E.cast_scale(dq32, dq)
    else:
        dq.copy_(dq32.to(dq.dtype))
        dk.copy_(dkv.dk.to(dk.dtype))
        dv.copy_(dkv.dv.to(dv.dtype))
    return softmax_d


def _flash_attn_forward(q, k, v, dropout_p, softmax_scale, causal, window_size=(-1, -1), alibi_slopes=None,
                        return_softmax=False, out: Optional[torch.Tensor] = None):
    """``q`` ``[B, Sq, H, D]``, ``k`` / ``v`` ``[B, Skv, Hkv, D]``. Returns the fork's 8-tuple
    ``(out, q, k, v, out_padded, softmax_lse [B, H, Sq] fp32, S_dmask (None), rng_state (None))``."""
    _check(dropout_p, window_size, alibi_slopes, windows_ok=True)
    sq, skv = q.shape[1], k.shape[1]
    if _windowed(window_size):
        o, lse = W.window_forward(q, k, v, window_size, bool(causal), _scale(q, softmax_scale), out)
        return o, q, k, v, o, lse, None, None
    rows = [A.Row(0, 0, sq, (A.Seg(0, 0, skv, bool(causal), skv - sq),), 0, 0, False)]
    o, lse = _forward(q, k, v, rows, out, _scale(q, softmax_scale))
    return o, q, k, v, o, lse, None, None


def _flash_attn_backward(dout, q, k, v, out, softmax_lse, dq, dk, dv, dropout_p, softmax_scale, causal,
                         window_size=(-1, -1), alibi_slopes=None, deterministic=False, rng_state=None,
                         softmax_d: Optional[torch.Tensor] = None):
    """Writes ``dq``, ``dk``, ``dv`` in place; returns ``(dq, dk, dv, softmax_d)``. With
    ``softmax_d`` given, ``out`` is not read."""
    _check(dropout_p, window_size, alibi_slopes, windows_ok=True)
    sq, skv = q.shape[1], k.shape[1]
    if _windowed(window_size):
        if softmax_d is None:
            softmax_d = torch.empty(q.shape[0], q.shape[2], sq, dtype=torch.float32, device=q.device)
            for b in range(q.shape[0]):
                E.rowdot(out[b], dout[b], softmax_d[b])
        g = W.window_backward(dout, q, k, v, out, softmax_lse, window_size, bool(causal), _scale(q, softmax_scale),
                              softmax_d)
        for dst, src in zip((dq, dk, dv), g):
            dst.copy_(src)
        return dq, dk, dv, softmax_d
    cols = [A.Col(0, 0, skv, (A.Seg(0, 0, sq, bool(causal), skv - sq),), 0, 0)]
    d = _backward(dout, q, k, v, out, softmax_lse, dq, dk, dv, cols, _scale(q, softmax_scale), softmax_d)
    return dq, dk, dv, d


def _bounds(cu):
    cu = [int(c) for c in cu]
    return list(zip(cu[:-1], cu[1:]))


def _pad_lse(lse_packed, cu_q, max_seqlen_q):
    """packed [H, T] -> padded [n_seq, H, max_seqlen] (the layout of flash-attention 2.5)."""
    bq = _bounds(cu_q)
    out = torch.zeros(len(bq), lse_packed.shape[0], max_seqlen_q, dtype=torch.float32, device=lse_packed.device)
    for i, (a, b) in enumerate(bq):
        out[i, :, :b - a] = lse_packed[:, a:b]
    return out


def _flash_attn_varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
                               softmax_scale, causal, window_size=(-1, -1), alibi_slopes=None,
                               return_softmax=False, block_table=None, out: Optional[torch.Tensor] = None):
    """Packed batch: ``q`` ``[Tq, H, D]``, ``k`` / ``v`` ``[Tk, Hkv, D]``; sequence i spans
    ``cu_seqlens[i] : cu_seqlens[i + 1]`` and attends only itself. Returns the 8-tuple with
    ``softmax_lse`` padded ``[n_seq, H, max_seqlen_q]``."""
    _check(dropout_p, window_size, alibi_slopes, windows_ok=True)
    assert block_table is None, "paged key/value caches are not supported"
    if _windowed(window_size):
        assert _bounds(cu_seqlens_q) == _bounds(cu_seqlens_k), "sliding windows need equal query and key lengths"
        o, lse = W.window_forward(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), window_size, bool(causal),
                                  _scale(q, softmax_scale), out.unsqueeze(0) if out is not None else None,
                                  cu_seqlens=cu_seqlens_q)
        o = o.squeeze(0)
        return o, q, k, v, o, _pad_lse(lse[0], cu_seqlens_q, max_seqlen_q), None, None
    rows = []
    for (qa, qb), (ka, kb) in zip(_bounds(cu_seqlens_q), _bounds(cu_seqlens_k)):
        if qb > qa and kb > ka:
            rows.append(A.Row(0, qa, qb - qa, (A.Seg(0, ka, kb - ka, bool(causal), (kb - ka) - (qb - qa)),), 0, qa, False))
    o, lse = _forward(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), rows,
                      out.unsqueeze(0) if out is not None else None, _scale(q, softmax_scale))
    o = o.squeeze(0)
    return o, q, k, v, o, _pad_lse(lse[0], cu_seqlens_q, max_seqlen_q), None, None


def _flash_attn_varlen_backward(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                                max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal,
                                window_size=(-1, -1), alibi_slopes=None, deterministic=False, rng_state=None,
                                softmax_d: Optional[torch.Tensor] = None):
    """``softmax_lse``: padded ``[n_seq, H, max_seqlen_q]`` (as returned by the forward) or packed
    ``[H, Tq]``. Writes ``dq``, ``dk``, ``dv`` (packed) in place."""
    _check(dropout_p, window_size, alibi_slopes, windows_ok=True)
    bq, bk = _bounds(cu_seqlens_q), _bounds(cu_seqlens_k)
    if softmax_lse.dim() == 3:
        lse = torch.cat([softmax_lse[i, :, :b - a] for i, (a, b) in enumerate(bq)], dim=1)
    else:
        lse = softmax_lse
    if _windowed(window_size):
        assert bq == bk, "sliding windows need equal query and key lengths"
        if softmax_d is None:
            softmax_d = E.rowdot(out, dout)
        g = W.window_backward(dout.unsqueeze(0), q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), out.unsqueeze(0),
                              lse.unsqueeze(0), window_size, bool(causal), _scale(q, softmax_scale),
                              softmax_d.unsqueeze(0), cu_seqlens=cu_seqlens_q)
        for dst, src in zip((dq, dk, dv), g):
            dst.copy_(src[0])
        return dq, dk, dv, softmax_d
    cols = []
    for (qa, qb), (ka, kb) in zip(bq, bk):
        if qb > qa and kb > ka:
            cols.append(A.Col(0, ka, kb - ka, (A.Seg(0, qa, qb - qa, bool(causal), (kb - ka) - (qb - qa)),), 0, ka))
    dk.zero_()          # keys of empty sequences belong to no work item
    dv.zero_()
    d = _backward(dout.unsqueeze(0), q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), out.unsqueeze(0),
                  lse.unsqueeze(0).contiguous(), dq.unsqueeze(0), dk.unsqueeze(0), dv.unsqueeze(0), cols,
                  _scale(q, softmax_scale), None if softmax_d is None else softmax_d.unsqueeze(0))
    return dq, dk, dv, d.squeeze(0)


# -------------------------------------------------------------------------------------------------
# The public calling convention of flash-attention (flash_attn_func and its packed / varlen forms),
# with autograd, for code that used the library directly (the reference's benchmark scripts and
# LightSeq checks do: bench_ring_attn_old.py:2, easy_context/dist_flash_attn/lightseq_async_attn.py:547).
# -------------------------------------------------------------------------------------------------
class _FlashFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, window_size):
        out = _flash_attn_forward(q, k, v, 0.0, softmax_scale, causal, window_size)
        ctx.save_for_backward(q, k, v, out[0], out[5])
        ctx.args = (softmax_scale, causal, tuple(window_size))
        ctx.mark_non_differentiable(out[5])
        return out[0], out[5]

    @staticmethod
    def backward(ctx, d_o, _d_lse):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, window = ctx.args
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_attn_backward(d_o.contiguous(), q, k, v, o, lse, dq, dk, dv, 0.0, scale, causal, window)
        return dq, dk, dv, None, None, None


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                    alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """``q`` ``[B, Sq, H, D]``, ``k`` / ``v`` ``[B, Skv, Hkv, D]`` -> ``out`` (or ``(out, lse, None)``
    with ``return_attn_probs``); differentiable. Same dtype / head-dim rules as the private calls."""
    _check(dropout_p, window_size, alibi_slopes, windows_ok=True)
    o, lse = _FlashFunc.apply(q.contiguous(), k.contiguous(), v.contiguous(), softmax_scale, bool(causal),
                              tuple(window_size))
    return (o, lse, None) if return_attn_probs else o


def flash_attn_qkvpacked_func(qkv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                              alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """``qkv`` ``[B, S, 3, H, D]``."""
    return flash_attn_func(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], dropout_p, softmax_scale, causal, window_size,
                           alibi_slopes, deterministic, return_attn_probs)


def flash_attn_kvpacked_func(q, kv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                             alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """``q`` ``[B, Sq, H, D]``, ``kv`` ``[B, Skv, 2, Hkv, D]``."""
    return flash_attn_func(q, kv[:, :, 0], kv[:, :, 1], dropout_p, softmax_scale, causal, window_size,
                           alibi_slopes, deterministic, return_attn_probs)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q=None, max_seqlen_k=None,
                           dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                           alibi_slopes=None, deterministic=False, return_attn_probs=False, block_table=None):
    """Packed batch ``[tokens, heads, head_dim]``; every sequence has as many keys as queries."""
    from ..api import varlen_attention
    _check(dropout_p, window_size, alibi_slopes, windows_ok=True)
    assert block_table is None, "paged key/value caches are not supported"
    assert _bounds(cu_seqlens_q) == _bounds(cu_seqlens_k), "the differentiable varlen form needs equal query and key lengths"
    assert not return_attn_probs, "use _flash_attn_varlen_forward for the log-sum-exp"
    return varlen_attention(q, k, v, cu_seqlens_q, bool(causal), softmax_scale, window_size)
