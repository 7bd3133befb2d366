"""Ring-family context-parallel baselines on this framework's kernels: ring, zigzag ring, striped
ring (K/V travel around a ring of ranks, every rank keeps its queries) and Ulysses head-parallel
attention (all-to-all between sequence and head sharding).

Reference: ring_flash_attn/ring_flash_attn.py:7-135, zigzag_ring_flash_attn.py:78-283,
stripe_flash_attn.py:7-185, head_parallel_attn/deepspeed_ulysses_attn.py:10-198. The reference
merges partial outputs with a chain of PyTorch element-wise ops (and its zigzag merge is
short-circuited); here every step's kernel merges into the running (O, lse) in its epilogue, so
the results are numerically correct and there is no merge kernel. The striped variant needs no
slicing of Q / K: the kernels take the diagonal offset of the causal mask as a parameter.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import attention as A
from ..ops import elementwise as E
from .comm import A2AComm, RingComm


# per-step work: list of (q_start, q_len, [(k_start, k_len, causal, diag), ...]) or None to skip
def _ring_rule(step, rank, world, S, causal):
    if not causal:
        return [(0, S, [(0, S, False, 0)])]
    if step == 0:
        return [(0, S, [(0, S, True, 0)])]
    if step <= rank:
        return [(0, S, [(0, S, False, 0)])]
    return None


def _zigzag_rule(step, rank, world, S, causal):
    assert causal, "zigzag sharding is defined for causal attention"
    c = S // 2
    if step == 0:
        return [(0, c, [(0, c, True, 0)]), (c, c, [(0, c, False, 0), (c, c, True, 0)])]
    if step <= rank:
        return [(0, S, [(0, c, False, 0)])]
    return [(c, c, [(0, S, False, 0)])]


def _stripe_rule(step, rank, world, S, causal):
    assert causal, "striped sharding is defined for causal attention"
    # token t of the shard is global token t * world + rank; the K/V at this step come from rank
    # (rank - step) % world: visible iff k_global <= q_global
    return [(0, S, [(0, S, True, 0 if step <= rank else -1)])]


_RULES = {"ring": _ring_rule, "zigzag": _zigzag_rule, "stripe": _stripe_rule}


def _fwd_rows(work, started):
    return [A.Row(0, qs, ql, tuple(A.Seg(0, ks, kl, c, d) for ks, kl, c, d in segs), 0, qs, started)
            for qs, ql, segs in work]


def _bwd_cols(work, S):
    """Transpose a step's work into key-major form."""
    by_kv = {}
    for qs, ql, segs in work:
        for ks, kl, c, d in segs:
            by_kv.setdefault((ks, kl), []).append(A.Seg(0, qs, ql, c, d))
    return [A.Col(0, ks, kl, tuple(segs), 0, ks) for (ks, kl), segs in sorted(by_kv.items())]


def ring_forward(q, k, v, group, kind: str, causal: bool, softmax_scale=None):
    rule = _RULES[kind]
    comm = RingComm(group)
    S = q.shape[1]
    o = torch.zeros_like(q)
    lse = torch.full((q.shape[0], q.shape[2], S), float("-inf"), dtype=torch.float32, device=q.device)
    started = False
    for step in range(comm.world):
        if step + 1 != comm.world:
            nk, nv = comm.send_recv(k), comm.send_recv(v)
            comm.commit()
        work = rule(step, comm.rank, comm.world, S, causal)
        if work:
            A.attn_fwd([q], [k], [v], [(o, lse)], A.FwdPlan(_fwd_rows(work, started), q.device), softmax_scale)
            started = True
        if step + 1 != comm.world:
            comm.wait()
            k, v = nk, nv
    return o, lse


def ring_backward(d_o, q, k, v, o, lse, group, kind: str, causal: bool, softmax_scale=None):
    rule = _RULES[kind]
    kv_comm, g_comm = RingComm(group), RingComm(group)
    B, S, H, D = q.shape
    dvec = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    for b in range(B):
        E.rowdot(o[b], d_o[b], dvec[b])
    dq = torch.zeros(B, S, H, D, dtype=torch.float32, device=q.device)
    dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    side = A.BwdQSide(q, d_o, lse, dvec, dq)
    for step in range(kv_comm.world):
        last = step + 1 == kv_comm.world
        if not last:
            nk, nv = kv_comm.send_recv(k), kv_comm.send_recv(v)
            kv_comm.commit()
        work = rule(step, kv_comm.rank, kv_comm.world, S, causal)
        if work:
            A.attn_bwd([side], [k], [v], [A.BwdKvOut(dk, dv)], A.BwdPlan(_bwd_cols(work, S), q.device),
                       softmax_scale)
        # the gradient buffers travel with their K/V block; after the last step one more hop
        # brings them home
        ndk, ndv = g_comm.send_recv(dk), g_comm.send_recv(dv)
        g_comm.commit()
        if not last:
            kv_comm.wait()
            k, v = nk, nv
        g_comm.wait()
        dk, dv = ndk, ndv
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


class _RingFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, group, kind):
        o, lse = ring_forward(q, k, v, group, kind, causal, softmax_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.args = (softmax_scale, causal, group, kind)
        return o, lse

    @staticmethod
    def backward(ctx, d_o, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, group, kind = ctx.args
        dq, dk, dv = ring_backward(d_o.contiguous(), q, k, v, o, lse, group, kind, causal, scale)
        return dq, dk, dv, None, None, None, None


def _make_func(kind: str):
    def func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
             alibi_slopes=None, deterministic=False, return_attn_probs=False, group=None,
             PROC_INFO=None, opt=False):
        assert dropout_p == 0.0 and alibi_slopes is None and tuple(window_size) == (-1, -1), \
            "dropout, alibi and sliding windows are not part of these baselines"
        o, lse = _RingFunc.apply(q, k, v, softmax_scale, causal, group, kind)
        return (o, lse, None) if return_attn_probs else o
    func.__name__ = f"{kind}_flash_attn_func"
    func.__doc__ = (f"{kind} context-parallel attention: q, k, v are this rank's shard "
                    "[batch, tokens, heads, head_dim]; same signature as the reference's function.")
    return func


ring_flash_attn_func = _make_func("ring")
zigzag_ring_flash_attn_func = _make_func("zigzag")
stripe_flash_attn_func = _make_func("stripe")


def _packed(func, n):
    def f(packed, *a, **kw):
        parts = packed.unbind(dim=2)
        return func(*parts, *a, **kw) if n == 3 else None
    return f


def ring_flash_attn_qkvpacked_func(qkv, *a, **kw):
    return ring_flash_attn_func(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], *a, **kw)


def ring_flash_attn_kvpacked_func(q, kv, *a, **kw):
    return ring_flash_attn_func(q, kv[:, :, 0], kv[:, :, 1], *a, **kw)


def zigzag_ring_flash_attn_qkvpacked_func(qkv, *a, **kw):
    return zigzag_ring_flash_attn_func(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], *a, **kw)


def zigzag_ring_flash_attn_kvpacked_func(q, kv, *a, **kw):
    return zigzag_ring_flash_attn_func(q, kv[:, :, 0], kv[:, :, 1], *a, **kw)


def stripe_flash_attn_qkvpacked_func(qkv, *a, **kw):
    return stripe_flash_attn_func(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], *a, **kw)


def stripe_flash_attn_kvpacked_func(q, kv, *a, **kw):
    return stripe_flash_attn_func(q, kv[:, :, 0], kv[:, :, 1], *a, **kw)


# -------------------------------------------------------------------------------------------------
# input sharding helpers (reference: easy_context/zigzag_ring_attn/prepare_inputs.py:4-40)
# -------------------------------------------------------------------------------------------------
def shard_sequence(x: torch.Tensor, rank: int, world: int, kind: str, dim: int = 1) -> torch.Tensor:
    """This rank's shard of a full-sequence tensor under the layout each strategy expects."""
    if kind == "ring" or kind == "ulysses":
        return x.chunk(world, dim=dim)[rank].contiguous()
    if kind == "zigzag":
        ch = x.chunk(2 * world, dim=dim)
        return torch.cat([ch[rank], ch[2 * world - 1 - rank]], dim=dim).contiguous()
    if kind == "stripe":
        idx = torch.arange(rank, x.shape[dim], world, device=x.device)
        return x.index_select(dim, idx).contiguous()
    raise ValueError(kind)


# -------------------------------------------------------------------------------------------------
# Ulysses
# -------------------------------------------------------------------------------------------------
class _UlyssesFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, group):
        from ..api import local_plans
        from ..patterns import named
        a2a = A2AComm(group)
        qh, kh, vh = (a2a.all_to_all(t, 2, 1) for t in (q, k, v))       # [B, S, H/sp, D]
        pat = named.causal(1) if causal else named.full(1)
        fplan, bplan = local_plans(pat, qh.shape[1], qh.device)
        oh = torch.empty_like(qh)
        lse = torch.empty(qh.shape[0], qh.shape[2], qh.shape[1], dtype=torch.float32, device=qh.device)
        A.attn_fwd([qh], [kh], [vh], [(oh, lse)], fplan, softmax_scale)
        ctx.save_for_backward(qh, kh, vh, oh, lse)
        ctx.args = (softmax_scale, group, bplan)
        return a2a.all_to_all(oh, 1, 2)

    @staticmethod
    def backward(ctx, d_o):
        from ..api import local_backward
        qh, kh, vh, oh, lse = ctx.saved_tensors
        scale, group, bplan = ctx.args
        a2a = A2AComm(group)
        doh = a2a.all_to_all(d_o.contiguous(), 2, 1)
        dq, dk, dv = local_backward(qh, kh, vh, oh, lse, doh, bplan, scale)
        return tuple(a2a.all_to_all(t, 1, 2) for t in (dq, dk, dv)) + (None, None, None)


def deepspeed_ulysses_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                                window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                                return_attn_probs=False, group=None, PROC_INFO=None):
    """Head-parallel attention: inputs are sequence shards ``[B, S/sp, H, D]``; an all-to-all
    re-shards to ``[B, S, H/sp, D]``, attention runs on whole sequences, a second all-to-all
    restores the sequence sharding. (The reference's version is a stub whose compute step is
    missing, head_parallel_attn/deepspeed_ulysses_attn.py:43-47.)"""
    assert dropout_p == 0.0 and alibi_slopes is None
    return _UlyssesFunc.apply(q, k, v, softmax_scale, causal, group)
