"""The reference's kernel-level calls (forked flash-attention signatures) on the fp32 restatement."""
import math

import torch

from ultraattn_b200.ops.flash_compat import (_flash_attn_backward, _flash_attn_forward,
                                             _flash_attn_varlen_backward, _flash_attn_varlen_forward)


def _dense(q, k, v, d_o, causal):
    """[S, H, D] tensors; grouped-query heads repeated; bottom-right aligned causal mask."""
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    g = q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(q.shape[-1])
    if causal:
        sq, sk = q.shape[0], k.shape[0]
        mask = torch.arange(sk)[None, :] <= torch.arange(sq)[:, None] + (sk - sq)
        s = s.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv)
    o.backward(d_o)
    return o.detach(), lse.detach(), q.grad, k.grad, v.grad


def test_dense_calls_with_out_and_softmax_d():
    torch.manual_seed(0)
    Sq, Skv, H, Hk, D = 48, 80, 4, 2, 16
    q, d_o = torch.randn(1, Sq, H, D), torch.randn(1, Sq, H, D)
    k, v = torch.randn(1, Skv, Hk, D), torch.randn(1, Skv, Hk, D)
    for causal in (False, True):
        o_ref, lse_ref, dq_ref, dk_ref, dv_ref = _dense(q[0], k[0], v[0], d_o[0], causal)
        buf = torch.full_like(q, 7.0)
        ret = _flash_attn_forward(q, k, v, 0.0, None, causal, window_size=(-1, -1), alibi_slopes=None,
                                  return_softmax=False, out=buf)
        assert len(ret) == 8 and ret[0] is buf and ret[6] is None
        assert torch.allclose(buf[0], o_ref, atol=1e-5) and torch.allclose(ret[5][0], lse_ref, atol=1e-5)
        # the fork's way: D precomputed, a dummy tensor in place of O
        dvec = (o_ref * d_o[0]).sum(-1).t()[None].contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_attn_backward(d_o, q, k, v, q, ret[5], dq, dk, dv, 0.0, None, causal, (-1, -1), None, False,
                             rng_state=None, softmax_d=dvec)
        assert torch.allclose(dq[0], dq_ref, atol=1e-5) and torch.allclose(dk[0], dk_ref, atol=1e-5)
        assert torch.allclose(dv[0], dv_ref, atol=1e-5)
        # the stock way: D derived from O
        dq2, dk2, dv2 = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_attn_backward(d_o, q, k, v, buf, ret[5], dq2, dk2, dv2, 0.0, None, causal)
        assert torch.allclose(dq2, dq, atol=1e-6) and torch.allclose(dk2, dk, atol=1e-6)


def test_varlen_calls():
    torch.manual_seed(1)
    H, D = 2, 16
    cu = [0, 24, 24, 64, 72]
    T = cu[-1]
    q, k, v, d_o = (torch.randn(T, H, D) for _ in range(4))
    max_len = max(b - a for a, b in zip(cu[:-1], cu[1:]))
    ret = _flash_attn_varlen_forward(q, k, v, cu, cu, max_len, max_len, 0.0, None, True)
    o, lse = ret[0], ret[5]
    assert lse.shape == (len(cu) - 1, H, max_len)
    dq, dk, dv = torch.empty_like(q), torch.full_like(k, 3.0), torch.full_like(v, 3.0)
    _flash_attn_varlen_backward(d_o, q, k, v, o, lse, dq, dk, dv, cu, cu, max_len, max_len, 0.0, None, True)
    for i, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        if b == a:
            continue
        o_ref, lse_ref, dq_ref, dk_ref, dv_ref = _dense(q[a:b], k[a:b], v[a:b], d_o[a:b], True)
        assert torch.allclose(o[a:b], o_ref, atol=1e-5) and torch.allclose(lse[i, :, :b - a], lse_ref, atol=1e-5)
        assert torch.allclose(dq[a:b], dq_ref, atol=1e-5) and torch.allclose(dk[a:b], dk_ref, atol=1e-5)
        assert torch.allclose(dv[a:b], dv_ref, atol=1e-5)


def test_plan_restatement_matches_explicit_masks_property():
    """Property test of the fp32 restatement of the launch plans (the oracle of the GPU kernels):
    random query blocks with random key segments (offsets, lengths, causal diagonals) against an
    explicit token mask, forward and backward."""
    from hypothesis import given, settings, strategies as st
    from ultraattn_b200.ops import attention as A

    @st.composite
    def rows(draw):
        T = 48
        out, used = [], 0
        for _ in range(draw(st.integers(1, 3))):
            q_len = draw(st.integers(1, 12))
            if used + q_len > T:
                break
            segs = []
            for _ in range(draw(st.integers(1, 3))):
                start = draw(st.integers(0, T - 1))
                length = draw(st.integers(1, T - start))
                segs.append(A.Seg(0, start, length, draw(st.booleans()), draw(st.integers(-3, 3))))
            out.append(A.Row(0, used, q_len, tuple(segs), 0, used, False))
            used += q_len
        return out

    @settings(max_examples=40, deadline=None, derandomize=True)
    @given(rows())
    def check(rws):
        if not rws:
            return
        torch.manual_seed(0)
        T, H, D = 48, 2, 8
        q, k, v, d_o = (torch.randn(1, T, H, D) for _ in range(4))
        o = torch.zeros(1, T, H, D)
        lse = torch.full((1, H, T), float("-inf"))
        A.attn_fwd_reference([q], [k], [v], [(o, lse)], rws)
        # explicit: every row attends the concatenation of its segments (a key may appear twice)
        q_, k_, v_ = (t.clone().requires_grad_() for t in (q, k, v))
        o_ref = torch.zeros(1, T, H, D)
        for r in rws:
            idx, keep = [], []
            for s in r.segs:
                for c in range(s.length):
                    idx.append(s.start + c)
                    keep.append([(not s.causal) or c <= rr + s.diag for rr in range(r.q_len)])
            ks, vs = k_[0, idx], v_[0, idx]
            sc = torch.einsum("qhd,khd->hqk", q_[0, r.q_start:r.q_start + r.q_len], ks) / math.sqrt(D)
            mask = torch.tensor(keep).t()
            sc = sc.masked_fill(~mask[None], float("-inf"))
            p = torch.softmax(sc, -1)
            p = torch.where(torch.isnan(p), torch.zeros_like(p), p)
            o_ref[0, r.q_start:r.q_start + r.q_len] = torch.einsum("hqk,khd->qhd", p, vs)
        assert torch.allclose(o, o_ref.detach(), atol=1e-5)
        # backward of the restatement against autograd of the explicit form
        o_ref.backward(d_o)
        dvec = (o * d_o).sum(-1).permute(0, 2, 1).contiguous()
        dq = torch.zeros(1, T, H, D)
        by_kv = {}
        for r in rws:
            for s in r.segs:
                by_kv.setdefault((s.start, s.length), []).append(A.Seg(0, r.q_start, r.q_len, s.causal, s.diag))
        cols = [A.Col(0, ks_, kl_, tuple(sg), 0, ks_) for (ks_, kl_), sg in by_kv.items()]
        dk, dv = torch.zeros(1, T, H, D), torch.zeros(1, T, H, D)
        A.attn_bwd_reference([A.BwdQSide(q, d_o, lse, dvec, dq)], [k], [v], [A.BwdKvOut(dk, dv)], cols)
        assert torch.allclose(dq, q_.grad, atol=1e-4) and torch.allclose(dk, k_.grad, atol=1e-4)
        assert torch.allclose(dv, v_.grad, atol=1e-4)

    check()


def test_launch_order_keeps_groups_together_heaviest_first():
    """Launch order of a table-driven launch: a permutation of the tiles in which the tiles of one
    block row (column) are adjacent, rows ordered by their heaviest tile, tiles inside a row by
    weight. Global + local rows all weigh about the same: a pure weight sort would interleave them."""
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.ops import attention as A
    tab = P.global_local(8, 1, 2).block_table_int
    blk = 1024
    for plan, n_tiles_per_group in ((A.FwdPlan(A.rows_from_block_table(tab, blk)), blk // A.CTA_ROWS),
                                    (A.BwdPlan(A.cols_from_block_table(tab, blk)), blk // A.TILE)):
        tiles = plan.tiles_t.tolist()
        assert len(tiles) == plan.n_tiles == 8 * n_tiles_per_group
        assert len({tuple(t) for t in tiles}) == len(tiles)                     # every tile once
        groups = [g for g, _ in tiles]
        runs = [g for i, g in enumerate(groups) if i == 0 or groups[i - 1] != g]
        assert len(runs) == len(set(runs)) == 8                                  # each group is one run
    order = A._launch_order([(5, 0, 0), (9, 1, 0), (7, 1, 1), (6, 2, 0), (5, 0, 1)])
    assert order == [(9, 1, 0), (7, 1, 1), (6, 2, 0), (5, 0, 0), (5, 0, 1)]


def test_public_flash_attention_functions_with_autograd():
    """flash_attn_func and its packed / varlen forms: outputs and gradients against dense attention
    (causal, grouped-query, more keys than queries, a sliding window)."""
    from ultraattn_b200.ops.flash_compat import (flash_attn_func, flash_attn_kvpacked_func, flash_attn_qkvpacked_func,
                                                 flash_attn_varlen_func)
    torch.manual_seed(4)
    Sq, Skv, H, Hk, D = 40, 72, 4, 2, 16
    q = torch.randn(1, Sq, H, D, requires_grad=True)
    k = torch.randn(1, Skv, Hk, D, requires_grad=True)
    v = torch.randn(1, Skv, Hk, D, requires_grad=True)
    d_o = torch.randn(1, Sq, H, D)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = _dense(q[0], k[0], v[0], d_o[0], True)
    o, lse, _ = flash_attn_func(q, k, v, causal=True, return_attn_probs=True)
    o.backward(d_o)
    assert torch.allclose(o[0], o_ref, atol=1e-5) and torch.allclose(lse[0], lse_ref, atol=1e-5)
    assert torch.allclose(q.grad[0], dq_ref, atol=1e-5) and torch.allclose(k.grad[0], dk_ref, atol=1e-5)
    assert torch.allclose(v.grad[0], dv_ref, atol=1e-5)
    o2 = flash_attn_kvpacked_func(q.detach(), torch.stack([k.detach(), v.detach()], dim=2), causal=True)
    assert torch.allclose(o2, o.detach(), atol=1e-6)
    qkv = torch.randn(1, 64, 3, 2, D)
    o3 = flash_attn_qkvpacked_func(qkv, causal=True, window_size=(20, 0))
    r, c = torch.arange(64)[:, None], torch.arange(64)[None, :]
    s = torch.einsum("qhd,khd->hqk", qkv[0, :, 0], qkv[0, :, 1]) / math.sqrt(D)
    s = s.masked_fill(~((c <= r) & (c >= r - 20)), float("-inf"))
    assert torch.allclose(o3[0], torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), qkv[0, :, 2]), atol=1e-5)
    cu = torch.tensor([0, 24, 64])
    o4 = flash_attn_varlen_func(qkv[0, :, 0], qkv[0, :, 1], qkv[0, :, 2], cu, cu, 40, 40, causal=True)
    for a, b in ((0, 24), (24, 64)):
        s = torch.einsum("qhd,khd->hqk", qkv[0, a:b, 0], qkv[0, a:b, 1]) / math.sqrt(D)
        s = s.masked_fill(~torch.ones(b - a, b - a, dtype=torch.bool).tril(), float("-inf"))
        assert torch.allclose(o4[a:b], torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), qkv[0, a:b, 2]), atol=1e-5)
