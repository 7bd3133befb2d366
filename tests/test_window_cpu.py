"""Sliding-window attention assembled from the one-sided masks of the block-sparse kernels
(usual order for the upper bound, reversed order for the lower bound) against dense masked
attention: outputs, log-sum-exps and gradients, on the fp32 restatement of the kernels."""
import math

import pytest
import torch

from ultraattn_b200.ops import window as W


def _dense(q, k, v, left, right, scale):
    B, S, H, D = q.shape
    g = H // k.shape[2]
    kk, vv = k.repeat_interleave(g, 2), v.repeat_interleave(g, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * scale
    r = torch.arange(S)[:, None]
    c = torch.arange(S)[None, :]
    mask = (c >= r - left) & (c <= r + right)
    s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv), torch.logsumexp(s, -1)


@pytest.mark.parametrize("S,window,causal", [
    (1024, (300, 0), False),         # causal band wider than a row block
    (1024, (255, 0), True),          # exactly one row block
    (768, (100, 37), False),         # two-sided, narrower than a row block
    (640, (-1, 64), False),          # unbounded to the left
    (640, (128, -1), False),         # unbounded to the right
    (520, (300, 300), False),        # token count that is no multiple of the tiles
    (512, (700, 0), True),           # window longer than the sequence: plain causal
    (96, (0, 0), False),             # each token sees itself only
])
def test_window_attention_matches_dense_masked_attention(S, window, causal):
    torch.manual_seed(S + window[0])
    B, H, Hk, D = 2, 4, 2, 32
    q = torch.randn(B, S, H, D, dtype=torch.float64).float().requires_grad_()
    k = torch.randn(B, S, Hk, D).requires_grad_()
    v = torch.randn(B, S, Hk, D).requires_grad_()
    left = S if window[0] < 0 else window[0]
    right = 0 if causal else (S if window[1] < 0 else window[1])
    scale = 1.0 / math.sqrt(D)
    o_ref, lse_ref = _dense(q, k, v, left, right, scale)
    g = torch.randn_like(o_ref)
    dq_ref, dk_ref, dv_ref = torch.autograd.grad(o_ref, (q, k, v), g)

    o, lse = W.window_forward(q.detach(), k.detach(), v.detach(), window, causal)
    assert (o - o_ref).abs().max() < 2e-5 and (lse - lse_ref).abs().max() < 2e-5
    out = W.sliding_window_attention(q, k, v, window, causal)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), g)
    for a, b in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert (a - b).abs().max() < 5e-5 * max(1.0, b.abs().max().item())


def _coverage(rows, cols, T):
    """(forward, backward) count matrices [T, T]: how many segments cover each (query, key) pair,
    in the usual token order."""
    def to_std(idx, slot):
        return idx if slot == 0 else T - 1 - idx

    def mark(mat, q_slot, q_start, q_len, k_slot, k_start, k_len, causal, diag):
        rr = torch.arange(q_len)[:, None]
        cc = torch.arange(k_len)[None, :]
        vis = (cc <= rr + diag) if causal else torch.ones(q_len, k_len, dtype=torch.bool)
        qi = to_std(q_start + rr, q_slot).expand_as(vis)[vis]
        ki = to_std(k_start + cc, k_slot).expand_as(vis)[vis]
        mat.index_put_((qi, ki), torch.ones_like(qi, dtype=torch.int32), accumulate=True)

    fwd = torch.zeros(T, T, dtype=torch.int32)
    for row in rows:
        for seg in row.segs:
            assert seg.src == row.q_src == row.o_slot and row.o_start == row.q_start
            mark(fwd, row.q_src, row.q_start, row.q_len, seg.src, seg.start, seg.length, seg.causal, seg.diag)
    bwd = torch.zeros(T, T, dtype=torch.int32)
    for col in cols:
        for seg in col.segs:
            assert seg.src == col.kv_src and col.g_slot in (col.kv_src, 2) and col.g_start == col.kv_start
            mark(bwd, seg.src, seg.start, seg.length, col.kv_src, col.kv_start, col.kv_len, seg.causal, seg.diag)
    return fwd, bwd


def _band(bounds, T, left, right):
    want = torch.zeros(T, T, dtype=torch.int32)
    for a, b in bounds:
        r = torch.arange(a, b)[:, None]
        c = torch.arange(a, b)[None, :]
        want[a:b, a:b] = ((c >= r - left) & (c <= r + right)).int()
    return want


def test_window_plan_covers_every_visible_pair_exactly_once():
    """Count, per (query, key) pair, how many segments of the forward rows and of the backward
    columns cover it: exactly the band, once each; and no gradient row has two writers."""
    S, left, right = 700, 290, 45
    rows, cols = W.window_rows_cols(S, left, right)
    fwd, bwd = _coverage(rows, cols, S)
    band = _band([(0, S)], S, left, right)
    assert torch.equal(fwd, band) and torch.equal(bwd, band)
    for slot in (0, 1):
        covered = torch.zeros(S, dtype=torch.int32)
        for col in cols:
            if col.g_slot == slot:
                covered[col.g_start:col.g_start + col.kv_len] += 1
        assert covered.max() <= 1


def test_window_plans_of_random_shapes_and_packed_batches_cover_the_band():
    """Forty random cases: sequence lengths from 1 to 900 tokens (up to three sequences packed in
    one buffer, with slack behind them), windows from 0 to beyond the sequence, one- and two-sided."""
    import random
    rng = random.Random(7)
    for _ in range(40):
        lens = [rng.choice([1, 2, 17, 255, 256, 257, 400, 513, 900]) for _ in range(rng.randint(1, 3))]
        slack = rng.choice([0, 0, 5])
        T = sum(lens) + slack
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        bounds = list(zip(cu[:-1], cu[1:]))
        window = (rng.choice([-1, 0, 1, 63, 254, 255, 256, 300, 1000]), rng.choice([-1, 0, 0, 1, 70, 256, 1000]))
        causal = rng.random() < 0.3
        rows, cols = [], []
        for a, b in bounds:
            left, right = W._bounds(b - a, window, causal)
            r, c = W.window_rows_cols(b - a, left, right, a, T)
            rows += r
            cols += c
        fwd, bwd = _coverage(rows, cols, T)
        want = torch.zeros(T, T, dtype=torch.int32)
        for a, b in bounds:
            left, right = W._bounds(b - a, window, causal)
            want += _band([(a, b)], T, left, right)
        assert torch.equal(fwd, want), (lens, window, causal)
        assert torch.equal(bwd, want), (lens, window, causal)


def test_window_size_through_the_flash_attention_calling_convention():
    """``_flash_attn_forward`` / ``_flash_attn_backward`` with ``window_size``: the caller's output
    buffer is filled, the 8-tuple keeps its layout, gradients land in the buffers passed in, with O
    present or with a precomputed D."""
    from ultraattn_b200.ops.flash_compat import _flash_attn_backward, _flash_attn_forward
    torch.manual_seed(5)
    B, S, H, Hk, D = 1, 600, 4, 4, 16
    q = torch.randn(B, S, H, D).requires_grad_()
    k = torch.randn(B, S, Hk, D).requires_grad_()
    v = torch.randn(B, S, Hk, D).requires_grad_()
    d_o = torch.randn(B, S, H, D)
    o_ref, lse_ref = _dense(q, k, v, 260, 0, 1.0 / math.sqrt(D))
    dq_ref, dk_ref, dv_ref = torch.autograd.grad(o_ref, (q, k, v), d_o)
    buf = torch.full((B, S, H, D), 3.0)
    with torch.no_grad():
        ret = _flash_attn_forward(q, k, v, 0.0, None, True, window_size=(260, -1), alibi_slopes=None,
                                  return_softmax=False, out=buf)
        assert len(ret) == 8 and ret[0] is buf and (buf - o_ref).abs().max() < 2e-5
        assert (ret[5] - lse_ref).abs().max() < 2e-5
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        out = _flash_attn_backward(d_o, q, k, v, buf, ret[5], dq, dk, dv, 0.0, None, True, (260, -1), None, False)
        assert out[0] is dq and (dq - dq_ref).abs().max() < 5e-5 and (dk - dk_ref).abs().max() < 5e-5
        assert (dv - dv_ref).abs().max() < 5e-5
        dvec = (o_ref * d_o).sum(-1).transpose(1, 2).contiguous()
        dq2 = torch.empty_like(q)
        _flash_attn_backward(d_o, q, k, v, q, ret[5], dq2, dk, dv, 0.0, None, True, (260, -1), None, False,
                             softmax_d=dvec)
        assert (dq2 - dq_ref).abs().max() < 5e-5


def test_windows_in_a_packed_batch():
    """Three sequences packed along the token axis (one empty-ish short one): each attends only
    itself and the window counts positions inside the sequence; operator with autograd and the
    varlen calling convention against per-sequence dense masked attention."""
    from ultraattn_b200.ops.flash_compat import _flash_attn_varlen_backward, _flash_attn_varlen_forward
    torch.manual_seed(11)
    lens = [300, 5, 415]
    cu = torch.tensor([0, 300, 305, 720], dtype=torch.int32)
    T, H, Hk, D = 720, 4, 2, 16
    left, right = 130, 20
    q = torch.randn(1, T, H, D).requires_grad_()
    k = torch.randn(1, T, Hk, D).requires_grad_()
    v = torch.randn(1, T, Hk, D).requires_grad_()
    d_o = torch.randn(1, T, H, D)
    outs, lses = [], []
    for a, b in zip(cu[:-1].tolist(), cu[1:].tolist()):
        o_i, lse_i = _dense(q[:, a:b], k[:, a:b], v[:, a:b], left, right, 1.0 / math.sqrt(D))
        outs.append(o_i)
        lses.append(lse_i)
    o_ref = torch.cat(outs, 1)
    dq_ref, dk_ref, dv_ref = torch.autograd.grad(o_ref, (q, k, v), d_o)

    o = W.sliding_window_attention(q, k, v, (left, right), cu_seqlens=cu)
    assert (o - o_ref).abs().max() < 2e-5
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), d_o)
    for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
        assert (got - ref).abs().max() < 5e-5

    with torch.no_grad():
        ret = _flash_attn_varlen_forward(q[0], k[0], v[0], cu, cu, max(lens), max(lens), 0.0, None, False,
                                         window_size=(left, right))
        assert (ret[0] - o_ref[0]).abs().max() < 2e-5 and ret[5].shape == (3, H, max(lens))
        for i, n in enumerate(lens):
            assert (ret[5][i, :, :n] - lses[i][0]).abs().max() < 2e-5
        gq, gk, gv = torch.empty_like(q[0]), torch.empty_like(k[0]), torch.empty_like(v[0])
        _flash_attn_varlen_backward(d_o[0], q[0], k[0], v[0], ret[0], ret[5], gq, gk, gv, cu, cu, max(lens), max(lens),
                                    0.0, None, False, window_size=(left, right))
        assert (gq - dq_ref[0]).abs().max() < 5e-5 and (gk - dk_ref[0]).abs().max() < 5e-5
        assert (gv - dv_ref[0]).abs().max() < 5e-5


def _band_with_sinks(S, left, right, sink):
    r = torch.arange(S)[:, None]
    c = torch.arange(S)[None, :]
    return ((c >= r - left) & (c <= r + right)) | ((c < sink) & (c <= r + right))


@pytest.mark.parametrize("S,left,right,sink", [(1000, 300, 0, 4), (700, 255, 0, 256), (520, 40, 0, 41),
                                               (900, 128, 30, 16), (300, 1000, 0, 8), (256, 100, 0, 3)])
def test_attention_sinks_cover_and_match_dense(S, left, right, sink):
    """Sliding window plus attention sinks (the first tokens stay visible to every later query):
    every visible pair once in the forward rows and in the backward columns, and outputs and
    gradients equal dense masked attention."""
    l, r_ = W._bounds(S, (left, right), False)
    rows, cols = W.window_rows_cols(S, l, r_, sink=sink)
    fwd, bwd = _coverage(rows, cols, S)
    want = _band_with_sinks(S, l, r_, sink).int()
    assert torch.equal(fwd, want) and torch.equal(bwd, want)
    for slot in (0, 1, 2):                  # one writer per gradient row and slot
        covered = torch.zeros(S, dtype=torch.int32)
        for col in cols:
            if col.g_slot == slot:
                covered[col.g_start:col.g_start + col.kv_len] += 1
        assert covered.max() <= 1
    torch.manual_seed(S + sink)
    B, H, Hk, D = 1, 2, 1, 16
    q = torch.randn(B, S, H, D).requires_grad_()
    k = torch.randn(B, S, Hk, D).requires_grad_()
    v = torch.randn(B, S, Hk, D).requires_grad_()
    g = torch.randn(B, S, H, D)
    sc = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(H // Hk, 2)) / math.sqrt(D)
    sc = sc.masked_fill(~_band_with_sinks(S, l, r_, sink), float("-inf"))
    o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), v.repeat_interleave(H // Hk, 2))
    ref = torch.autograd.grad(o_ref, (q, k, v), g)
    o = W.sliding_window_attention(q, k, v, (left, right), sink_tokens=sink)
    assert (o - o_ref).abs().max() < 2e-5
    got = torch.autograd.grad(o, (q, k, v), g)
    for a, b in zip(got, ref):
        assert (a - b).abs().max() < 5e-5 * max(1.0, b.abs().max().item())


def test_too_many_sinks_are_refused():
    with pytest.raises(AssertionError, match="sink tokens"):
        W.window_rows_cols(1000, 50, 0, sink=52)


def test_sinks_in_a_packed_batch():
    """Every sequence of a packed batch has its own sinks; operator against per-sequence dense attention."""
    torch.manual_seed(3)
    cu = [0, 350, 400, 1000]
    T, H, D, left, sink = 1000, 2, 16, 90, 5
    q, k, v = (torch.randn(1, T, H, D) for _ in range(3))
    o = W.sliding_window_attention(q, k, v, (left, 0), cu_seqlens=cu, sink_tokens=sink)
    for a, b in zip(cu[:-1], cu[1:]):
        n = b - a
        sc = torch.einsum("bqhd,bkhd->bhqk", q[:, a:b], k[:, a:b]) / math.sqrt(D)
        sc = sc.masked_fill(~_band_with_sinks(n, left, 0, sink), float("-inf"))
        o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), v[:, a:b])
        assert (o[:, a:b] - o_ref).abs().max() < 2e-5


@pytest.mark.parametrize("S,prefix,cu", [(300, 100, None), (257, 0, None), (128, 500, None), (600, 70, [0, 50, 50, 400, 600])])
def test_prefix_lm_mask(S, prefix, cu):
    """Prefix-LM: bidirectional inside the prefix, causal behind it; also per sequence of a packed batch."""
    import ultraattn_b200 as ua
    torch.manual_seed(S)
    H, Hk, D = 4, 2, 16
    q = torch.randn(1, S, H, D).requires_grad_()
    k = torch.randn(1, S, Hk, D).requires_grad_()
    v = torch.randn(1, S, Hk, D).requires_grad_()
    g = torch.randn(1, S, H, D)
    mask = torch.zeros(S, S, dtype=torch.bool)
    for a, b in zip(*(([0], [S]) if cu is None else (cu[:-1], cu[1:]))):
        r = torch.arange(a, b)[:, None]
        c = torch.arange(a, b)[None, :]
        mask[a:b, a:b] = (c <= r) | (c < a + prefix)
    sc = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(2, 2)) / math.sqrt(D)
    o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc.masked_fill(~mask, float("-inf")), -1), v.repeat_interleave(2, 2))
    ref = torch.autograd.grad(o_ref, (q, k, v), g)
    o = ua.prefix_lm_attention(q, k, v, prefix, cu_seqlens=cu)
    assert (o - o_ref).abs().max() < 2e-5
    got = torch.autograd.grad(o, (q, k, v), g)
    for x, y in zip(got, ref):
        assert (x - y).abs().max() < 5e-5


def test_mask_benchmark_driver_checks_every_mask():
    """``drivers/bench_masks.py`` (the masks of the reference's FlexAttention benchmark as launch
    plans of these kernels): every mask matches dense attention and reports its density and times."""
    from ultraattn_b200.drivers.bench_masks import run
    recs = run(512, 4, 2, 16, ["causal", "sliding_window", "prefix_lm", "document"], 120, 70, 5, 1, 16384,
               torch.device("cpu"))
    assert [r["mask"] for r in recs] == ["causal", "sliding_window", "prefix_lm", "document"]
    for r in recs:
        assert r["max_err"] < 2e-5 and 0 < r["density"] < 0.6 and r["fwd_ms"] > 0 and r["fwd_bwd_tflops"] > 0
    assert recs[1]["density"] < recs[0]["density"] < recs[2]["density"]      # window < causal < prefix-LM


@pytest.mark.parametrize("Sq,Skv,window,causal", [(300, 1000, (400, 0), True), (256, 700, (100, 30), False),
                                                  (64, 64 + 513, (1000, 0), True), (500, 520, (10, -1), False),
                                                  (1, 900, (300, 0), True)])
def test_window_with_the_queries_at_the_end_of_a_longer_key_sequence(Sq, Skv, window, causal):
    """A chunk of queries behind context keys (bottom-right aligned band): coverage of the plan,
    outputs and gradients (those of the context keys included) against dense masked attention."""
    off = Skv - Sq
    left, right = W._bounds(Skv, window, causal)
    r = torch.arange(Sq)[:, None] + off
    c = torch.arange(Skv)[None, :]
    band = (c >= r - left) & (c <= r + right)
    rows, cols = W.window_rows_cols_suffix(Sq, Skv, left, right)
    for items, is_fwd in ((rows, True), (cols, False)):
        cover = torch.zeros(Sq, Skv, dtype=torch.int32)
        for it in items:
            for seg in it.segs:
                q_slot, q_start, q_len = (it.q_src, it.q_start, it.q_len) if is_fwd else (seg.src, seg.start, seg.length)
                k_slot, k_start, k_len = (seg.src, seg.start, seg.length) if is_fwd else (it.kv_src, it.kv_start, it.kv_len)
                rr, cc = torch.arange(q_len)[:, None], torch.arange(k_len)[None, :]
                vis = (cc <= rr + seg.diag) if seg.causal else torch.ones(q_len, k_len, dtype=torch.bool)
                qi = (q_start + rr if q_slot == 0 else Sq - 1 - (q_start + rr)).expand_as(vis)[vis]
                ki = (k_start + cc if k_slot == 0 else Skv - 1 - (k_start + cc)).expand_as(vis)[vis]
                cover.index_put_((qi, ki), torch.ones_like(qi, dtype=torch.int32), accumulate=True)
        assert torch.equal(cover, band.int()), ("rows" if is_fwd else "cols")
    torch.manual_seed(Sq)
    H, Hk, D = 4, 2, 16
    q = torch.randn(1, Sq, H, D).requires_grad_()
    k = torch.randn(1, Skv, Hk, D).requires_grad_()
    v = torch.randn(1, Skv, Hk, D).requires_grad_()
    g = torch.randn(1, Sq, H, D)
    sc = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(2, 2)) / math.sqrt(D)
    sc = sc.masked_fill(~band, float("-inf"))
    o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), v.repeat_interleave(2, 2))
    ref = torch.autograd.grad(o_ref, (q, k, v), g)
    o = W.sliding_window_attention(q, k, v, window, causal)
    assert (o - o_ref).abs().max() < 2e-5
    got = torch.autograd.grad(o, (q, k, v), g)
    for a, b in zip(got, ref):
        assert (a - b).abs().max() < 5e-5 * max(1.0, b.abs().max().item())


@pytest.mark.parametrize("Sq,Skv,off,window", [(300, 900, 250, (200, 120)), (256, 600, 0, (50, 400)), (100, 700, 300, (1000, 1000)),
                                               (513, 700, 100, (64, 33)), (64, 64, 0, (10, 10))])
def test_window_with_the_queries_in_the_middle_of_the_keys(Sq, Skv, off, window):
    """Queries at positions ``off ... off + Sq`` of the key sequence (a shard between two halos):
    plan coverage, outputs and all gradients through ``window_forward`` / ``window_backward``."""
    left, right = W._bounds(Skv, window, False)
    r = torch.arange(Sq)[:, None] + off
    c = torch.arange(Skv)[None, :]
    band = (c >= r - left) & (c <= r + right)
    rows, cols = W.window_rows_cols_offset(Sq, Skv, left, right, off)
    for items, is_fwd in ((rows, True), (cols, False)):
        cover = torch.zeros(Sq, Skv, dtype=torch.int32)
        for it in items:
            for seg in it.segs:
                q_slot, q_start, q_len = (it.q_src, it.q_start, it.q_len) if is_fwd else (seg.src, seg.start, seg.length)
                k_slot, k_start, k_len = (seg.src, seg.start, seg.length) if is_fwd else (it.kv_src, it.kv_start, it.kv_len)
                rr, cc = torch.arange(q_len)[:, None], torch.arange(k_len)[None, :]
                vis = (cc <= rr + seg.diag) if seg.causal else torch.ones(q_len, k_len, dtype=torch.bool)
                qi = (q_start + rr if q_slot == 0 else Sq - 1 - (q_start + rr)).expand_as(vis)[vis]
                ki = (k_start + cc if k_slot == 0 else Skv - 1 - (k_start + cc)).expand_as(vis)[vis]
                cover.index_put_((qi, ki), torch.ones_like(qi, dtype=torch.int32), accumulate=True)
        assert torch.equal(cover, band.int()), ("rows" if is_fwd else "cols")
    for slot in (0, 1):                     # one writer per gradient row and slot
        covered = torch.zeros(Skv, dtype=torch.int32)
        for col in cols:
            if col.g_slot == slot:
                covered[col.g_start:col.g_start + col.kv_len] += 1
        assert covered.max() <= 1
    torch.manual_seed(Sq + off)
    H, Hk, D = 2, 1, 16
    q = torch.randn(1, Sq, H, D).requires_grad_()
    k = torch.randn(1, Skv, Hk, D).requires_grad_()
    v = torch.randn(1, Skv, Hk, D).requires_grad_()
    g = torch.randn(1, Sq, H, D)
    sc = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(2, 2)) / math.sqrt(D)
    sc = sc.masked_fill(~band, float("-inf"))
    o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), v.repeat_interleave(2, 2))
    ref = torch.autograd.grad(o_ref, (q, k, v), g)
    with torch.no_grad():
        o, lse = W.window_forward(q, k, v, window, False, q_offset=off)
        got = W.window_backward(g, q, k, v, o, lse, window, False, q_offset=off)
    assert (o - o_ref).abs().max() < 2e-5 and (lse - torch.logsumexp(sc, -1)).abs().max() < 2e-5
    for a, b in zip(got, ref):
        assert (a - b).abs().max() < 5e-5 * max(1.0, b.abs().max().item())


def test_window_that_covers_every_sequence_takes_the_plain_path(monkeypatch):
    """A window at least as long as every sequence is plain causal / full attention: no reversed
    copies are made (here: making one would raise), results as usual."""
    def no_flip(*a, **k):
        raise AssertionError("a reversed copy was made")
    monkeypatch.setattr(W, "_flip", no_flip)
    torch.manual_seed(2)
    cu = [0, 200, 500]
    q = torch.randn(1, 500, 2, 16).requires_grad_()
    k = torch.randn(1, 500, 2, 16).requires_grad_()
    v = torch.randn(1, 500, 2, 16).requires_grad_()
    g = torch.randn(1, 500, 2, 16)
    o = W.sliding_window_attention(q, k, v, (4095, 0), True, cu_seqlens=cu, sink_tokens=4)
    got = torch.autograd.grad(o, (q, k, v), g)
    mask = torch.zeros(500, 500, dtype=torch.bool)
    for a, b in zip(cu[:-1], cu[1:]):
        mask[a:b, a:b] = torch.ones(b - a, b - a, dtype=torch.bool).tril()
    sc = (torch.einsum("bqhd,bkhd->bhqk", q, k) / 4).masked_fill(~mask, float("-inf"))
    o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), v)
    ref = torch.autograd.grad(o_ref, (q, k, v), g)
    assert (o - o_ref).abs().max() < 2e-5
    for x, y in zip(got, ref):
        assert (x - y).abs().max() < 5e-5
    with pytest.raises(AssertionError, match="reversed copy"):       # a shorter window does need them
        W.sliding_window_attention(q, k, v, (100, 0), True, cu_seqlens=cu)
