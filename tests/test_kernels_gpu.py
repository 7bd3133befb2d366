"""sm_100a kernels against fp32 PyTorch restatements of the same ops (run on a B200)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA GPU")
    from ultraattn_b200 import _lib
    _lib.load()          # fails loudly if the kernel library is missing
    return torch.device("cuda")


def _close(got, ref, tol):
    """Largest absolute error against the largest reference value, and, so that a wrong row of
    small magnitude cannot hide behind the large ones, every row (last dimension) on its own:
    |got - ref| <= 4 tol * max(|ref row|, a tenth of the median row norm)."""
    g, r = got.float(), ref.float()
    err = (g - r).abs().max().item()
    scale = r.abs().max().item() + 1e-6
    assert err <= tol * scale, f"max err {err} vs scale {scale}"
    if r.dim() >= 2 and r.shape[-1] > 1:
        d = (g - r).flatten(0, -2).norm(dim=-1)
        n = r.flatten(0, -2).norm(dim=-1)
        rel = d / torch.clamp(n, min=0.1 * n.median().item() + 1e-12)
        worst = int(rel.argmax())
        assert rel[worst].item() <= 4 * tol, f"row {worst}: relative error {rel[worst].item():.3e} (norm {n[worst].item():.3e})"


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 520, 264), (2048, 4096, 1024)])
def test_gemm_tn(dev, M, N, K):
    from ultraattn_b200.ops import attention as A, gemm as G
    torch.manual_seed(0)
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    c = G.gemm(a, b)
    A.check_status(dev)
    _close(c, a.float() @ b.float().t(), 1e-2)


def test_gemm_other_layouts(dev):
    from ultraattn_b200.ops import attention as A, gemm as G
    torch.manual_seed(1)
    M, N, K = 512, 768, 512
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    bkn = torch.randn(K, N, device=dev, dtype=torch.bfloat16)
    _close(G.gemm(a, bkn, b_is_kn=True), a.float() @ bkn.float(), 1e-2)
    akm = torch.randn(K, M, device=dev, dtype=torch.bfloat16)
    _close(G.gemm(akm, bkn, a_is_km=True, b_is_kn=True), akm.float().t() @ bkn.float(), 1e-2)
    A.check_status(dev)


def test_gemm_scatter_gather_single_gpu(dev):
    """The all-to-all fusions with every 'peer' buffer on this GPU: column groups land in
    different buffers (scatter) and K groups come from different buffers (gather)."""
    from ultraattn_b200.ops import attention as A, gemm as G
    torch.manual_seed(2)
    M, N, K, P = 256, 512, 256, 4
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    dsts = [torch.zeros(2 * M, N // P, device=dev, dtype=torch.bfloat16) for _ in range(P)]
    G.gemm_scatter(a, w, [d.data_ptr() for d in dsts], N // P, M)
    for g, d in enumerate(dsts):
        _close(d[M:], ref[:, g * (N // P):(g + 1) * (N // P)], 1e-2)
        assert d[:M].abs().max().item() == 0
    srcs = [torch.randn(3 * M, K // P, device=dev, dtype=torch.bfloat16) for _ in range(P)]
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    G.gemm_gather([s.data_ptr() for s in srcs], 3 * M, K // P, M, M, K // P, w, out)
    a_full = torch.cat([s[M:2 * M] for s in srcs], dim=1)
    _close(out, a_full.float() @ w.float().t(), 1e-2)
    A.check_status(dev)


@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (1000, 520, 264), (4096, 2048, 1024), (320, 256, 64)])
def test_gemm_cta_pair_all_layouts(dev, monkeypatch, M, N, K):
    """The 256 x 256 tile computed by a pair of CTAs (cta_group::2), forced on for shapes the
    heuristic would give to the single-CTA kernel: x W^T, dy W and dy^T x storage orders, ragged
    edges, and the scatter / gather fusions."""
    from ultraattn_b200.ops import attention as A, gemm as G
    monkeypatch.setenv("UA_GEMM_PAIR", "1")
    torch.manual_seed(3)
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    _close(G.gemm(a, b), a.float() @ b.float().t(), 1e-2)
    bkn = torch.randn(K, N, device=dev, dtype=torch.bfloat16)
    _close(G.gemm(a, bkn, b_is_kn=True), a.float() @ bkn.float(), 1e-2)
    akm = torch.randn(K, M, device=dev, dtype=torch.bfloat16)
    _close(G.gemm(akm, bkn, a_is_km=True, b_is_kn=True), akm.float().t() @ bkn.float(), 1e-2)
    _close(G.gemm(akm, b, a_is_km=True), akm.float().t() @ b.float().t(), 1e-2)
    A.check_status(dev)
    if N % 128 == 0 and K % 128 == 0:
        P = 2
        ref = a.float() @ b.float().t()
        dsts = [torch.zeros(2 * M, N // P, device=dev, dtype=torch.bfloat16) for _ in range(P)]
        G.gemm_scatter(a, b, [d.data_ptr() for d in dsts], N // P, M)
        for g, d in enumerate(dsts):
            _close(d[M:], ref[:, g * (N // P):(g + 1) * (N // P)], 1e-2)
            assert d[:M].abs().max().item() == 0
        srcs = [torch.randn(3 * M, K // P, device=dev, dtype=torch.bfloat16) for _ in range(P)]
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        G.gemm_gather([t.data_ptr() for t in srcs], 3 * M, K // P, M, M, K // P, b, out)
        _close(out, torch.cat([t[M:2 * M] for t in srcs], dim=1).float() @ b.float().t(), 1e-2)
        A.check_status(dev)


def test_gemm_large_uses_pair_kernel_and_matches(dev):
    """A projection-sized problem (the heuristic picks the CTA-pair kernel) against torch."""
    from ultraattn_b200.ops import attention as A, gemm as G
    torch.manual_seed(4)
    a = torch.randn(8192, 4096, device=dev, dtype=torch.bfloat16)
    b = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
    c = G.gemm(a, b)
    A.check_status(dev)
    _close(c, (a @ b.t()).float(), 1e-2)


CASES = [
    ("full", 256, 1, 1, [[1]], 256),
    ("causal", 256, 2, 2, [[2]], 256),
    ("causal-1k", 1024, 4, 4, [[2]], 1024),
    ("bsa", 2048, 4, 4, [[2, 0, 0, 0], [1, 2, 0, 0], [1, 0, 2, 0], [1, 0, 1, 2]], 512),
    ("gqa", 1024, 8, 2, [[2]], 1024),
    ("ragged", 320, 2, 2, [[2]], 320),
    ("global-local", 2048, 2, 2, None, 256),
]


@pytest.mark.parametrize("name,S,H,Hk,table,block", CASES, ids=[c[0] for c in CASES])
def test_attention_fwd_bwd(dev, name, S, H, Hk, table, block):
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.ops import attention as A, elementwise as E
    torch.manual_seed(0)
    tab = P.global_local(8, 1, 2).block_table_int if table is None else np.array(table)
    q = torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16)
    k = torch.randn(1, S, Hk, 128, device=dev, dtype=torch.bfloat16)
    v = torch.randn(1, S, Hk, 128, device=dev, dtype=torch.bfloat16)
    d_o = torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16)
    rows = A.rows_from_block_table(tab, block)
    cols = A.cols_from_block_table(tab, block)
    o = torch.zeros_like(q)
    lse = torch.zeros(1, H, S, device=dev, dtype=torch.float32)
    A.attn_fwd_cuda([q], [k], [v], [(o, lse)], A.FwdPlan(rows, dev))
    o_ref = torch.zeros(1, S, H, 128, device=dev)
    lse_ref = torch.zeros(1, H, S, device=dev)
    A.attn_fwd_reference([q], [k], [v], [(o_ref, lse_ref)], rows)
    A.check_status(dev)
    _close(o, o_ref, 1e-2)
    fin = torch.isfinite(lse_ref)
    assert (lse[fin] - lse_ref[fin]).abs().max().item() < 2e-3
    dvec = E.rowdot(o[0], d_o[0]).unsqueeze(0)
    _close(dvec, (o.float() * d_o.float()).sum(-1).permute(0, 2, 1), 1e-3)
    dq = torch.zeros(1, S, H, 128, device=dev)
    dk = torch.zeros(1, S, Hk, 128, device=dev, dtype=torch.bfloat16)
    dv = torch.zeros_like(dk)
    A.attn_bwd_cuda([A.BwdQSide(q, d_o, lse, dvec, dq)], [k], [v], [A.BwdKvOut(dk, dv)], A.BwdPlan(cols, dev))
    dq_r = torch.zeros_like(dq)
    dk_r = torch.zeros(1, S, Hk, 128, device=dev)
    dv_r = torch.zeros_like(dk_r)
    A.attn_bwd_reference([A.BwdQSide(q, d_o, lse_ref, dvec, dq_r)], [k], [v], [A.BwdKvOut(dk_r, dv_r)], cols)
    A.check_status(dev)
    _close(dq, dq_r, 2e-2)
    _close(dk, dk_r, 2e-2)
    _close(dv, dv_r, 2e-2)


def test_attention_accumulate_and_add_modes(dev):
    """Forward merge-into-existing (the running-state mode) and backward fp32 add mode."""
    from ultraattn_b200.ops import attention as A, elementwise as E
    torch.manual_seed(3)
    S, H = 512, 2
    q, k, v, d_o = (torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16) for _ in range(4))
    o = torch.zeros_like(q)
    lse = torch.zeros(1, H, S, device=dev)
    first = [A.Row(0, 0, S, (A.Seg(0, 0, 256, False, 0),), 0, 0, False)]
    second = [A.Row(0, 0, S, (A.Seg(0, 256, 256, False, 0),), 0, 0, True)]
    A.attn_fwd_cuda([q], [k], [v], [(o, lse)], A.FwdPlan(first, dev))
    A.attn_fwd_cuda([q], [k], [v], [(o, lse)], A.FwdPlan(second, dev))
    both = [A.Row(0, 0, S, (A.Seg(0, 0, S, False, 0),), 0, 0, False)]
    o_ref = torch.zeros(1, S, H, 128, device=dev)
    lse_ref = torch.zeros(1, H, S, device=dev)
    A.attn_fwd_reference([q], [k], [v], [(o_ref, lse_ref)], both)
    _close(o, o_ref, 1.5e-2)
    assert (lse - lse_ref).abs().max().item() < 2e-3
    dvec = E.rowdot(o[0], d_o[0]).unsqueeze(0)
    cols = [A.Col(0, 0, S, (A.Seg(0, 0, S, False, 0),), 0, 0)]
    dq = torch.zeros(1, S, H, 128, device=dev)
    dk = torch.ones(1, S, H, 128, device=dev)
    dv = torch.ones(1, S, H, 128, device=dev)
    A.attn_bwd_cuda([A.BwdQSide(q, d_o, lse, dvec, dq)], [k], [v], [A.BwdKvOut(dk, dv)], A.BwdPlan(cols, dev))
    dq_r = torch.zeros_like(dq)
    dk_r = torch.ones_like(dk)
    dv_r = torch.ones_like(dv)
    A.attn_bwd_reference([A.BwdQSide(q, d_o, lse, dvec, dq_r)], [k], [v], [A.BwdKvOut(dk_r, dv_r)], cols)
    A.check_status(dev)
    _close(dk, dk_r, 2e-2)
    _close(dv, dv_r, 2e-2)


@pytest.mark.parametrize("T,V,ld", [(300, 32000, 32000), (64, 1000, 1024)])
def test_token_cross_entropy(dev, T, V, ld):
    """Fused cross-entropy over bf16 logits (strided rows, an ignored target): log-sum-exp and loss
    against fp32 PyTorch, and the in-place gradient g * (softmax - one-hot)."""
    from ultraattn_b200.ops import elementwise as E
    torch.manual_seed(5)
    store = torch.randn(T, ld, device=dev) * 4
    logits = store.to(torch.bfloat16)[:, :V]
    targets = torch.randint(0, V, (T,), device=dev)
    targets[3] = -100
    ref = logits.float()
    lse_r = torch.logsumexp(ref, dim=-1)
    ok = targets >= 0
    loss_r = torch.where(ok, lse_r - ref.gather(1, targets.clamp(min=0)[:, None]).squeeze(1), torch.zeros_like(lse_r))
    lse, loss = E.xent_fwd(logits, targets)
    assert (lse - lse_r).abs().max().item() < 1e-3 and (loss - loss_r).abs().max().item() < 1e-3
    g = torch.tensor(0.37, device=dev)
    p = torch.softmax(ref, dim=-1)
    p[torch.arange(T, device=dev)[ok], targets[ok]] -= 1.0
    want = p * 0.37 * ok[:, None]
    work = logits.clone() if ld == V else logits       # the strided view is updated in place inside `store`'s copy
    got = E.xent_bwd_(work, targets, lse, g)
    assert got.data_ptr() == work.data_ptr()
    _close(got, want, 1e-2)
    assert got[3].abs().max().item() == 0.0


def test_tensor_maps_are_encoded_once_per_buffer(dev):
    """A repeated launch over the same buffers finds all of its TMA tensor maps in the library's
    cache; a launch over other buffers of the same shape encodes new ones and computes from them."""
    from ultraattn_b200.ops import attention as A
    torch.manual_seed(11)
    S, H = 512, 2
    q, k, v = (torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16) for _ in range(3))
    o, lse = torch.zeros_like(q), torch.zeros(1, H, S, device=dev)
    rows = [A.Row(0, 0, S, (A.Seg(0, 0, S, True, 0),), 0, 0, False)]
    plan = A.FwdPlan(rows, dev)
    A.attn_fwd_cuda([q], [k], [v], [(o, lse)], plan)
    h0, m0 = A.tensor_map_cache_stats()
    A.attn_fwd_cuda([q], [k], [v], [(o, lse)], plan)
    h1, m1 = A.tensor_map_cache_stats()
    assert m1 == m0 and h1 - h0 >= 3
    k2, v2 = torch.randn_like(k), torch.randn_like(v)
    o2 = torch.zeros_like(q)
    A.attn_fwd_cuda([q], [k2], [v2], [(o2, lse)], plan)
    h2, m2 = A.tensor_map_cache_stats()
    assert m2 - m1 == 2 and h2 > h1
    o_ref, lse_ref = torch.zeros(1, S, H, 128, device=dev), torch.zeros(1, H, S, device=dev)
    A.attn_fwd_reference([q], [k2], [v2], [(o_ref, lse_ref)], rows)
    A.check_status(dev)
    _close(o2, o_ref, 1.5e-2)


def test_autograd_api(dev):
    import ultraattn_b200 as ua
    from ultraattn_b200 import patterns as P
    torch.manual_seed(4)
    S, H = 1024, 2
    pat = P.strided(8, 4, 2)
    q, k, v = (torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    d_o = torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16)
    o = ua.attention(q, k, v, pat)
    o.backward(d_o)
    o_ref, _, dq, dk, dv = P.dense_attention_with_grads(q, k, v, d_o, pat)
    _close(o, o_ref, 1e-2)
    _close(q.grad, dq, 2e-2)
    _close(k.grad, dk, 2e-2)
    _close(v.grad, dv, 2e-2)


def test_head_dim_64_runs_zero_padded(dev):
    """Head dim 64 on the GPU: the operator pads to the kernels' 128, keeps the scale of the true
    head dim and returns outputs and gradients of the true shape."""
    import ultraattn_b200 as ua
    from ultraattn_b200 import patterns as P
    torch.manual_seed(8)
    S, H, D = 1024, 2, 64
    pat = P.global_local(4, 1, 2)
    q, k, v = (torch.randn(1, S, H, D, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    d_o = torch.randn(1, S, H, D, device=dev, dtype=torch.bfloat16)
    o = ua.attention(q, k, v, pat)
    assert o.shape == (1, S, H, D)
    o.backward(d_o)
    o_r, _, dq_r, dk_r, dv_r = P.dense_attention_with_grads(q.detach().float().cpu(), k.detach().float().cpu(),
                                                            v.detach().float().cpu(), d_o.float().cpu(), pat)
    _close(o.detach().cpu(), o_r, 1.5e-2)
    for got, ref in ((q.grad, dq_r), (k.grad, dk_r), (v.grad, dv_r)):
        assert got.shape == (1, S, H, D)
        _close(got.cpu(), ref, 2e-2)


def test_lse_merge(dev):
    from ultraattn_b200.ops import elementwise as E
    torch.manual_seed(5)
    T, H, k = 300, 3, 4
    parts = [(torch.randn(T, H, 128, device=dev, dtype=torch.bfloat16),
              torch.randn(H, T, device=dev) * 3) for _ in range(k)]
    parts[1][1][0, :17] = float("-inf")
    o_ref, l_ref = E.lse_merge_reference(parts)
    out = (torch.empty(T, H, 128, device=dev, dtype=torch.bfloat16), torch.empty(H, T, device=dev))
    E.lse_merge(parts, out)
    _close(out[0], o_ref, 1e-2)
    assert (out[1] - l_ref).abs().max().item() < 1e-4


def test_model_ops(dev):
    from ultraattn_b200.ops import elementwise as E
    torch.manual_seed(6)
    rows, Hd, F = 257, 4096, 1024
    x = torch.randn(rows, Hd, device=dev, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(Hd, device=dev)).to(torch.bfloat16)
    g = torch.randn(rows, Hd, device=dev, dtype=torch.bfloat16)
    y, rstd = E.rmsnorm_fwd(x, w, 1e-5)
    y_ref, rstd_ref = E.rmsnorm_fwd(x.cpu(), w.cpu(), 1e-5)
    _close(y, y_ref.to(dev), 1e-2)
    dx, dw = E.rmsnorm_bwd(x, w, g, rstd)
    dx_ref, dw_ref = E.rmsnorm_bwd(x.cpu(), w.cpu(), g.cpu(), rstd_ref)
    _close(dx, dx_ref.to(dev), 1e-2)
    _close(dw, dw_ref.to(dev), 1e-2)
    T, Hh = 130, 4
    xr = torch.randn(T, Hh, 128, device=dev, dtype=torch.bfloat16)
    cos, sin = E.rope_tables(512, 128, device=dev)
    pos = torch.randint(0, 512, (T,), device=dev, dtype=torch.int32)
    yr = E.rope(xr, cos, sin, pos)
    yr_ref = E.rope(xr.cpu(), cos.cpu(), sin.cpu(), pos.cpu())
    _close(yr, yr_ref.to(dev), 1e-2)
    back = E.rope(yr, cos, sin, pos, inverse=True)
    _close(back, xr, 2e-2)
    gu = torch.randn(rows, 2 * F, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(rows, F, device=dev, dtype=torch.bfloat16)
    _close(E.swiglu_fwd(gu), E.swiglu_fwd(gu.cpu()).to(dev), 1e-2)
    _close(E.swiglu_bwd(gu, dy), E.swiglu_bwd(gu.cpu(), dy.cpu()).to(dev), 1e-2)
    n = 1000
    master = torch.randn(n, device=dev)
    m = torch.zeros(n, device=dev)
    vv = torch.zeros(n, device=dev)
    grad = torch.randn(n, device=dev, dtype=torch.bfloat16)
    param = master.to(torch.bfloat16)
    ref = [t.cpu().clone() for t in (master, m, vv, grad, param)]
    E.adam_step(master, m, vv, grad, param, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1)
    E.adam_step(*ref, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1)
    _close(master, ref[0].to(dev), 1e-5)
    _close(param, ref[4].to(dev), 1e-2)


@pytest.mark.parametrize("Hd", [4096, 768])       # the sliced single-pass kernels (H % 2048 == 0) and the warp-per-row ones
def test_rmsnorm_with_fused_residual(dev, Hd):
    """x + res and RMSNorm(x + res) from one kernel, and the backward that adds the residual
    branch's gradient inside the norm's backward kernel, against the fp32 restatement."""
    from ultraattn_b200.ops import elementwise as E
    torch.manual_seed(7)
    rows = 259
    x, res, g, dres = (torch.randn(rows, Hd, device=dev, dtype=torch.bfloat16) for _ in range(4))
    w = (1 + 0.1 * torch.randn(Hd, device=dev)).to(torch.bfloat16)
    xsum, y, rstd = E.add_rmsnorm_fwd(x, res, w, 1e-5)
    xsum_ref, y_ref, rstd_ref = E.add_rmsnorm_fwd(x.cpu(), res.cpu(), w.cpu(), 1e-5)
    assert torch.equal(xsum.cpu(), xsum_ref)                       # one bf16 rounding of the sum on both sides
    _close(y, y_ref.to(dev), 1e-2)
    _close(rstd, rstd_ref.to(dev), 1e-3)
    dx, dw = E.rmsnorm_bwd(xsum, w, g, rstd, dres=dres)
    dx_ref, dw_ref = E.rmsnorm_bwd(xsum_ref, w.cpu(), g.cpu(), rstd_ref, dres=dres.cpu())
    _close(dx, dx_ref.to(dev), 1e-2)
    _close(dw, dw_ref.to(dev), 1e-2)


def test_varlen_packed_attention(dev):
    """Packed sequences of ragged lengths (document mask) through the same kernels."""
    from ultraattn_b200.api import varlen_attention
    torch.manual_seed(7)
    cu = [0, 100, 421, 1000, 1024]
    T, H = 1024, 2
    q, k, v = (torch.randn(T, H, 128, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    d_o = torch.randn(T, H, 128, device=dev, dtype=torch.bfloat16)
    o = varlen_attention(q, k, v, cu, causal=True)
    o.backward(d_o)
    mask = torch.zeros(T, T, dtype=torch.bool, device=dev)
    for a, b in zip(cu[:-1], cu[1:]):
        mask[a:b, a:b] = torch.tril(torch.ones(b - a, b - a, dtype=torch.bool, device=dev))
    q2, k2, v2 = (t.detach().float().requires_grad_() for t in (q, k, v))
    sc = torch.einsum("qhd,khd->hqk", q2, k2) / math.sqrt(128)
    o2 = torch.einsum("hqk,khd->qhd", torch.softmax(sc.masked_fill(~mask, float("-inf")), -1), v2)
    o2.backward(d_o.float())
    _close(o, o2, 1e-2)
    _close(q.grad, q2.grad, 2e-2)
    _close(k.grad, k2.grad, 2e-2)
    _close(v.grad, v2.grad, 2e-2)


def test_llama_train_steps_match_cpu(dev):
    """Three optimizer steps of a small Llama on the GPU kernels against the same model (same
    weights) run through the CPU reference path: losses must agree step by step."""
    import math
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.models.llama import LlamaConfig, LlamaModel
    from ultraattn_b200.ops import attention as A
    cfg = LlamaConfig(n_layers=2, hidden=256, n_heads=2, head_dim=128, ffn=512, vocab=1000)
    pat = P.global_local(4, 1, 2)
    S = 2048
    g = torch.Generator().manual_seed(3)
    ids_all = torch.randint(0, cfg.vocab, (S + 1,), generator=g)
    ref = LlamaModel(cfg, device=torch.device("cpu"), pattern=pat, seed=0)
    got = LlamaModel(cfg, device=dev, pattern=pat, seed=0)
    got.flat.copy_(ref.flat.to(dev))
    got.master.copy_(ref.master.to(dev))
    losses = []
    for m, d in ((ref, torch.device("cpu")), (got, dev)):
        pos = torch.arange(S, device=d)
        losses.append([m.train_step(ids_all[:-1].to(d), ids_all[1:].to(d), pos, n_total_tokens=S)
                       for _ in range(3)])
    A.check_status(dev)
    assert abs(losses[0][0] - math.log(cfg.vocab)) < 0.3, losses
    for a, b in zip(*losses):
        assert abs(a - b) < 3e-2, losses


def test_llama_offloaded_checkpoints_match(dev):
    """Keeping the layer checkpoints in pinned host memory must not change a training step."""
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.models.llama import LlamaConfig, LlamaModel
    from ultraattn_b200.ops import attention as A
    cfg = LlamaConfig(n_layers=3, hidden=256, n_heads=2, head_dim=128, ffn=512, vocab=1000)
    pat = P.causal(1)
    S = 1024
    g = torch.Generator().manual_seed(4)
    ids_all = torch.randint(0, cfg.vocab, (S + 1,), generator=g).to(dev)
    pos = torch.arange(S, device=dev)
    out = []
    for off in (False, True):
        m = LlamaModel(cfg, device=dev, pattern=pat, seed=1, offload_checkpoints=off)
        out.append([m.train_step(ids_all[:-1], ids_all[1:], pos, n_total_tokens=S) for _ in range(2)])
        if off:
            assert len(m._host_ckpt) == 2 * cfg.n_layers and all(h.is_pinned() for h in m._host_ckpt.values())
    A.check_status(dev)
    assert out[0] == out[1], out


def test_forward_and_dkdv_are_bitwise_reproducible(dev):
    """The forward and dK / dV have a fixed reduction order (one CTA owns each output tile), so
    two runs must agree bit for bit; dQ is summed by memory-side reductions in arrival order and
    is only required to agree to rounding."""
    import ultraattn_b200 as ua
    from ultraattn_b200 import patterns as P
    torch.manual_seed(11)
    S, H = 2048, 4
    pat = P.strided(8, 4, 2)
    q, k, v, d_o = (torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16) for _ in range(4))
    runs = []
    for _ in range(2):
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        o = ua.attention(qq, kk, vv, pat)
        o.backward(d_o)
        runs.append((o.detach().clone(), qq.grad.clone(), kk.grad.clone(), vv.grad.clone()))
    assert torch.equal(runs[0][0], runs[1][0])
    assert torch.equal(runs[0][2], runs[1][2]) and torch.equal(runs[0][3], runs[1][3])
    _close(runs[0][1], runs[1][1], 1e-2)
