"""CUDA-graph replay of the attention kernels and the host-offloaded checkpoint on CUDA tensors
(run on a B200)."""
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
    err = (got.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err <= tol * scale, f"max err {err} vs scale {scale}"


def test_forward_backward_replay_in_cuda_graph(dev):
    """Forward, D pre-pass and backward captured once on a side stream into a CUDA graph and
    replayed on new inputs (the reference checks the same for its flash-attention call,
    tests/test_cuda_graph.py:48-164): the launches take no host-side tables at replay time, so a
    per-rank kernel list can be frozen into a graph."""
    from ultraattn_b200.ops import attention as A, elementwise as E
    torch.manual_seed(11)
    S, H = 512, 2
    tab = np.array([[2, 0], [1, 2]])
    q, k, v, d_o = (torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16) for _ in range(4))
    o = torch.zeros_like(q)
    lse = torch.zeros(1, H, S, device=dev)
    dvec = torch.zeros(1, H, S, device=dev)
    dq = torch.zeros(1, S, H, 128, device=dev)
    dk = torch.zeros(1, S, H, 128, device=dev, dtype=torch.bfloat16)
    dv = torch.zeros_like(dk)
    rows, cols = A.rows_from_block_table(tab, 256), A.cols_from_block_table(tab, 256)
    fplan, bplan = A.FwdPlan(rows, dev), A.BwdPlan(cols, dev)

    def step():
        A.attn_fwd_cuda([q], [k], [v], [(o, lse)], fplan)
        E.rowdot(o[0], d_o[0], dvec[0])
        dq.zero_()
        A.attn_bwd_cuda([A.BwdQSide(q, d_o, lse, dvec, dq)], [k], [v], [A.BwdKvOut(dk, dv)], bplan)

    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        step()                                   # warm-up: one-time set-up happens outside capture
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    for seed in (12, 13):
        g = torch.Generator(device=dev).manual_seed(seed)
        for t in (q, k, v, d_o):
            t.copy_(torch.randn(t.shape, device=dev, generator=g).to(torch.bfloat16))
        graph.replay()
        torch.cuda.synchronize(dev)
        A.check_status(dev)
        o_r = torch.zeros(1, S, H, 128, device=dev)
        lse_r = torch.zeros(1, H, S, device=dev)
        A.attn_fwd_reference([q], [k], [v], [(o_r, lse_r)], rows)
        dvec_r = (o_r * d_o.float()).sum(-1).permute(0, 2, 1).contiguous()
        dq_r = torch.zeros_like(dq)
        dk_r = torch.zeros(1, S, H, 128, device=dev)
        dv_r = torch.zeros_like(dk_r)
        A.attn_bwd_reference([A.BwdQSide(q, d_o, lse_r, dvec_r, dq_r)], [k], [v], [A.BwdKvOut(dk_r, dv_r)], cols)
        _close(o, o_r, 1e-2)
        _close(dq, dq_r, 2e-2)
        _close(dk, dk_r, 2e-2)
        _close(dv, dv_r, 2e-2)


def test_graphed_attention_runtime_mode(dev):
    """`runtime.GraphedAttention`: forward and backward replay from graphs on new inputs, match the
    eager operator, encode no tensor map and upload no table after construction, and cost less host
    time per step than the eager path on a launch-bound shape."""
    import time
    import ultraattn_b200 as ua
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.ops import attention as A
    from ultraattn_b200.runtime import GraphedAttention
    pat = P.strided(4, 2, 1)
    S, H = 1024, 2
    run = GraphedAttention(pat, S, H, 128, device=dev)
    for seed in (21, 22):
        g = torch.Generator(device=dev).manual_seed(seed)
        q, k, v, d_o = (torch.randn(1, S, H, 128, device=dev, generator=g).to(torch.bfloat16) for _ in range(4))
        qe, ke, ve = (t.clone().requires_grad_() for t in (q, k, v))
        ua.attention(qe, ke, ve, pat).backward(d_o)
        qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
        o = run(qg, kg, vg)
        o.backward(d_o)
        torch.cuda.synchronize(dev)
        A.check_status(dev)
        _close(o, ua.attention(q, k, v, pat), 1e-2)
        for got, ref in ((qg.grad, qe.grad), (kg.grad, ke.grad), (vg.grad, ve.grad)):
            _close(got, ref, 2e-2)
    bufs = run.inputs()
    torch.cuda.synchronize(dev)
    _, misses1 = A.tensor_map_cache_stats()

    def host_seconds(fn, n=50):
        fn()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        dt = time.perf_counter() - t0
        torch.cuda.synchronize(dev)
        return dt / n

    def replayed():
        run.forward(bufs["q"], bufs["k"], bufs["v"])
        run.backward(bufs["d_o"])

    def eager():
        run._fwd_step()
        run._bwd_step()

    t_replay, t_eager = host_seconds(replayed), host_seconds(eager)
    _, misses2 = A.tensor_map_cache_stats()
    assert misses2 == misses1                      # static buffers: every map was encoded at construction
    assert t_replay < t_eager, (t_replay, t_eager)
    print(f"host time per fwd+bwd step: replay {t_replay * 1e6:.1f} us, eager {t_eager * 1e6:.1f} us")


def test_offloaded_checkpoint_on_gpu(dev):
    """The generic host-offloaded checkpoint (pinned copy on a side stream) on CUDA tensors."""
    from ultraattn_b200.models.glue import OffloadedCheckpoint
    torch.manual_seed(14)
    lin = torch.nn.Linear(256, 256).to(dev)
    layer = lambda h, scale: torch.tanh(lin(h)) * scale
    x = torch.randn(1024, 256, device=dev, requires_grad=True)
    layer(x, 2.0).sum().backward()
    gx, gw = x.grad.clone(), lin.weight.grad.clone()
    x.grad = None
    lin.weight.grad = None
    OffloadedCheckpoint.apply(layer, x, 2.0).sum().backward()
    assert torch.allclose(x.grad, gx, atol=1e-5) and torch.allclose(lin.weight.grad, gw, atol=1e-3, rtol=1e-4)


def test_start_gate_holds_and_releases_the_stream(dev):
    """Work queued behind a closed gate does not run until the host opens it; the timing harness
    with the gate gives a sane number; a gate that is never opened gives up after its budget."""
    import time
    from ultraattn_b200.drivers.benchmark import benchmark_ops
    from ultraattn_b200.ops import attention as A
    from ultraattn_b200.ops.gate import StartGate
    A.status_buffer(dev).zero_()
    gate = StartGate(dev, budget_s=3.0)
    x = torch.zeros(1024, device=dev)
    torch.cuda.synchronize(dev)
    gate.close()
    x.add_(1)
    done = torch.cuda.Event()
    done.record()
    time.sleep(0.05)
    assert not done.query(), "the kernel behind the gate ran before the gate was opened"
    gate.open()
    torch.cuda.synchronize(dev)
    assert gate.check() and x.sum().item() == 1024
    A.check_status(dev)
    y = torch.randn(1 << 20, device=dev)
    t = benchmark_ops(lambda: y.mul_(1.0001), warmup=2, num_iter=20, repeats=2, device=dev, start_gate=True)
    assert 0 < t < 1e-2
    A.check_status(dev)
    short = StartGate(dev, budget_s=0.1)
    short.close()
    torch.cuda.synchronize(dev)                       # never opened: returns after its budget
    assert not short.check() and short.timed_out
    A.check_status(dev)                               # and leaves no error behind


def test_reference_kernel_calls_on_gpu(dev):
    """The forked-flash-attention signatures on the sm_100a kernels: rectangular causal (mask
    aligned bottom-right), caller-named output, precomputed D with a dummy O, packed batch."""
    import math
    from ultraattn_b200.ops import attention as A
    from ultraattn_b200.ops.flash_compat import (_flash_attn_backward, _flash_attn_forward,
                                                 _flash_attn_varlen_backward, _flash_attn_varlen_forward)

    def dense(q, k, v, d_o, causal):            # [S, H, D] fp32 on the CPU
        q, k, v = (t.detach().float().cpu().clone().requires_grad_() for t in (q, k, v))
        g = q.shape[1] // k.shape[1]
        s = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(g, 1)) / math.sqrt(q.shape[-1])
        if causal:
            sq, sk = q.shape[0], k.shape[0]
            s = s.masked_fill(~(torch.arange(sk)[None, :] <= torch.arange(sq)[:, None] + (sk - sq))[None], float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v.repeat_interleave(g, 1))
        o.backward(d_o.float().cpu())
        return o.detach(), q.grad, k.grad, v.grad

    torch.manual_seed(15)
    Sq, Skv, H, Hk = 256, 384, 4, 2
    mk = lambda s, h: torch.randn(1, s, h, 128, device=dev, dtype=torch.bfloat16)
    q, d_o, k, v = mk(Sq, H), mk(Sq, H), mk(Skv, Hk), mk(Skv, Hk)
    o_ref, dq_ref, dk_ref, dv_ref = dense(q[0], k[0], v[0], d_o[0], True)
    buf = torch.empty_like(q)
    ret = _flash_attn_forward(q, k, v, 0.0, None, True, (-1, -1), None, False, out=buf)
    assert ret[0] is buf
    _close(buf[0].cpu(), o_ref, 1e-2)
    dvec = (buf.float() * d_o.float()).sum(-1).permute(0, 2, 1).contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    _flash_attn_backward(d_o, q, k, v, q, ret[5], dq, dk, dv, 0.0, None, True, (-1, -1), None, False, None,
                         softmax_d=dvec)
    torch.cuda.synchronize(dev)
    A.check_status(dev)
    _close(dq[0].cpu(), dq_ref, 2e-2)
    _close(dk[0].cpu(), dk_ref, 2e-2)
    _close(dv[0].cpu(), dv_ref, 2e-2)
    cu = [0, 256, 256, 640, 768]
    T = cu[-1]
    qp, kp, vp, dop = (torch.randn(T, H, 128, device=dev, dtype=torch.bfloat16) for _ in range(4))
    r = _flash_attn_varlen_forward(qp, kp, vp, cu, cu, 384, 384, 0.0, None, True)
    dq, dk, dv = torch.empty_like(qp), torch.empty_like(kp), torch.empty_like(vp)
    _flash_attn_varlen_backward(dop, qp, kp, vp, r[0], r[5], dq, dk, dv, cu, cu, 384, 384, 0.0, None, True)
    torch.cuda.synchronize(dev)
    A.check_status(dev)
    for a, b in zip(cu[:-1], cu[1:]):
        if b > a:
            o_ref, dq_ref, dk_ref, dv_ref = dense(qp[a:b], kp[a:b], vp[a:b], dop[a:b], True)
            _close(r[0][a:b].cpu(), o_ref, 1e-2)
            _close(dq[a:b].cpu(), dq_ref, 2e-2)
            _close(dk[a:b].cpu(), dk_ref, 2e-2)
            _close(dv[a:b].cpu(), dv_ref, 2e-2)


@pytest.mark.skipif(__import__("os").environ.get("UA_TEST_RANDOM_PLANS") != "1",
                    reason="opt-in (UA_TEST_RANDOM_PLANS=1): randomised launch plans against the fp32 restatement")
def test_random_launch_plans_against_the_restatement(dev):
    """Seeded random forward plans (several query blocks, several key segments each, arbitrary
    offsets and lengths inside the tensors, causal diagonals) on the sm_100a kernel against the
    fp32 restatement of the same plan."""
    import random
    from ultraattn_b200.ops import attention as A
    T, H = 2048, 2
    torch.manual_seed(16)
    q, k, v = (torch.randn(1, T, H, 128, device=dev, dtype=torch.bfloat16) for _ in range(3))
    for seed in range(6):
        rng = random.Random(seed)
        rows, used = [], 0
        while used < T and len(rows) < 5:
            q_len = min(T - used, rng.choice([64, 128, 200, 256, 512]))
            segs = []
            for _ in range(rng.randint(1, 3)):
                start = rng.randrange(0, T - 64)
                length = rng.randint(32, min(768, T - start))
                segs.append(A.Seg(0, start, length, rng.random() < 0.5, rng.choice([-1, 0, 0, 64])))
            rows.append(A.Row(0, used, q_len, tuple(segs), 0, used, False))
            used += q_len
        o = torch.zeros_like(q)
        lse = torch.full((1, H, T), float("-inf"), device=dev)
        A.attn_fwd_cuda([q], [k], [v], [(o, lse)], A.FwdPlan(rows, dev))
        o_ref = torch.zeros(1, T, H, 128, device=dev)
        lse_ref = torch.full((1, H, T), float("-inf"), device=dev)
        A.attn_fwd_reference([q], [k], [v], [(o_ref, lse_ref)], rows)
        torch.cuda.synchronize(dev)
        A.check_status(dev)
        _close(o[:, :used], o_ref[:, :used], 1.5e-2)
        fin = torch.isfinite(lse_ref)
        assert (lse[fin] - lse_ref[fin]).abs().max().item() < 3e-3, seed
