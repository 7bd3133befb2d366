"""The graph-replay runtime mode (runtime/graphed.py) on CPU: there it runs its two passes eagerly,
so the static-buffer bookkeeping, the autograd wrapper and its misuse check are testable without a
GPU. The replay itself is tested on a B200 in tests/test_z_graph_offload_gpu.py."""
import pytest
import torch

import ultraattn_b200 as ua
from ultraattn_b200 import patterns as P
from ultraattn_b200.runtime import GraphedAttention


def test_matches_the_eager_operator_and_reuses_its_buffers():
    torch.manual_seed(0)
    pat = P.strided(4, 2, 1)
    S, H, D = 256, 2, 32
    run = GraphedAttention(pat, S, H, D, device="cpu", dtype=torch.float32)
    for it in range(2):
        q, k, v = (torch.randn(1, S, H, D, requires_grad=True) for _ in range(3))
        d_o = torch.randn(1, S, H, D)
        ua.attention(q, k, v, pat).backward(d_o)
        want = [t.grad.clone() for t in (q, k, v)]
        q2, k2, v2 = (t.detach().clone().requires_grad_() for t in (q, k, v))
        o = run(q2, k2, v2)
        assert torch.allclose(o, ua.attention(q, k, v, pat).detach(), atol=1e-5)
        o.backward(d_o)
        for got, ref in zip((q2.grad, k2.grad, v2.grad), want):
            assert torch.allclose(got, ref, atol=1e-4), (got - ref).abs().max()
    assert run.replays == {"fwd": 2, "bwd": 2}
    # writing straight into the static buffers skips the copies
    bufs = run.inputs()
    bufs["q"].normal_()
    o, lse = run.forward(bufs["q"], bufs["k"], bufs["v"])
    assert o.data_ptr() == run.o.data_ptr() and lse.shape == (1, H, S)


def test_backward_of_an_overwritten_call_is_refused_and_shapes_are_checked():
    pat = P.causal(1)
    run = GraphedAttention(pat, 128, 1, 32, device="cpu", dtype=torch.float32)
    q, k, v = (torch.randn(1, 128, 1, 32, requires_grad=True) for _ in range(3))
    first = run(q, k, v)
    run(q.detach(), k.detach(), v.detach())            # a second forward overwrites the buffers
    with pytest.raises(RuntimeError, match="another forward ran"):
        first.sum().backward()
    with pytest.raises(AssertionError, match="built for"):
        run.forward(torch.randn(1, 64, 1, 32), k.detach(), v.detach())
