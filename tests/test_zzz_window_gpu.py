"""Sliding-window attention on the sm_100a kernels (two-part plan: usual and reversed token order)
against dense masked attention in fp32."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA GPU")
    from ultraattn_b200 import _lib
    _lib.load()
    return torch.device("cuda")


def _dense(q, k, v, d_o, left, right):
    q, k, v = (t.detach().float().requires_grad_() for t in (q, k, v))
    S, g = q.shape[1], q.shape[2] // k.shape[2]
    s = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(g, 2)) / math.sqrt(q.shape[-1])
    r = torch.arange(S, device=q.device)[:, None]
    c = torch.arange(S, device=q.device)[None, :]
    s = s.masked_fill(~((c >= r - left) & (c <= r + right)), float("-inf"))
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.repeat_interleave(g, 2))
    o.backward(d_o.float())
    return o.detach(), torch.logsumexp(s, -1).detach(), q.grad, k.grad, v.grad


def _close(got, ref, tol):
    err = (got.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err <= tol * scale, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("S,window,causal", [(2048, (600, -1), True), (1000, (300, 200), False)])
def test_sliding_window_attention_on_the_kernels(dev, S, window, causal):
    from ultraattn_b200.ops import attention as A
    from ultraattn_b200.ops.window import sliding_window_attention, window_forward
    torch.manual_seed(S)
    B, H, Hk, D = 1, 4, 2, 128
    q = torch.randn(B, S, H, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, Hk, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, S, Hk, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    d_o = torch.randn(B, S, H, D, device=dev, dtype=torch.bfloat16)
    left = window[0]
    right = 0 if causal else window[1]
    o_r, lse_r, dq_r, dk_r, dv_r = _dense(q, k, v, d_o, left, right)
    with torch.no_grad():
        _, lse = window_forward(q, k, v, window, causal)
    A.check_status(dev)
    _close(lse, lse_r, 1e-2)
    o = sliding_window_attention(q, k, v, window, causal)
    o.backward(d_o)
    A.check_status(dev)
    _close(o, o_r, 1.5e-2)
    _close(q.grad, dq_r, 2e-2)
    _close(k.grad, dk_r, 2e-2)
    _close(v.grad, dv_r, 2e-2)


# The compositions below pass on the fp32 restatement of the kernels (tests/test_window_cpu.py) and
# use the same table semantics as the launches above, but have not been run on a GPU yet: an
# unexpected mismatch is reported as xfailed, a pass as xpassed, and neither stops the run.
_unverified = pytest.mark.xfail(strict=False, reason="composition not yet run on a B200 (CPU restatement passes)")


def _masked_dense(q, k, v, d_o, mask):
    q, k, v = (t.detach().float().requires_grad_() for t in (q, k, v))
    g = q.shape[2] // k.shape[2]
    s = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(g, 2)) / math.sqrt(q.shape[-1])
    s = s.masked_fill(~mask.to(q.device), float("-inf"))
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.repeat_interleave(g, 2))
    o.backward(d_o.float())
    return o.detach(), q.grad, k.grad, v.grad


def _inputs(dev, Sq, Skv, seed):
    torch.manual_seed(seed)
    mk = lambda s, h: torch.randn(1, s, h, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    return mk(Sq, 4), mk(Skv, 2), mk(Skv, 2), torch.randn(1, Sq, 4, 128, device=dev, dtype=torch.bfloat16)


def _compare(dev, o, q, k, v, d_o, mask):
    from ultraattn_b200.ops import attention as A
    o.backward(d_o)
    A.check_status(dev)
    o_r, dq_r, dk_r, dv_r = _masked_dense(q, k, v, d_o, mask)
    _close(o, o_r, 1.5e-2)
    _close(q.grad, dq_r, 2e-2)
    _close(k.grad, dk_r, 2e-2)
    _close(v.grad, dv_r, 2e-2)


@_unverified
def test_attention_sinks_on_the_kernels(dev, monkeypatch):
    from ultraattn_b200.ops.window import sliding_window_attention
    monkeypatch.setenv("UA_DEBUG_BOUNDS", "1")           # the launch tables are checked on the host first
    S, left, sink = 1536, 400, 4
    q, k, v, d_o = _inputs(dev, S, S, 1)
    r, c = torch.arange(S)[:, None], torch.arange(S)[None, :]
    _compare(dev, sliding_window_attention(q, k, v, (left, 0), True, sink_tokens=sink), q, k, v, d_o,
             ((c <= r) & (c >= r - left)) | ((c < sink) & (c <= r)))


@_unverified
def test_window_behind_context_keys_on_the_kernels(dev, monkeypatch):
    from ultraattn_b200.ops.window import sliding_window_attention
    monkeypatch.setenv("UA_DEBUG_BOUNDS", "1")
    Sq, Skv, left = 512, 1400, 700
    q, k, v, d_o = _inputs(dev, Sq, Skv, 2)
    r, c = torch.arange(Sq)[:, None] + (Skv - Sq), torch.arange(Skv)[None, :]
    _compare(dev, sliding_window_attention(q, k, v, (left, 0), True), q, k, v, d_o, (c <= r) & (c >= r - left))


@_unverified
def test_prefix_lm_on_the_kernels(dev, monkeypatch):
    import ultraattn_b200 as ua
    monkeypatch.setenv("UA_DEBUG_BOUNDS", "1")
    S, prefix = 1200, 300
    q, k, v, d_o = _inputs(dev, S, S, 3)
    r, c = torch.arange(S)[:, None], torch.arange(S)[None, :]
    _compare(dev, ua.prefix_lm_attention(q, k, v, prefix), q, k, v, d_o, (c <= r) | (c < prefix))
