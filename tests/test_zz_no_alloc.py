"""The allocation-free backward entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory where the backward has to run (inside
a stream capture or a latency-critical loop, as a guest in another program's process, or after
handing all free HBM to their own pool). ``ua_attn_bwd_dense_noalloc`` serves them: its scratch
is a fixed device array inside the library. This test calls it twice in a row — the array is
shared between calls and keeps the previous call's contents, so the second call checks that
everything that must start at zero is cleared — and compares dQ, dK, dV with the regular entry
point (caller-allocated scratch) within the tolerance of the other kernel tests. It also checks
that a problem larger than the built-in scratch is refused with a message instead of running.
The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(got, ref, tol):
    err = (got.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err <= tol * scale, f"max err {err} vs scale {scale}"


# each case is a series of (tokens, heads, kv heads) calls made one after the other on the shared scratch
CASES = {
    "same-shape-twice": [(2048, 4, 2), (2048, 4, 2)],
    "large-then-small-ragged": [(4096, 4, 4), (1000, 4, 2)],     # stale tails of the first call must not leak
    "at-the-size-limit": [(32768, 4, 4), (2048, 2, 1)],          # tokens * heads == 131072 exactly
}


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("case", list(CASES), ids=list(CASES))
def test_noalloc_backward_matches_regular_entry_point(case, causal):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA GPU")
    from ultraattn_b200 import _lib
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.ops import attention as A, elementwise as E
    lib = _lib.load()
    fn = lib.ua_attn_bwd_dense_noalloc              # the exported C symbol itself
    vp = ctypes.c_void_p
    fn.restype = ctypes.c_int
    fn.argtypes = [vp] * 9 + [ctypes.c_int] * 4 + [ctypes.c_float, vp, vp]
    dev = torch.device("cuda", 0)
    for call, (S, H, Hk) in enumerate(CASES[case]):  # calls in a row on the shared scratch
        torch.manual_seed(10 + call)
        q = torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16)
        k = torch.randn(1, S, Hk, 128, device=dev, dtype=torch.bfloat16)
        v = torch.randn(1, S, Hk, 128, device=dev, dtype=torch.bfloat16)
        d_o = torch.randn(1, S, H, 128, device=dev, dtype=torch.bfloat16)
        seg = A.Seg(0, 0, S, causal, 0)
        o = torch.empty_like(q)
        lse = torch.empty(1, H, S, device=dev, dtype=torch.float32)
        A.attn_fwd_cuda([q], [k], [v], [(o, lse)], A.FwdPlan([A.Row(0, 0, S, (seg,), 0, 0, False)], dev))
        dvec = E.rowdot(o[0], d_o[0]).unsqueeze(0)
        # regular entry point: scratch (fp32 dQ accumulator, launch tables) allocated by the caller
        dq32 = torch.zeros(1, S, H, 128, device=dev, dtype=torch.float32)
        dk_ref, dv_ref = torch.empty_like(k), torch.empty_like(v)
        A.attn_bwd_cuda([A.BwdQSide(q, d_o, lse, dvec, dq32)], [k], [v], [A.BwdKvOut(dk_ref, dv_ref)],
                        A.BwdPlan([A.Col(0, 0, S, (seg,), 0, 0)], dev))
        dq_ref = torch.empty_like(q)
        E.cast_scale(dq32, dq_ref)
        # allocation-free entry point: outputs only, everything else inside the library
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        st = A.status_buffer(dev)
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), d_o.data_ptr(), lse.data_ptr(), dvec.data_ptr(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), S, H, Hk, int(causal), 1.0 / 128 ** 0.5,
                st.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
        assert rc == 0, lib.ua_last_error().decode()
        torch.cuda.synchronize()
        A.check_status(dev)
        _close(dq, dq_ref, 2e-2)
        _close(dk, dk_ref, 2e-2)
        _close(dv, dv_ref, 2e-2)
        if S <= 1024:
            # and once against plain fp32 attention with autograd, so the test also stands alone
            pat = P.causal(1) if causal else P.full(1)
            _, _, dq_o, dk_o, dv_o = P.dense_attention_with_grads(q.cpu().float(), k.cpu().float(), v.cpu().float(),
                                                                  d_o.cpu().float(), pat)
            _close(dq.cpu(), dq_o, 2e-2)
            _close(dk.cpu(), dk_o, 2e-2)
            _close(dv.cpu(), dv_o, 2e-2)
    # beyond the built-in scratch: refused, nothing launched
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), d_o.data_ptr(), lse.data_ptr(), dvec.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), 1 << 20, H, Hk, int(causal), 0.1, None,
            torch.cuda.current_stream(dev).cuda_stream)
    assert rc != 0 and b"exceeds the built-in scratch" in lib.ua_last_error()
