"""The flash-attention 2.5 private API, as the reference calls it, on top of the stock flash_attn
2.8 that is installed.

The reference was written against a fork of flash-attention 2.5.7 whose source is not shipped with
it. It calls

    _flash_attn_forward(q, k, v, dropout_p, softmax_scale, causal=, window_size=(l, r),
                        alibi_slopes=, return_softmax=, out=)  ->  8-tuple
    _flash_attn_backward(dout, q, k, v, out, lse, dq, dk, dv, dropout_p, softmax_scale, causal,
                         window_size, alibi_slopes, deterministic, rng_state=, softmax_d=)

(the ``out=`` and ``softmax_d=`` arguments are the fork's additions). flash_attn 2.8 changed both
signatures (separate window arguments, ``softcap``, a 4-tuple). ``install()`` rebinds the two names
in ``flash_attn.flash_attn_interface`` to adapters that forward to the stock CUDA entry points
``flash_attn_2_cuda.fwd`` / ``.bwd``: the kernels that run are flash-attention's own, nothing of
this repository's. ``out=`` is honoured (the stock entry point takes an output tensor).
``softmax_d=`` is accepted and ignored: the stock backward recomputes rowsum(dO * O) from the
``out`` it is given, which costs one small extra pass and leaves the attention kernels unchanged.
"""
from __future__ import annotations


def install() -> None:
    import flash_attn.flash_attn_interface as iface
    import flash_attn_2_cuda as cuda_impl

    def _contig(x):
        return x if x is None or x.stride(-1) == 1 else x.contiguous()

    def _flash_attn_forward(q, k, v, dropout_p, softmax_scale, causal, window_size=(-1, -1),
                            alibi_slopes=None, return_softmax=False, out=None):
        q, k, v = _contig(q), _contig(k), _contig(v)
        o, lse, s_dmask, rng_state = cuda_impl.fwd(
            q, k, v, out, alibi_slopes, dropout_p, softmax_scale, causal,
            window_size[0], window_size[1], 0.0, return_softmax, None)
        return o, q, k, v, o, lse, s_dmask, rng_state

    def _flash_attn_backward(dout, q, k, v, out, softmax_lse, dq, dk, dv, dropout_p, softmax_scale,
                             causal, window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                             rng_state=None, softmax_d=None):
        dout, q, k, v, out = (_contig(x) for x in (dout, q, k, v, out))
        dq, dk, dv, d = cuda_impl.bwd(
            dout, q, k, v, out, softmax_lse, dq, dk, dv, alibi_slopes, dropout_p, softmax_scale,
            causal, window_size[0], window_size[1], 0.0, deterministic, None, rng_state)
        return dq, dk, dv, d

    iface._flash_attn_forward = _flash_attn_forward
    iface._flash_attn_backward = _flash_attn_backward
