"""bf16 GEMM on the tcgen05 kernel, with the optional all-to-all fusions of the head-parallel path.

``linear(x, w)`` computes ``x @ w.T`` like ``torch.nn.functional.linear``; the general
:func:`gemm` takes explicit storage orders so that the backward products ``dy @ w`` and
``dy.T @ x`` run without transposes. On CPU tensors the same functions fall back to an fp32
PyTorch matmul (the oracle of the kernel tests).
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from .. import _lib
from .attention import status_buffer

_sm_count: dict[int, int] = {}
# (M, N, K, a_is_km, b_is_kn) -> 1 if the CTA-pair form of the kernel was faster when first timed
_pair_choice: dict[tuple, int] = {}
_TUNE_MIN_FLOPS = 2.0 * 4096 * 4096 * 4096       # below this a launch is too short for the choice to matter


def _sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_is_km: bool = False, b_is_kn: bool = False,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """``C[M,N] = A[M,K] @ B[K,N]`` in bf16 with fp32 accumulation.

    ``a`` is stored ``[M,K]`` (default) or ``[K,M]`` (``a_is_km``); ``b`` is stored ``[N,K]``
    (default, the layout of a ``linear`` weight) or ``[K,N]`` (``b_is_kn``).
    """
    if a_is_km:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_is_kn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if not a.is_cuda:
        af = a.float().t() if a_is_km else a.float()
        bf = b.float() if b_is_kn else b.float().t()
        res = (af @ bf).to(a.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(1) == 1 and b.stride(1) == 1
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    assert out.stride(1) == 1
    lib = _lib.load()
    a_ptrs = (ctypes.c_void_p * 1)(a.data_ptr())
    c_ptrs = (ctypes.c_void_p * 1)(out.data_ptr())

    def launch():
        rc = lib.ua_gemm_bf16(a_ptrs, 1, a.shape[0], a.stride(0), 0, int(a_is_km), b.data_ptr(),
                              b.stride(0), int(b_is_kn), c_ptrs, 1, out.stride(0), 0, M, N, K,
                              status_buffer(a.device).data_ptr(), _sms(a.device),
                              torch.cuda.current_stream(a.device).cuda_stream)
        _lib.check(rc, "ua_gemm_bf16")

    lib.ua_gemm_pair_mode(_pick_form(lib, (M, N, K, bool(a_is_km), bool(b_is_kn)), launch, a.device))
    launch()
    return out


def _pick_form(lib, key: tuple, launch, device) -> int:
    """0 = one CTA per output tile, 1 = a pair of CTAs per 256 x 256 tile. The first large call of
    a shape times both forms (three launches each, CUDA events) and the choice is kept; nothing is
    timed while a CUDA graph is being captured."""
    if key in _pair_choice:
        return _pair_choice[key]
    M, N, K = key[:3]
    if 2.0 * M * N * K < _TUNE_MIN_FLOPS or torch.cuda.is_current_stream_capturing():
        return 0
    times = []
    for mode in (0, 1):
        lib.ua_gemm_pair_mode(mode)
        launch()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            launch()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    _pair_choice[key] = int(times[1] < 0.97 * times[0])
    return _pair_choice[key]


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x[..., K] @ w[N, K].T`` -> ``[..., N]``."""
    lead = x.shape[:-1]
    y = gemm(x.reshape(-1, x.shape[-1]), w, out=None if out is None else out.reshape(-1, w.shape[0]))
    return y.reshape(*lead, w.shape[0])


def gemm_scatter(a: torch.Tensor, b: torch.Tensor, dst_ptrs: Sequence[int], ldc: int,
                 dst_row_off: int, b_is_kn: bool = False) -> None:
    """``A[M,K] @ B`` (``b`` stored ``[N,K]``, or ``[K,N]`` with ``b_is_kn``) with the all-to-all
    fused into the epilogue: output columns are split into ``len(dst_ptrs)`` equal groups; group g
    is written to the buffer at ``dst_ptrs[g]`` (typically peer GPU g's receive buffer) at rows
    ``dst_row_off .. dst_row_off + M``."""
    M, K = a.shape
    N = b.shape[1] if b_is_kn else b.shape[0]
    assert (b.shape[0] if b_is_kn else b.shape[1]) == K
    lib = _lib.load()
    a_ptrs = (ctypes.c_void_p * 1)(a.data_ptr())
    c_ptrs = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    lib.ua_gemm_pair_mode(0)
    rc = lib.ua_gemm_bf16(a_ptrs, 1, M, a.stride(0), 0, 0, b.data_ptr(), b.stride(0), int(b_is_kn), c_ptrs,
                          len(dst_ptrs), ldc, dst_row_off, M, N, K,
                          status_buffer(a.device).data_ptr(), _sms(a.device),
                          torch.cuda.current_stream(a.device).cuda_stream)
    _lib.check(rc, "ua_gemm_bf16(scatter)")


def gemm_gather(src_ptrs: Sequence[int], src_rows_total: int, lda: int, a_row_off: int, M: int,
                k_per_src: int, b: torch.Tensor, out: torch.Tensor, b_is_kn: bool = False) -> torch.Tensor:
    """``A @ B`` (``b`` stored ``[N,K]``, or ``[K,N]`` with ``b_is_kn``) with the all-to-all fused
    into the operand load: the K dimension of A is the concatenation of ``len(src_ptrs)`` buffers
    (typically one per peer GPU, each ``[src_rows_total, k_per_src]`` bf16 with row stride
    ``lda``); rows ``a_row_off .. +M`` of every buffer are read directly by TMA."""
    K, N = b.shape if b_is_kn else (b.shape[1], b.shape[0])
    assert K == k_per_src * len(src_ptrs)
    lib = _lib.load()
    a_ptrs = (ctypes.c_void_p * len(src_ptrs))(*src_ptrs)
    c_ptrs = (ctypes.c_void_p * 1)(out.data_ptr())
    lib.ua_gemm_pair_mode(0)
    rc = lib.ua_gemm_bf16(a_ptrs, len(src_ptrs), src_rows_total, lda, a_row_off, 0, b.data_ptr(),
                          b.stride(0), int(b_is_kn), c_ptrs, 1, out.stride(0), 0, M, N, K,
                          status_buffer(out.device).data_ptr(), _sms(out.device),
                          torch.cuda.current_stream(out.device).cuda_stream)
    _lib.check(rc, "ua_gemm_bf16(gather)")
    return out
