"""ctypes loader for the in-tree sm_100a kernel library.

The library is loaded lazily the first time a kernel is needed. If it has not been built yet it is
built on the spot; if that is impossible an ImportError is raised — there is no silent fallback to
another implementation on a GPU machine.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_long, c_void_p

from . import build as _build

_lib = None
LAUNCHES = [0]      # kernels of this library launched so far (every wrapper reports here)


class UaTensorSrc(Structure):
    _fields_ = [("ptr", c_void_p), ("tokens", c_long), ("heads", c_long), ("batch", c_long),
                ("token_stride", c_long), ("head_stride", c_long), ("batch_stride", c_long)]


class UaOutDst(Structure):
    _fields_ = [("o_ptr", c_void_p), ("lse_ptr", c_void_p), ("o_row_stride", c_long),
                ("o_batch_stride", c_long), ("lse_head_stride", c_long),
                ("lse_batch_stride", c_long)]


class UaBwdQSide(Structure):
    _fields_ = [("lse", c_void_p), ("dvec", c_void_p), ("lse_head_stride", c_long),
                ("lse_batch_stride", c_long), ("dq", c_void_p), ("dq_row_stride", c_long),
                ("dq_batch_stride", c_long)]


class UaBwdKvOut(Structure):
    _fields_ = [("dk", c_void_p), ("dv", c_void_p), ("row_stride", c_long),
                ("batch_stride", c_long), ("add_f32", c_int), ("pad", c_int)]


def _declare(lib):
    vp, i, l, f = c_void_p, c_int, c_long, c_float
    lib.ua_last_error.restype = c_char_p
    lib.ua_last_error.argtypes = []
    sigs = {
        "ua_gemm_bf16": [POINTER(vp), i, l, i, i, i, vp, i, i, POINTER(vp), i, i, i, i, i, i, vp, i,
                         vp],
        "ua_attn_fwd": [POINTER(UaTensorSrc), i, POINTER(UaTensorSrc), POINTER(UaTensorSrc), i,
                        POINTER(UaOutDst), i, vp, vp, vp, i, i, i, i, f, vp, vp, i, i, vp, i, vp, vp],
        "ua_attn_bwd": [POINTER(UaTensorSrc), POINTER(UaTensorSrc), POINTER(UaBwdQSide), i,
                        POINTER(UaTensorSrc), POINTER(UaTensorSrc), i, POINTER(UaBwdKvOut), i,
                        vp, vp, vp, i, i, i, i, f, vp, vp, i, i, vp, i, vp, vp],
        "ua_barrier": [POINTER(vp), i, i, i, ctypes.c_uint, ctypes.c_double, vp, vp],
        "ua_xent_fwd": [vp, vp, vp, vp, l, l, i, vp],
        "ua_xent_bwd": [vp, vp, vp, vp, l, l, i, vp],
        "ua_peer_add_f32": [vp, vp, l, i, i, vp],
        "ua_peer_pull": [vp, vp, l, i, vp],
        "ua_multimem_bcast": [vp, vp, l, i, vp],
        "ua_multimem_reduce": [vp, vp, vp, l, i, i, vp],
        "ua_wait_flag": [vp, ctypes.c_uint, ctypes.c_double, vp, vp],
        "ua_lse_merge": [POINTER(vp), POINTER(vp), POINTER(l), POINTER(l), i, vp, vp, l, l, i, i,
                         vp],
        "ua_rowdot": [vp, vp, vp, l, l, l, i, i, vp],
        "ua_cast_scale": [vp, vp, l, f, i, vp],
        "ua_rmsnorm_fwd": [vp, vp, vp, vp, i, i, f, vp],
        "ua_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, i, i, vp],
        "ua_add_rmsnorm_fwd": [vp, vp, vp, vp, vp, vp, i, i, f, vp],
        "ua_rmsnorm_bwd_res": [vp, vp, vp, vp, vp, vp, vp, i, i, vp],
        "ua_rope": [vp, vp, vp, vp, vp, l, i, l, l, i, vp],
        "ua_swiglu_fwd": [vp, vp, l, i, vp],
        "ua_swiglu_bwd": [vp, vp, vp, l, i, vp],
        "ua_adam": [vp, vp, vp, vp, vp, l, f, f, f, f, f, i, f, vp],
        "ua_mma_rate": [i, i, i, i, vp, vp, vp],
    }
    if hasattr(lib, "ua_gemm_pair_mode"):
        lib.ua_gemm_pair_mode.restype = None
        lib.ua_gemm_pair_mode.argtypes = [c_int]
    for name, args in sigs.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = c_int
            fn.argtypes = args
    return lib


def load():
    """Return the loaded library, (re)building it first when it is missing or older than any of
    its sources or headers: the ctypes structures of this module mirror structs of those headers,
    so a stale binary must never be loaded."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if os.environ.get("UA_LIB_PATH"):           # explicit library file (development builds)
        _lib = _declare(ctypes.CDLL(os.environ["UA_LIB_PATH"]))
        return _lib
    try:
        # cheap when the library is up to date (a few stat calls); takes a lock when it builds
        _build.build_all(force=os.environ.get("UA_REBUILD") == "1")
    except Exception as e:  # noqa: BLE001
        if not path.exists():
            raise ImportError(f"ultraattn_b200: kernel library missing and build failed: {e}") from e
        raise ImportError(f"ultraattn_b200: kernel library is older than its sources and the rebuild failed: {e}") from e
    _lib = _declare(ctypes.CDLL(str(path)))
    return _lib


def check(rc: int, what: str) -> None:
    LAUNCHES[0] += 1
    if rc != 0:
        msg = load().ua_last_error().decode(errors="replace")
        raise RuntimeError(f"{what} failed: {msg}")


def available() -> bool:
    """True when CUDA kernels can run here (a GPU is visible)."""
    import torch
    return torch.cuda.is_available()
