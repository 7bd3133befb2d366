"""NCCL through ctypes: a communicator whose every call takes the CUDA stream as an argument.

``torch.distributed`` hides the stream (it uses its own and synchronises with the current one) and
adds a few microseconds of Python and c10d bookkeeping per call. A launch plan that issues one
send / recv per tile wants neither: it owns three streams and orders them with events. This module
binds the NCCL library that PyTorch already ships (no second copy of NCCL in the process, hence no
second set of NVLink / NVLS resources) and builds communicators over arbitrary rank lists, with the
unique id carried by any existing (CPU) process group or store.

Counterpart of the reference's ``NCCLLibrary`` / ``PyNcclCommunicator``
(tests/distributed/device_communicators/pynccl_wrapper.py:126-327, pynccl.py:17-322), which load a
privately built libnccl 2.21.5 from a fixed path. Differences: the library is located through the
``nvidia.nccl`` wheel or ``UA_NCCL_LIBRARY``; the table below also covers ``ncclBroadcast``,
``ncclCommAbort``, ``ncclCommCount`` / ``ncclCommUserRank`` and ``ncclCommGetAsyncError`` (so a
failed peer can be detected and the communicator torn down without waiting on it); calls inside
``group()`` are batched by NCCL itself (``ncclGroupStart`` / ``ncclGroupEnd``).

The fused runtime does not use NCCL at all; this binding serves the NCCL launch-plan executor, the
ring baselines and anything else that wants explicit streams.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from pathlib import Path
from typing import Optional, Sequence

import torch
import torch.distributed as dist

ncclResult_t = ctypes.c_int
ncclComm_t = ctypes.c_void_p
cudaStream_t = ctypes.c_void_p
NCCL_UNIQUE_ID_BYTES = 128


class ncclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * NCCL_UNIQUE_ID_BYTES)]


# ncclDataType_t / ncclRedOp_t values of nccl.h (stable since NCCL 2.10)
DTYPES = {
    torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4,
    torch.float16: 6, torch.float32: 7, torch.float64: 8, torch.bfloat16: 9,
}
RED_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}

# name -> (restype, argtypes)
_SIGNATURES = {
    "ncclGetErrorString": (ctypes.c_char_p, [ncclResult_t]),
    "ncclGetVersion": (ncclResult_t, [ctypes.POINTER(ctypes.c_int)]),
    "ncclGetUniqueId": (ncclResult_t, [ctypes.POINTER(ncclUniqueId)]),
    "ncclCommInitRank": (ncclResult_t, [ctypes.POINTER(ncclComm_t), ctypes.c_int, ncclUniqueId, ctypes.c_int]),
    "ncclCommDestroy": (ncclResult_t, [ncclComm_t]),
    "ncclCommAbort": (ncclResult_t, [ncclComm_t]),
    "ncclCommCount": (ncclResult_t, [ncclComm_t, ctypes.POINTER(ctypes.c_int)]),
    "ncclCommUserRank": (ncclResult_t, [ncclComm_t, ctypes.POINTER(ctypes.c_int)]),
    "ncclCommGetAsyncError": (ncclResult_t, [ncclComm_t, ctypes.POINTER(ncclResult_t)]),
    "ncclAllReduce": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                     ncclComm_t, cudaStream_t]),
    "ncclAllGather": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ncclComm_t,
                                     cudaStream_t]),
    "ncclReduceScatter": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                         ncclComm_t, cudaStream_t]),
    "ncclBroadcast": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                     ncclComm_t, cudaStream_t]),
    "ncclSend": (ncclResult_t, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
    "ncclRecv": (ncclResult_t, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
    "ncclGroupStart": (ncclResult_t, []),
    "ncclGroupEnd": (ncclResult_t, []),
}


class NcclError(RuntimeError):
    pass


def find_nccl_library() -> str:
    """Path of the NCCL shared library to bind: ``UA_NCCL_LIBRARY`` if set, else the one of the
    ``nvidia.nccl`` wheel that PyTorch links against, else the bare soname (system search path)."""
    env = os.environ.get("UA_NCCL_LIBRARY")
    if env:
        return env
    try:
        import nvidia.nccl as pkg
        for root in list(getattr(pkg, "__path__", [])):
            hits = sorted(Path(root).glob("lib/libnccl.so*"))
            if hits:
                return str(hits[0])
    except ImportError:
        pass
    return "libnccl.so.2"


class NcclLibrary:
    """The bound functions, each checked: a non-zero ``ncclResult_t`` raises :class:`NcclError` with
    NCCL's own text. One instance per library path and process."""

    _instances: dict = {}

    def __new__(cls, path: Optional[str] = None):
        path = path or find_nccl_library()
        if path not in cls._instances:
            self = super().__new__(cls)
            self.path = path
            self.lib = ctypes.CDLL(path)
            self.fn = {}
            for name, (res, args) in _SIGNATURES.items():
                f = getattr(self.lib, name)
                f.restype, f.argtypes = res, args
                self.fn[name] = f
            cls._instances[path] = self
        return cls._instances[path]

    def error_string(self, code: int) -> str:
        return self.fn["ncclGetErrorString"](code).decode()

    def check(self, code: int, what: str) -> None:
        if code != 0:
            raise NcclError(f"{what}: {self.error_string(code)} (ncclResult_t {code})")

    def version(self) -> tuple:
        """(major, minor, patch)."""
        v = ctypes.c_int(0)
        self.check(self.fn["ncclGetVersion"](ctypes.byref(v)), "ncclGetVersion")
        n = v.value
        return (n // 10000, (n % 10000) // 100, n % 100) if n >= 10000 else (n // 1000, (n % 1000) // 100, n % 100)

    def unique_id(self) -> bytes:
        uid = ncclUniqueId()
        self.check(self.fn["ncclGetUniqueId"](ctypes.byref(uid)), "ncclGetUniqueId")
        return bytes(bytearray(uid.internal))

    @staticmethod
    def unique_id_from_bytes(raw: bytes) -> ncclUniqueId:
        assert len(raw) == NCCL_UNIQUE_ID_BYTES
        uid = ncclUniqueId()
        ctypes.memmove(ctypes.byref(uid), raw, NCCL_UNIQUE_ID_BYTES)
        return uid


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


class NcclCommunicator:
    """An NCCL communicator over ``ranks`` (global ranks, any order; position in the list = rank
    inside the communicator), bound to ``device``. Construction is collective over the members:
    the first member makes the unique id and ``control_group`` (any process group that carries
    Python objects, e.g. gloo) or ``store`` (a ``torch.distributed`` key-value store) hands it to the
    others. Every operation takes ``stream`` (default: the current stream of ``device``) and only
    enqueues work there, so calls may be captured into a CUDA graph."""

    def __init__(self, ranks: Sequence[int], device, control_group=None, store=None, tag: str = "",
                 library: Optional[NcclLibrary] = None):
        self.nccl = library or NcclLibrary()
        self.ranks = list(ranks)
        self.device = torch.device(device)
        me = dist.get_rank() if dist.is_initialized() else 0
        self.rank = self.ranks.index(me) if me in self.ranks else -1
        self.world_size = len(self.ranks)
        self.comm = ncclComm_t()
        self.disabled = self.rank < 0
        self._depth = 0
        if self.disabled:
            return
        raw = self._exchange_id(control_group, store, tag)
        with torch.cuda.device(self.device):
            self.nccl.check(self.nccl.fn["ncclCommInitRank"](ctypes.byref(self.comm), self.world_size,
                                                             NcclLibrary.unique_id_from_bytes(raw), self.rank),
                            "ncclCommInitRank")

    def _exchange_id(self, control_group, store, tag: str) -> bytes:
        key = "ua_nccl_id/" + tag + "/" + ",".join(map(str, self.ranks))
        if self.world_size == 1:
            return self.nccl.unique_id()
        if store is not None:
            if self.rank == 0:
                store.set(key, self.nccl.unique_id())
            return bytes(store.get(key))
        box = [self.nccl.unique_id() if self.rank == 0 else None]
        dist.broadcast_object_list(box, src=self.ranks[0], group=control_group)
        return box[0]

    # ---- helpers -------------------------------------------------------------------------------
    def _stream(self, stream) -> cudaStream_t:
        if stream is None:
            stream = torch.cuda.current_stream(self.device)
        return cudaStream_t(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))

    def _check_tensor(self, t: torch.Tensor) -> None:
        if t.device != self.device or not t.is_contiguous() or t.dtype not in DTYPES:
            raise ValueError(f"NCCL operand must be a contiguous tensor of a supported dtype on {self.device}; "
                             f"got {t.dtype} on {t.device}, contiguous={t.is_contiguous()}")

    def _call(self, name: str, *args) -> None:
        self.nccl.check(self.nccl.fn[name](*args), name)

    @contextlib.contextmanager
    def group(self):
        """Batch the calls made inside into one NCCL group (needed for a send and a recv that wait
        for each other; also one launch instead of many)."""
        if self.disabled:
            yield self
            return
        self._call("ncclGroupStart")
        self._depth += 1
        try:
            yield self
        finally:
            self._depth -= 1
            self._call("ncclGroupEnd")

    # ---- operations ----------------------------------------------------------------------------
    def all_reduce(self, tensor: torch.Tensor, op: str = "sum", stream=None, out: Optional[torch.Tensor] = None):
        if self.disabled:
            return tensor
        out = tensor if out is None else out
        self._check_tensor(tensor), self._check_tensor(out)
        self._call("ncclAllReduce", _ptr(tensor), _ptr(out), tensor.numel(), DTYPES[tensor.dtype], RED_OPS[op],
                   self.comm, self._stream(stream))
        return out

    def all_gather(self, output: torch.Tensor, input: torch.Tensor, stream=None):
        """``output`` = every member's ``input`` concatenated along dim 0 in member order."""
        if self.disabled:
            return output
        self._check_tensor(output), self._check_tensor(input)
        assert output.numel() == input.numel() * self.world_size and output.dtype == input.dtype
        self._call("ncclAllGather", _ptr(input), _ptr(output), input.numel(), DTYPES[input.dtype], self.comm,
                   self._stream(stream))
        return output

    def reduce_scatter(self, output: torch.Tensor, input: torch.Tensor, op: str = "sum", stream=None):
        """``output`` = this member's slice (along dim 0) of the reduction of every member's ``input``."""
        if self.disabled:
            return output
        self._check_tensor(output), self._check_tensor(input)
        assert input.numel() == output.numel() * self.world_size and output.dtype == input.dtype
        self._call("ncclReduceScatter", _ptr(input), _ptr(output), output.numel(), DTYPES[input.dtype], RED_OPS[op],
                   self.comm, self._stream(stream))
        return output

    def broadcast(self, tensor: torch.Tensor, src: int, stream=None):
        """``src``: rank inside the communicator."""
        if self.disabled:
            return tensor
        self._check_tensor(tensor)
        self._call("ncclBroadcast", _ptr(tensor), _ptr(tensor), tensor.numel(), DTYPES[tensor.dtype], int(src),
                   self.comm, self._stream(stream))
        return tensor

    def send(self, tensor: torch.Tensor, dst: int, stream=None) -> None:
        """``dst``: rank inside the communicator."""
        if self.disabled:
            return
        self._check_tensor(tensor)
        self._call("ncclSend", _ptr(tensor), tensor.numel(), DTYPES[tensor.dtype], int(dst), self.comm,
                   self._stream(stream))

    def recv(self, tensor: torch.Tensor, src: int, stream=None) -> None:
        if self.disabled:
            return
        self._check_tensor(tensor)
        self._call("ncclRecv", _ptr(tensor), tensor.numel(), DTYPES[tensor.dtype], int(src), self.comm,
                   self._stream(stream))

    def exchange(self, send: torch.Tensor, recv: torch.Tensor, peer: int, stream=None) -> None:
        """Send ``send`` to and receive ``recv`` from ``peer`` as one group (the pairwise step of a
        launch plan: neither side can deadlock on the order of the two calls)."""
        with self.group():
            self.send(send, peer, stream)
            self.recv(recv, peer, stream)

    # ---- state ---------------------------------------------------------------------------------
    def async_error(self) -> Optional[str]:
        """NCCL's asynchronous error state of this communicator (``None``: healthy). A rank whose
        peer died finds the failure here without blocking in a collective."""
        if self.disabled or not self.comm:
            return None
        res = ncclResult_t(0)
        self._call("ncclCommGetAsyncError", self.comm, ctypes.byref(res))
        return None if res.value == 0 else self.nccl.error_string(res.value)

    def size_and_rank(self) -> tuple:
        n, r = ctypes.c_int(0), ctypes.c_int(0)
        self._call("ncclCommCount", self.comm, ctypes.byref(n))
        self._call("ncclCommUserRank", self.comm, ctypes.byref(r))
        return n.value, r.value

    def destroy(self, abort: bool = False) -> None:
        """Free the communicator. ``abort=True`` does not wait for outstanding operations (the way
        out after a peer failure). CUDA graphs that captured calls of this communicator must be
        destroyed first: ``ncclCommDestroy`` waits for them."""
        if self.comm:
            self._call("ncclCommAbort" if abort else "ncclCommDestroy", self.comm)
            self.comm = ncclComm_t()
        self.disabled = True
