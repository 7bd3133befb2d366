"""Communicators with explicit streams, and the registry that hands them out by rank tuple.

Reference: tests/distributed/device_communicators/pynccl.py:17-322 (``PyNcclCommunicator``: a
communicator over an arbitrary rank list whose every operation takes the stream to run on, so
sends, receives and compute can sit on three streams and be captured in CUDA graphs),
search_algo/initialize.py:108-136 and search_algo/benchmark.py:511-570 (dictionaries of
communicators keyed by ``tuple(ranks)``: world, prefix groups, one per ordered pair, row / column
groups of a Y x X grid), orchestrated_attn/utils.py:300-380 (``IntraComm`` / ``InterComm`` and
their ``_fused`` forms).

The reference binds NCCL through ctypes because ``torch.distributed`` of its day gave no control
over the stream. Here a communicator is a ``torch.distributed`` process group plus the stream
discipline (the operation is enqueued under ``torch.cuda.stream(stream)``; NCCL work of PyTorch
runs on the current stream's successor and is ordered after it), which serves the NCCL baseline
executor. The fused path does not use communicators at all. On CPU tensors the same calls run over
gloo with the stream ignored, so the host logic is testable without a GPU.
"""
from __future__ import annotations

import contextlib
from typing import Iterable, Optional, Sequence

import torch
import torch.distributed as dist


class StreamCommunicator:
    """A communicator over ``ranks`` (global ranks, any order; index in the list = rank inside the
    communicator). Construction is collective over the default group (``dist.new_group``)."""

    def __init__(self, ranks: Sequence[int], backend: Optional[str] = None, group=None):
        self.ranks = list(ranks)
        self.group = group if group is not None else dist.new_group(self.ranks, backend=backend)
        me = dist.get_rank()
        self.rank = self.ranks.index(me) if me in self.ranks else -1
        self.world_size = len(self.ranks)
        self.disabled = False
        self._batch: Optional[list] = None
        self._pending: list = []

    # ---- state ---------------------------------------------------------------------------------
    @contextlib.contextmanager
    def change_state(self, enable: bool = True):
        """Temporarily enable / disable the communicator (a disabled one ignores every call)."""
        old, self.disabled = self.disabled, not enable
        try:
            yield self
        finally:
            self.disabled = old

    @staticmethod
    def _on(stream, tensor):
        if stream is not None and tensor.is_cuda:
            return torch.cuda.stream(stream)
        return contextlib.nullcontext()

    # ---- collectives ---------------------------------------------------------------------------
    def all_reduce(self, tensor: torch.Tensor, op=dist.ReduceOp.SUM, stream=None) -> torch.Tensor:
        if self.disabled or self.world_size == 1:
            return tensor
        with self._on(stream, tensor):
            dist.all_reduce(tensor, op=op, group=self.group)
        return tensor

    def all_gather(self, output: torch.Tensor, input: torch.Tensor, stream=None) -> torch.Tensor:
        """``output`` = the ``input`` of every member, concatenated along dim 0 in member order."""
        if self.disabled:
            return output
        with self._on(stream, input):
            if input.is_cuda:
                dist.all_gather_into_tensor(output, input, group=self.group)
            else:
                parts = [torch.empty_like(input) for _ in range(self.world_size)]
                dist.all_gather(parts, input.contiguous(), group=self.group)
                output.copy_(torch.cat(parts, dim=0).view_as(output))
        return output

    def reduce_scatter(self, output: torch.Tensor, input: torch.Tensor, op=dist.ReduceOp.SUM,
                       stream=None) -> torch.Tensor:
        """``output`` = this member's slice (along dim 0) of the element-wise reduction of all
        members' ``input``."""
        if self.disabled:
            return output
        with self._on(stream, input):
            if input.is_cuda:
                dist.reduce_scatter_tensor(output, input, op=op, group=self.group)
            else:                                   # gloo has no reduce-scatter
                full = input.clone()
                dist.all_reduce(full, op=op, group=self.group)
                output.copy_(full.chunk(self.world_size, dim=0)[self.rank].view_as(output))
        return output

    # ---- point to point ------------------------------------------------------------------------
    def _p2p(self, fn, tensor, peer: int, stream):
        if self.disabled:
            return
        op = dist.P2POp(fn, tensor, self.ranks[peer], group=self.group)
        if self._batch is not None:
            self._batch.append((op, stream))
            return
        with self._on(stream, tensor):
            self._pending.extend(dist.batch_isend_irecv([op]))

    def send(self, tensor: torch.Tensor, dst: int, stream=None) -> None:
        """Send to member index ``dst``. Asynchronous with respect to the host: :meth:`wait` (or a
        stream / event dependency on CUDA) completes it."""
        self._p2p(dist.isend, tensor, dst, stream)

    def recv(self, tensor: torch.Tensor, src: int, stream=None) -> None:
        self._p2p(dist.irecv, tensor, src, stream)

    def group_start(self) -> None:
        """Begin a batch: the sends and receives up to :meth:`group_end` are issued together, so
        neither side can block the other."""
        assert self._batch is None, "group_start called twice"
        self._batch = []

    def group_end(self) -> None:
        batch, self._batch = self._batch, None
        if not batch:
            return
        stream, first = batch[0][1], batch[0][0].tensor
        with self._on(stream, first):
            self._pending.extend(dist.batch_isend_irecv([op for op, _ in batch]))

    def wait(self) -> None:
        """Host-side completion of every outstanding send / receive."""
        pending, self._pending = self._pending, []
        for w in pending:
            w.wait()

    def barrier(self) -> None:
        if not self.disabled and self.world_size > 1:
            dist.barrier(group=self.group)


PyNcclCommunicator = StreamCommunicator     # the reference's class name


class CommRegistry(dict):
    """Communicators keyed by ``tuple(ranks)``. ``create`` is collective: every rank of the job
    must call it with the same list of rank lists, in the same order."""

    def create(self, rank_lists: Iterable[Sequence[int]], backend: Optional[str] = None) -> "CommRegistry":
        for ranks in rank_lists:
            key = tuple(ranks)
            if key not in self:
                self[key] = StreamCommunicator(key, backend=backend)
        return self

    def for_pairs(self, ranks: Sequence[int], backend: Optional[str] = None) -> "CommRegistry":
        """One communicator per unordered pair (the reference creates one per ordered pair)."""
        ranks = list(ranks)
        return self.create([(a, b) for i, a in enumerate(ranks) for b in ranks[i + 1:]], backend)

    def for_grid(self, ranks: Sequence[int], X: int, backend: Optional[str] = None) -> "CommRegistry":
        """Row groups (ranks sharing ``g // X``) and column groups (ranks sharing ``g % X``) of a
        Y x X grid over ``ranks``."""
        ranks = list(ranks)
        rows = [tuple(ranks[r * X:(r + 1) * X]) for r in range(len(ranks) // X)]
        cols = [tuple(ranks[c::X]) for c in range(X)]
        return self.create([g for g in rows + cols if len(g) > 1], backend)

    def pair(self, a: int, b: int) -> StreamCommunicator:
        return self[(min(a, b), max(a, b))]


class IntraComm:
    """Point-to-point transfer of a whole data carrier (one flat buffer = one message) between two
    ranks, through the pair's communicator (reference: orchestrated_attn/utils.py:300-334)."""

    def __init__(self, registry: CommRegistry, rank: Optional[int] = None):
        self.registry = registry
        self.rank = dist.get_rank() if rank is None else rank

    def _comm(self, peer: int, ncclcomm):
        return ncclcomm if ncclcomm is not None else self.registry.pair(self.rank, peer)

    def send(self, dst: int, idata, stream=None, ncclcomm=None) -> None:
        c = self._comm(dst, ncclcomm)
        c.send(getattr(idata, "data", idata), c.ranks.index(dst), stream)

    def recv(self, src: int, idata, stream=None, ncclcomm=None) -> None:
        c = self._comm(src, ncclcomm)
        c.recv(getattr(idata, "data", idata), c.ranks.index(src), stream)


InterComm = IntraComm       # one NVSwitch domain: both levels use the same transport


class IntraComm_fused:
    """Row / column collectives of the kernel-tile path (reference: orchestrated_attn/utils.py:
    336-380): ``rc`` 'r' selects this rank's row group, 'c' its column group."""

    def __init__(self, registry: CommRegistry, ranks: Sequence[int], X: int, rank: Optional[int] = None):
        ranks = list(ranks)
        me = dist.get_rank() if rank is None else rank
        g = ranks.index(me)
        self.groups = {"r": tuple(ranks[g // X * X:(g // X + 1) * X]), "c": tuple(ranks[g % X::X])}
        self.registry = registry

    def _comm(self, rc: str) -> Optional[StreamCommunicator]:
        key = self.groups[rc]
        return self.registry[key] if len(key) > 1 else None

    def all_gather(self, rc: str, output, input, stream=None):
        c = self._comm(rc)
        return output.copy_(input.view_as(output)) if c is None else c.all_gather(output, input, stream)

    def reduce_scatter(self, rc: str, output, input, stream=None):
        c = self._comm(rc)
        return output.copy_(input.view_as(output)) if c is None else c.reduce_scatter(output, input, stream=stream)


InterComm_fused = IntraComm_fused
