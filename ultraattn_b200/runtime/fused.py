"""Context-parallel attention with the collectives fused into the attention kernels.

Every rank keeps its shard of Q, K, V (and, for the backward, dO, lse, D) in *symmetric memory*:
buffers allocated identically on all ranks and mapped into every peer's address space over
NVLink. One forward call is then, per rank:

    copy inputs into the symmetric buffers  ->  device barrier
    ONE attention kernel: its first CTAs pull the remote K/V (and Q) blocks this rank's tiles
        need from the peers' memory into local staging mirrors with plain peer loads (each
        block crosses NVLink once) while the other CTAs already compute tiles whose inputs are
        local; a tile that needs a staged block waits (bounded) on that block's flag; partial
        (O, lse) of rows owned by a peer are stored by the epilogue straight into the owner's
        mailbox through its peer mapping
    device barrier  ->  owner merges its own partial with the mailbox slots (log-sum-exp merge)

and one backward call is the mirror image: staging of Q / dO / lse / D and K / V blocks inside
the backward kernel, dQ of foreign rows added into the owner's fp32 accumulator by TMA
reduce-add through a tensor map over the peer mapping, dK / dV of foreign columns added with
``red.global.add.v4.f32`` on peer pointers, barrier, cast of the own accumulators to bf16.

Which rank computes which tile comes from the planner's tile-allocation program; the message
kernels of the plan (reference: one NCCL send/recv per (row-or-column, peer),
orchestrated_attn/utils.py:300-380, search_algo/dependent_graph.py:268-305) have no separate
existence here — they are the staging prologue and the epilogues of the two kernels.

``PeerSpace`` abstracts the symmetric memory so that the whole host-side logic (tables, slots,
staging lists, merge lists) also runs on CPU with all ranks simulated in one process
(:class:`FakeSpace`), which is how it is tested without GPUs.
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from .. import _lib
from ..ops import attention as A
from ..ops import elementwise as E
from ..patterns.blocks import BSA_Repr, CAUSAL

CHUNK_BYTES = 1 << 20       # staging granularity: one copy task moves at most this much
# Every CTA that waits for a staged block first helps to empty the launch's queue of copy tasks;
# in addition the first UA_COPY_CTAS CTAs of the grid help whether they wait or not (all SMs by
# default; fewer leave SMs free to start on tiles whose inputs are local while the copies run)
MAX_COPY_CTAS = int(os.environ.get("UA_COPY_CTAS", "148"))


# =================================================================================================
# peer spaces
# =================================================================================================
class PeerSpace:
    rank: int
    world: int

    def alloc(self, name: str, shape, dtype) -> torch.Tensor: raise NotImplementedError
    def finalize(self) -> None: raise NotImplementedError
    def local(self, name: str) -> torch.Tensor: raise NotImplementedError
    def peer(self, name: str, r: int) -> torch.Tensor: raise NotImplementedError
    def barrier(self, channel: int) -> None: raise NotImplementedError

    def has_multicast(self) -> bool:
        """True when one store can reach every rank's replica of a buffer (NVSwitch multicast)."""
        return False

    def multicast_store(self, name: str, index, src: torch.Tensor) -> None:
        """replica[index] = src in every rank's buffer ``name`` (``index``: leading-dimension
        indices / slices selecting a contiguous piece)."""
        raise NotImplementedError

    def multicast_reduce(self, name: str, index, dst: torch.Tensor) -> None:
        """dst = sum over all ranks of replica[index] of buffer ``name`` (fp32), computed inside
        the switch (``multimem.ld_reduce``): the owner receives one block however many ranks
        contributed."""
        raise NotImplementedError


class FakeSpace(PeerSpace):
    """All ranks in one process on CPU; ``peer`` hands out the other rank's tensor itself."""

    def __init__(self, rank: int, world: int, registry: dict, device="cpu", multicast: bool = False):
        self.rank, self.world, self.registry, self.device = rank, world, registry, torch.device(device)
        self.multicast = multicast

    def has_multicast(self): return self.multicast

    def multicast_store(self, name, index, src):
        for r in range(self.world):
            self.registry[(r, name)][index].copy_(src)

    def multicast_reduce(self, name, index, dst):
        dst.copy_(sum(self.registry[(r, name)][index].to(torch.float32) for r in range(self.world)))

    def alloc(self, name, shape, dtype):
        t = torch.zeros(*shape, dtype=dtype, device=self.device)
        self.registry[(self.rank, name)] = t
        return t

    def finalize(self): pass
    def local(self, name): return self.registry[(self.rank, name)]
    def peer(self, name, r): return self.registry[(r, name)]
    def barrier(self, channel): pass


class SymmMemSpace(PeerSpace):
    """Symmetric memory of a process group (``torch.distributed._symmetric_memory`` as the
    allocator front-end: CUDA VMM allocations exchanged between the ranks of one node). All
    named buffers are carved out of one allocation, so one rendezvous maps everything."""

    def __init__(self, group, device: torch.device, timeout_s: float = 20.0):
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.specs: list = []
        self.offsets: dict = {}
        self.total = 0
        self.hdl = None
        self.timeout_s = timeout_s
        self.epochs: dict = {}
        self._views: dict = {}

    def alloc(self, name, shape, dtype):
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        self.offsets[name] = (self.total, tuple(shape), dtype)
        self.total += (n + 255) // 256 * 256
        return None

    def finalize(self):
        import torch.distributed._symmetric_memory as symm
        self.heap = symm.empty(self.total, dtype=torch.uint8, device=self.device)
        self.heap.zero_()
        self.hdl = symm.rendezvous(self.heap, self.group)
        torch.cuda.synchronize(self.device)
        import ctypes
        self._pads = (ctypes.c_void_p * self.world)(*[int(p) for p in self.hdl.signal_pad_ptrs])
        dist.barrier(self.group)

    def _view(self, r: int, name: str) -> torch.Tensor:
        key = (r, name)
        if key not in self._views:
            off, shape, dtype = self.offsets[name]
            es = torch.empty((), dtype=dtype).element_size()
            self._views[key] = self.hdl.get_buffer(r, shape, dtype, off // es)
        return self._views[key]

    def local(self, name): return self._view(self.rank, name)
    def peer(self, name, r): return self._view(r, name)

    def multicast_ptr(self, name: str) -> int:
        """NVSwitch multicast address of a named buffer (0 when the allocation has none: no NVLS
        on this machine, or ``UA_NVLS=0``)."""
        if os.environ.get("UA_NVLS", "1") == "0":
            return 0
        base = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        return base + self.offsets[name][0] if base else 0

    def has_multicast(self) -> bool:
        return self.hdl is not None and self.multicast_ptr(next(iter(self.offsets))) != 0

    def multicast_store(self, name, index, src):
        dst = self.local(name)[index]
        assert dst.is_contiguous() and dst.numel() == src.numel() and dst.dtype == src.dtype
        off = dst.data_ptr() - self.local(name).data_ptr()
        E.multimem_bcast_(self.multicast_ptr(name) + off, src.contiguous())

    def multicast_reduce(self, name, index, dst):
        src = self.local(name)[index]
        assert src.is_contiguous() and dst.is_contiguous() and src.dtype == dst.dtype == torch.float32
        off = src.data_ptr() - self.local(name).data_ptr()
        E.multimem_reduce(self.multicast_ptr(name) + off, dst, src.numel() * 4, torch.float32, self.device)

    def barrier(self, channel: int) -> None:
        """Device barrier on the current stream (bounded wait; errors land in the status word)."""
        ep = self.epochs.get(channel, 0) + 1
        self.epochs[channel] = ep
        st = A.status_buffer(self.device)
        rc = _lib.load().ua_barrier(self._pads, self.rank, self.world, channel, ep, self.timeout_s,
                                    st.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(rc, "ua_barrier")


# =================================================================================================
# the runtime
# =================================================================================================
class FusedContextParallel:
    """Host-side state of the fused path for one (pattern, shape, group)."""

    def __init__(self, table: np.ndarray, cmap: np.ndarray, pattern: BSA_Repr, seq_len: int,
                 n_heads: int, head_dim: int, space: PeerSpace, n_kv_heads: Optional[int] = None,
                 batch: int = 1, dtype=torch.bfloat16, device=None, defer_build: bool = False,
                 nvls_min_consumers: int = 2, nvls_reduce: Optional[bool] = None):
        """``nvls_reduce``: deliver dK/dV of the broadcast (one-to-many) key/value blocks by an
        in-switch sum instead of one peer reduction per consumer: every rank adds its share into
        its own replica of a symmetric buffer and the block's owner reads the sum of all replicas
        with ``multimem.ld_reduce``. Default: the ``UA_NVLS_REDUCE=1`` environment switch (off)."""
        self.space = space
        self.nvls_min_consumers = nvls_min_consumers
        self.nvls_reduce = (os.environ.get("UA_NVLS_REDUCE") == "1") if nvls_reduce is None else bool(nvls_reduce)
        self.rank, self.world = space.rank, space.world
        self.table = np.asarray(table)
        self.cmap = np.asarray(cmap)
        self.par_d = self.table.shape[0]
        self.S, self.H, self.D = seq_len, n_heads, head_dim
        self.Hk = n_kv_heads or n_heads
        self.B = batch
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.cuda = self.device.type == "cuda"
        self.blk = seq_len // self.par_d
        self.types = pattern.refined(self.par_d)
        self.owned = {r: [i for i in range(self.par_d) if self.cmap[i] == r] for r in range(self.world)}
        self.S_loc = len(self.owned[self.rank]) * self.blk
        assert all(len(v) * self.blk == self.S_loc for v in self.owned.values()), "uneven shards"
        self.lidx = {b: self.owned[int(self.cmap[b])].index(b) for b in range(self.par_d)}
        g = self.rank
        self.my_tiles = [(r, c) for r in range(self.par_d) for c in range(self.par_d) if self.table[r, c] == g]
        self.my_rows = sorted({r for r, _ in self.my_tiles})
        self.my_cols = sorted({c for _, c in self.my_tiles})
        self.remote_rows = [r for r in self.my_rows if self.cmap[r] != g]
        self.remote_cols = [c for c in self.my_cols if self.cmap[c] != g]
        # mailbox slots of every owner: (row, contributor) pairs, contributor != owner
        self.slots = {p: [] for p in range(self.world)}
        for r in range(self.par_d):
            p = int(self.cmap[r])
            for contrib in sorted({int(x) for x in self.table[r] if x >= 0 and x != p}):
                self.slots[p].append((r, contrib))
        self.max_slots = max(1, max(len(v) for v in self.slots.values()))
        # key/value blocks that several other ranks need: their owner broadcasts them through the
        # switch (one multicast store) instead of every consumer pulling its own copy. Same list
        # on every rank; dropped again in _alloc when the memory has no multicast address.
        self.bc_cols = []
        for c in range(self.par_d):
            p = int(self.cmap[c])
            consumers = {int(x) for x in self.table[:, c] if x >= 0 and x != p}
            if len(consumers) >= max(1, nvls_min_consumers) and self.world > 1:
                self.bc_cols.append(c)
        self.bc_slot = {c: i for i, c in enumerate(self.bc_cols)}
        self.fwd_calls = 0
        self.bwd_calls = 0
        # UA_DEBUG_POISON=1: the staging mirrors are filled with NaN before every call, so a tile
        # that reads a block the staging plan did not deliver (or a stale copy from an earlier
        # call) shows up as NaN in the result instead of going unnoticed
        self.debug_poison = os.environ.get("UA_DEBUG_POISON") == "1"
        self._alloc()
        if not defer_build:
            self.build()

    def build(self) -> None:
        """Build the launch tables (needs every rank's buffers to exist)."""
        self._build_fwd()
        self._build_bwd()
        self._account_traffic()

    # ------------------------------- observability ----------------------------------------------
    def _account_traffic(self) -> None:
        """Bytes this rank moves over NVLink per call, by direction and purpose (what the fused
        kernels do no longer shows up as separate communication kernels, so it is accounted for
        here from the same tables the kernels execute)."""
        es = torch.empty((), dtype=self.dtype).element_size()
        nbytes = lambda pieces: sum(src.numel() * src.element_size() for _, src, _ in pieces)
        row_o = self.B * self.blk * self.H * self.D * es + self.B * self.H * self.blk * 4
        kv_blk = self.B * self.blk * self.Hk * self.D
        bc_in = sum(1 for c in self.remote_cols if c in self.bc_slot) * 2 * kv_blk * es
        bc_out = sum(1 for c in self.bc_cols if int(self.cmap[c]) == self.rank) * 2 * kv_blk * es
        self.traffic = {
            "fwd_pull_bytes": nbytes(self.f_pieces),                    # staged Q / K / V blocks (peer loads)
            "fwd_multicast_in_bytes": bc_in,                            # blocks received by multicast
            "fwd_multicast_out_bytes": bc_out,                          # blocks this rank broadcasts (leave once)
            "fwd_push_bytes": len(self.remote_rows) * row_o,            # partial (O, lse) into mailboxes
            "bwd_pull_bytes": nbytes(self.b_pieces),                    # dO / lse / D of foreign rows
            "bwd_pull_bytes_no_reuse": nbytes(self.b_pieces_full),
            "bwd_push_bytes": (len(self.remote_rows) * self.B * self.blk * self.H * self.D * 4      # dQ
                               + sum(1 for c in self.remote_cols
                                     if not (self.nvls_reduce and c in self.bc_slot)) * 2 * kv_blk * 4),  # dK, dV
            # dK / dV of broadcast blocks that this rank owns, summed in the switch: one block in
            "bwd_reduce_in_bytes": (sum(1 for c in self.bc_cols if int(self.cmap[c]) == self.rank)
                                    * 2 * kv_blk * 4 if self.nvls_reduce else 0),
        }

    def enable_trace(self, on: bool = True, kernels: bool = False) -> None:
        """Record CUDA events around every phase of the following calls (see :meth:`metrics`).
        ``kernels``: also let the two attention kernels record per-CTA time stamps (start, end of
        staging, end, SM): :meth:`metrics` then reports, for the last forward and backward launch,
        how long SMs copied before computing, how busy they were and how long the tail ran."""
        self._trace = [] if on else None
        self._ktrace = bool(on and kernels and self.cuda)
        if self.cuda:
            if self._ktrace:
                A.enable_kernel_trace(self.device)
            else:
                A.disable_kernel_trace(self.device)

    def _mark(self, name: str) -> None:
        tr = getattr(self, "_trace", None)
        if tr is not None and self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.device))
            tr.append((name, ev))

    def metrics(self) -> dict:
        """Phase durations (ms, this rank) of the calls since :meth:`enable_trace`, plus the
        per-call NVLink byte counts; synchronises the device."""
        out = {"traffic": dict(self.traffic), "phases_ms": {}}
        tr = getattr(self, "_trace", None)
        if tr and self.cuda:
            torch.cuda.synchronize(self.device)
            for (n0, e0), (n1, e1) in zip(tr[:-1], tr[1:]):
                if n1.endswith(":begin"):
                    continue
                out["phases_ms"][n1] = out["phases_ms"].get(n1, 0.0) + e0.elapsed_time(e1)
            self._trace = []
        if getattr(self, "_ktrace", False):
            from ..utils.kernel_trace import summarize
            out["kernels"] = {k: summarize(A.read_kernel_trace(self.device, k)) for k in ("fwd", "bwd")}
        return out

    # ------------------------------- buffers ----------------------------------------------------
    def _alloc(self) -> None:
        sp, B, S, H, Hk, D, dt = self.space, self.B, self.S_loc, self.H, self.Hk, self.D, self.dtype
        for name, shape, dtype in [
            ("q", (B, S, H, D), dt), ("k", (B, S, Hk, D), dt), ("v", (B, S, Hk, D), dt),
            ("do", (B, S, H, D), dt), ("lse", (B, H, S), torch.float32), ("dvec", (B, H, S), torch.float32),
            ("mail_o", (B, self.max_slots * self.blk, H, D), dt),
            ("mail_lse", (B, H, self.max_slots * self.blk), torch.float32),
            ("dq_acc", (B, S, H, D), torch.float32), ("dk_acc", (B, S, Hk, D), torch.float32),
            ("dv_acc", (B, S, Hk, D), torch.float32),
        ] + ([("bc_k", (B, len(self.bc_cols) * self.blk, Hk, D), dt),
              ("bc_v", (B, len(self.bc_cols) * self.blk, Hk, D), dt)] if self.bc_cols else []) \
          + ([("bc_dk", (B, len(self.bc_cols) * self.blk, Hk, D), torch.float32),
              ("bc_dv", (B, len(self.bc_cols) * self.blk, Hk, D), torch.float32)]
             if self.bc_cols and self.nvls_reduce else []):
            sp.alloc(name, shape, dtype)
        sp.finalize()
        if self.bc_cols and not sp.has_multicast():
            self.bc_cols, self.bc_slot = [], {}
        self.nvls_reduce = self.nvls_reduce and bool(self.bc_cols)
        dev = self.device
        peers_rows = sorted({int(self.cmap[r]) for r in self.remote_rows})
        peers_cols = sorted({int(self.cmap[c]) for c in self.remote_cols})
        # Mirrors hold only the blocks this rank's tiles need from a peer (not the peer's whole
        # shard): mir_rows[p] / mir_cols[p] list those blocks in mirror order. Key/value blocks
        # that arrive through the broadcast buffer need no mirror.
        self.mir_rows = {p: [r for r in self.remote_rows if int(self.cmap[r]) == p] for p in peers_rows}
        self.mir_cols = {p: [c for c in self.remote_cols if int(self.cmap[c]) == p and c not in self.bc_slot]
                         for p in peers_cols}
        self.mslot = {}                  # ("r" | "c", block) -> index of the block inside its mirror
        for p, blocks in self.mir_rows.items():
            self.mslot.update({("r", r): i for i, r in enumerate(blocks)})
        for p, blocks in self.mir_cols.items():
            self.mslot.update({("c", c): i for i, c in enumerate(blocks)})
        self.mir = {}
        blk = self.blk
        for p in peers_rows:
            n = len(self.mir_rows[p]) * blk
            self.mir[("q", p)] = torch.zeros(B, n, H, D, dtype=dt, device=dev)
            self.mir[("do", p)] = torch.zeros(B, n, H, D, dtype=dt, device=dev)
            self.mir[("lse", p)] = torch.zeros(B, H, n, dtype=torch.float32, device=dev)
            self.mir[("dvec", p)] = torch.zeros(B, H, n, dtype=torch.float32, device=dev)
            # dQ of foreign rows is accumulated here (every key tile adds into it) and pushed to
            # the owner once per step; adding straight into the owner's memory would send every
            # partial sum over NVLink
            self.mir[("dq", p)] = torch.zeros(B, n, H, D, dtype=torch.float32, device=dev)
        for p in peers_cols:
            n = max(1, len(self.mir_cols[p])) * blk      # (a peer whose blocks all come by broadcast keeps a stub)
            self.mir[("k", p)] = torch.zeros(B, n, Hk, D, dtype=dt, device=dev)
            self.mir[("v", p)] = torch.zeros(B, n, Hk, D, dtype=dt, device=dev)
        self.peers_rows, self.peers_cols = peers_rows, peers_cols
        self.mirror_bytes = sum(t.numel() * t.element_size() for t in self.mir.values())

    def _tok(self, blk_id: int) -> slice:
        """Tokens of a block inside its owner's shard."""
        i = self.lidx[blk_id]
        return slice(i * self.blk, (i + 1) * self.blk)

    def _mtok(self, side: str, blk_id: int) -> slice:
        """Tokens of a foreign block inside this rank's mirror of its owner (side "r" or "c")."""
        i = self.mslot[(side, blk_id)]
        return slice(i * self.blk, (i + 1) * self.blk)

    # ------------------------------- staging lists ----------------------------------------------
    def _stage_list(self, kinds_rows: Sequence[str], kinds_cols: Sequence[str]):
        """[(flag id, src view, dst view)] of contiguous pieces, and pieces-per-flag counts."""
        pieces = []
        for r in self.remote_rows:
            p = int(self.cmap[r])
            for kind in kinds_rows:
                src, dst = self.space.peer(kind, p), self.mir[(kind, p)]
                if kind in ("lse", "dvec"):
                    for b in range(self.B):
                        for h in range(self.H):
                            pieces.append((r, src[b, h, self._tok(r)], dst[b, h, self._mtok("r", r)]))
                else:
                    for b in range(self.B):
                        pieces.append((r, src[b, self._tok(r)], dst[b, self._mtok("r", r)]))
        for c in self.remote_cols:
            if c in self.bc_slot:
                continue                  # arrives by multicast before the barrier
            p = int(self.cmap[c])
            for kind in kinds_cols:
                src, dst = self.space.peer(kind, p), self.mir[(kind, p)]
                for b in range(self.B):
                    pieces.append((self.par_d + c, src[b, self._tok(c)], dst[b, self._mtok("c", c)]))
        return pieces

    def _device_tasks(self, pieces):
        """Chunk the pieces into copy tasks; returns (StagePlan or None, chunks per flag)."""
        counts = {}
        rows = []
        for flag, src, dst in pieces:
            assert src.is_contiguous() and dst.is_contiguous()
            nbytes = src.numel() * src.element_size()
            assert nbytes % 16 == 0 and src.data_ptr() % 16 == 0 and dst.data_ptr() % 16 == 0
            off = 0
            while off < nbytes:
                n = min(CHUNK_BYTES, nbytes - off)
                rows.append((src.data_ptr() + off, dst.data_ptr() + off, n // 16, flag))
                counts[flag] = counts.get(flag, 0) + 1
                off += n
        return rows, counts

    def _make_stage(self, pieces):
        if not self.cuda:
            counts = {}
            for flag, _, _ in pieces:
                counts[flag] = counts.get(flag, 0) + 1
            return None, counts
        rows, counts = self._device_tasks(pieces)
        flags = torch.zeros(2 * self.par_d + 1, dtype=torch.int32, device=self.device)
        if rows:
            # interleave tasks of different blocks so that blocks complete in parallel
            tasks = torch.tensor(rows, dtype=torch.int64).to(self.device)
        else:
            tasks = torch.zeros(1, 4, dtype=torch.int64, device=self.device)
        stage = A.StagePlan(tasks, len(rows), min(MAX_COPY_CTAS, max(1, len(rows))), flags, 0)
        return stage, counts

    # ------------------------------- forward tables ---------------------------------------------
    def _build_fwd(self) -> None:
        g = self.rank
        self.f_pieces = self._stage_list(["q"], ["k", "v"])
        self.f_stage, counts = self._make_stage(self.f_pieces)
        q_src = {g: 0}
        for p in self.peers_rows:
            q_src[p] = len(q_src)
        kv_src = {g: 0}
        for p in self.peers_cols:
            kv_src[p] = len(kv_src)
        if self.bc_cols:
            kv_src["bc"] = len(kv_src)          # the broadcast buffer (this rank's replica)
        out_slot = {g: 0}
        for p in self.peers_rows:
            out_slot[p] = len(out_slot)
        self.f_q_src, self.f_kv_src, self.f_out_slot = q_src, kv_src, out_slot
        assert max(len(q_src), len(kv_src), len(out_slot)) <= 10, "too many source tensors for one launch"
        rows = []
        for r in self.my_rows:
            p = int(self.cmap[r])
            segs = []
            cols = [c for (rr, c) in self.my_tiles if rr == r]
            cols.sort(key=lambda c: (self.cmap[c] != g, c))        # local key blocks first
            for c in cols:
                pc = int(self.cmap[c])
                remote = pc != g
                if remote and c in self.bc_slot:
                    segs.append(A.Seg(kv_src["bc"], self.bc_slot[c] * self.blk, self.blk,
                                      self.types[r, c] == CAUSAL, 0, 0, 0))
                    continue
                segs.append(A.Seg(kv_src[pc], (self.mslot[("c", c)] if remote else self.lidx[c]) * self.blk, self.blk,
                                  self.types[r, c] == CAUSAL, 0,
                                  (self.par_d + c + 1) if remote else 0,
                                  counts.get(self.par_d + c, 0) if remote else 0))
            if p == g:
                o_start = self.lidx[r] * self.blk
            else:
                o_start = self.slots[p].index((r, g)) * self.blk
            rows.append(A.Row(q_src[p], (self.lidx[r] if p == g else self.mslot[("r", r)]) * self.blk, self.blk,
                              tuple(segs), out_slot[p],
                              o_start, False, (r + 1) if p != g else 0, counts.get(r, 0) if p != g else 0))
        # rows whose inputs are all local first: they can start while the staging runs
        rows.sort(key=lambda row: (row.q_wait_flag != 0) + sum(s.wait_flag != 0 for s in row.segs))
        self.f_rows = rows
        self.f_plan = A.FwdPlan(rows, self.device)
        # merge lists for own rows
        self.f_merge = []
        for r in self.owned[g]:
            own = any(rr == r for rr, _ in self.my_tiles)
            slots = [i for i, (row, _) in enumerate(self.slots[g]) if row == r]
            if slots or not own:
                self.f_merge.append((r, own, slots))

    # ------------------------------- backward tables --------------------------------------------
    def _build_bwd(self) -> None:
        g = self.rank
        self.b_pieces = self._stage_list(["do", "lse", "dvec"], [])     # q / k / v mirrors come from the forward
        self.b_pieces_full = self._stage_list(["q", "do", "lse", "dvec"], ["k", "v"])
        self.b_stage, counts = self._make_stage(self.b_pieces)
        self.b_stage_full, counts_full = self._make_stage(self.b_pieces_full)
        self.b_counts = (counts, counts_full)
        q_src = {g: 0}
        for p in self.peers_rows:
            q_src[p] = len(q_src)
        kv_src = {g: 0}
        for p in self.peers_cols:
            kv_src[p] = len(kv_src)
        if self.bc_cols:
            kv_src["bc"] = len(kv_src)
        if self.nvls_reduce:
            kv_src["bcg"] = len(kv_src)         # gradient slot only: this rank's replica of bc_dk / bc_dv
        self.b_q_src, self.b_kv_src = q_src, kv_src
        assert len(kv_src) <= 10 and len(q_src) <= 10, "too many source tensors for one launch"
        self.b_plans = []
        for cnt in (counts, counts_full):
            cols = []
            for c in self.my_cols:
                pc = int(self.cmap[c])
                rows = [r for (r, cc) in self.my_tiles if cc == c]
                rows.sort(key=lambda r: (self.cmap[r] != g, r))
                segs = []
                for r in rows:
                    pr = int(self.cmap[r])
                    remote = pr != g
                    segs.append(A.Seg(q_src[pr], (self.mslot[("r", r)] if remote else self.lidx[r]) * self.blk, self.blk,
                                      self.types[r, c] == CAUSAL, 0,
                                      (r + 1) if remote else 0, cnt.get(r, 0) if remote else 0))
                kv_remote = pc != g
                kv_cnt = cnt.get(self.par_d + c, 0)
                if self.nvls_reduce and c in self.bc_slot:
                    # gradients of a broadcast block go into this rank's own replica of the
                    # reduction buffer (the owner's share too); the owner sums the replicas
                    src = kv_src["bc"] if kv_remote else kv_src[pc]
                    start = self.bc_slot[c] * self.blk if kv_remote else self.lidx[c] * self.blk
                    cols.append(A.Col(src, start, self.blk, tuple(segs), kv_src["bcg"],
                                      self.bc_slot[c] * self.blk, 0, 0))
                    continue
                if kv_remote and c in self.bc_slot:
                    # keys / values from the broadcast buffer, gradients into the owner's accumulators
                    cols.append(A.Col(kv_src["bc"], self.bc_slot[c] * self.blk, self.blk, tuple(segs),
                                      kv_src[pc], self.lidx[c] * self.blk, 0, 0))
                    continue
                # keys / values: own shard or the compact mirror; gradients: the owner's accumulator
                cols.append(A.Col(kv_src[pc], (self.mslot[("c", c)] if kv_remote else self.lidx[c]) * self.blk,
                                  self.blk, tuple(segs), kv_src[pc], self.lidx[c] * self.blk,
                                  (self.par_d + c + 1) if (kv_remote and kv_cnt) else 0, kv_cnt if kv_remote else 0))
            self.b_plans.append(A.BwdPlan(cols, self.device))
            self.b_cols = cols

    # =============================== forward ====================================================
    def _broadcast_kv(self, k, v) -> None:
        """Owner side of the one-to-many blocks: one multicast store per block and tensor."""
        for c in self.bc_cols:
            if int(self.cmap[c]) != self.rank:
                continue
            i = self.bc_slot[c]
            dst = slice(i * self.blk, (i + 1) * self.blk)
            for b in range(self.B):
                self.space.multicast_store("bc_k", (b, dst), k[b, self._tok(c)])
                self.space.multicast_store("bc_v", (b, dst), v[b, self._tok(c)])

    def fwd_prepare(self, q, k, v) -> None:
        sp = self.space
        sp.local("q").copy_(q)
        sp.local("k").copy_(k)
        sp.local("v").copy_(v)
        self._broadcast_kv(k, v)

    def stage_on_host(self, pieces) -> None:
        """CPU stand-in of the in-kernel staging prologue."""
        for _, src, dst in pieces:
            dst.copy_(src)

    def fwd_compute(self, softmax_scale=None):
        sp, g = self.space, self.rank
        B, S, H, D = self.B, self.S_loc, self.H, self.D
        o = torch.zeros(B, S, H, D, dtype=self.dtype, device=self.device)
        lse = torch.full((B, H, S), float("-inf"), dtype=torch.float32, device=self.device)
        q_srcs = [None] * len(self.f_q_src)
        k_srcs = [None] * len(self.f_kv_src)
        v_srcs = [None] * len(self.f_kv_src)
        outs = [None] * len(self.f_out_slot)
        for p, i in self.f_q_src.items():
            q_srcs[i] = sp.local("q") if p == g else self.mir[("q", p)]
        for p, i in self.f_kv_src.items():
            if p == "bc":
                k_srcs[i], v_srcs[i] = sp.local("bc_k"), sp.local("bc_v")
                continue
            k_srcs[i] = sp.local("k") if p == g else self.mir[("k", p)]
            v_srcs[i] = sp.local("v") if p == g else self.mir[("v", p)]
        for p, i in self.f_out_slot.items():
            outs[i] = (o, lse) if p == g else (sp.peer("mail_o", p), sp.peer("mail_lse", p))
        self.fwd_calls += 1
        if self.f_stage is not None:
            self.f_stage.epoch = self.fwd_calls
        A.attn_fwd(q_srcs, k_srcs, v_srcs, outs, self.f_plan, softmax_scale, self.f_stage)
        return o, lse

    def fwd_finish(self, o, lse) -> None:
        sp = self.space
        mo, ml = sp.local("mail_o"), sp.local("mail_lse")
        for r, own, slots in self.f_merge:
            tok = self._tok(r)
            for b in range(self.B):
                parts = [(o[b, tok], lse[b, :, tok])] if own else []
                for s in slots:
                    ms = slice(s * self.blk, (s + 1) * self.blk)
                    parts.append((mo[b, ms], ml[b, :, ms]))
                if parts:
                    E.lse_merge(parts, (o[b, tok], lse[b, :, tok]))

    def _poison(self, kinds) -> None:
        for (kind, _), t in self.mir.items():
            if kind in kinds and t.is_floating_point():
                t.fill_(float("nan"))

    def forward_steps(self, q, k, v, softmax_scale=None):
        """The forward call as a generator that yields the barrier channel wherever all ranks have
        to meet; :meth:`forward` drives it with the device barrier, the single-process tests drive
        all simulated ranks in lock step."""
        self._mark("fwd:begin")
        if self.debug_poison:
            self._poison(("q", "k", "v"))
        self.fwd_prepare(q, k, v)
        self._mark("fwd_prepare")
        yield 0
        self._mark("fwd_barrier_in")
        if not self.cuda:
            self.stage_on_host(self.f_pieces)
        o, lse = self.fwd_compute(softmax_scale)
        self._mark("fwd_compute")
        yield 1
        self._mark("fwd_barrier_out")
        self.fwd_finish(o, lse)
        self._mark("fwd_finish")
        # the peers' Q / K / V now sit in the mirrors: remember WHICH forward put them there (the
        # output tensor it returned), so that only the backward of that very call skips restaging
        self._staged_for = (o.data_ptr(), tuple(o.shape), self.fwd_calls)
        return o, lse

    def _drive(self, steps):
        try:
            while True:
                self.space.barrier(next(steps))
        except StopIteration as done:
            return done.value

    def forward(self, q, k, v, softmax_scale=None):
        return self._drive(self.forward_steps(q, k, v, softmax_scale))

    def staged_inputs_match(self, o: torch.Tensor) -> bool:
        """True when the mirrors still hold the inputs of the forward call that returned ``o``
        (no other forward or full-restage backward ran on this runtime since). Every rank runs the
        same sequence of calls, so every rank reaches the same answer."""
        st = getattr(self, "_staged_for", None)
        return st is not None and st[0] == o.data_ptr() and st[1] == tuple(o.shape)

    # =============================== backward ===================================================
    def bwd_prepare(self, d_o, q, k, v, o, lse, reuse_inputs: bool) -> None:
        sp = self.space
        if not reuse_inputs:
            sp.local("q").copy_(q)
            sp.local("k").copy_(k)
            sp.local("v").copy_(v)
            self._broadcast_kv(k, v)
        sp.local("do").copy_(d_o)
        sp.local("lse").copy_(lse)
        dvec = sp.local("dvec")
        for b in range(self.B):
            E.rowdot(o[b], d_o[b], dvec[b])

    def bwd_compute(self, reuse_inputs: bool, softmax_scale=None) -> None:
        sp, g = self.space, self.rank
        sides = [None] * len(self.b_q_src)
        for p, i in self.b_q_src.items():
            if p == g:
                sides[i] = A.BwdQSide(sp.local("q"), sp.local("do"), sp.local("lse"), sp.local("dvec"),
                                      sp.local("dq_acc"))
            else:
                sides[i] = A.BwdQSide(self.mir[("q", p)], self.mir[("do", p)], self.mir[("lse", p)],
                                      self.mir[("dvec", p)], self.mir[("dq", p)])
        k_srcs = [None] * len(self.b_kv_src)
        v_srcs = [None] * len(self.b_kv_src)
        outs = [None] * len(self.b_kv_src)
        for p, i in self.b_kv_src.items():
            if p == "bc":
                k_srcs[i], v_srcs[i] = sp.local("bc_k"), sp.local("bc_v")
                outs[i] = A.BwdKvOut(sp.local("dk_acc"), sp.local("dv_acc"))     # never written through
                continue
            if p == "bcg":
                k_srcs[i], v_srcs[i] = sp.local("bc_k"), sp.local("bc_v")        # never read through
                # cleared here, after the barrier: the owner's read of the previous call precedes
                # its arrival at that barrier
                sp.local("bc_dk").zero_()
                sp.local("bc_dv").zero_()
                outs[i] = A.BwdKvOut(sp.local("bc_dk"), sp.local("bc_dv"))
                continue
            k_srcs[i] = sp.local("k") if p == g else self.mir[("k", p)]
            v_srcs[i] = sp.local("v") if p == g else self.mir[("v", p)]
            outs[i] = A.BwdKvOut(sp.local("dk_acc") if p == g else sp.peer("dk_acc", p),
                                 sp.local("dv_acc") if p == g else sp.peer("dv_acc", p))
        self.bwd_calls += 1
        which = 0 if reuse_inputs else 1
        stage = self.b_stage if reuse_inputs else self.b_stage_full
        if stage is not None:
            # each of the two staging variants has its own flag counters and call count
            stage.epoch += 1
        A.attn_bwd(sides, k_srcs, v_srcs, outs, self.b_plans[which], softmax_scale, stage)
        # push the accumulated dQ of every foreign row to its owner, once
        for r in self.remote_rows:
            p = int(self.cmap[r])
            tok = self._tok(r)
            for b in range(self.B):
                E.peer_add_(sp.peer("dq_acc", p)[b, tok], self.mir[("dq", p)][b, self._mtok("r", r)], zero_src=True)

    def bwd_finish(self):
        sp = self.space
        if self.nvls_reduce:
            for c in self.bc_cols:
                if int(self.cmap[c]) != self.rank:
                    continue
                bs = slice(self.bc_slot[c] * self.blk, (self.bc_slot[c] + 1) * self.blk)
                for b in range(self.B):
                    sp.multicast_reduce("bc_dk", (b, bs), sp.local("dk_acc")[b, self._tok(c)])
                    sp.multicast_reduce("bc_dv", (b, bs), sp.local("dv_acc")[b, self._tok(c)])
        outs = []
        for name, like in (("dq_acc", (self.B, self.S_loc, self.H, self.D)),
                           ("dk_acc", (self.B, self.S_loc, self.Hk, self.D)),
                           ("dv_acc", (self.B, self.S_loc, self.Hk, self.D))):
            acc = sp.local(name)
            out = torch.empty(like, dtype=self.dtype, device=self.device)
            E.cast_scale(acc, out)
            acc.zero_()
            outs.append(out)
        return tuple(outs)

    def backward_steps(self, d_o, q, k, v, o, lse, softmax_scale=None, reuse_inputs: Optional[bool] = None):
        """The backward call as a generator of barrier channels (see :meth:`forward_steps`)."""
        # the forward's staged Q / K / V are reused only by the backward of that same forward call;
        # after fwd(A), fwd(B) the backward of A restages everything (its inputs were overwritten)
        reuse = self.staged_inputs_match(o) if reuse_inputs is None else reuse_inputs
        self._mark("bwd:begin")
        if self.debug_poison:
            self._poison(("do", "lse", "dvec") if reuse else ("q", "k", "v", "do", "lse", "dvec"))
        self.bwd_prepare(d_o, q, k, v, o, lse, reuse)
        self._mark("bwd_prepare")
        yield 2
        self._mark("bwd_barrier_in")
        if not self.cuda:
            self.stage_on_host(self.b_pieces if reuse else self.b_pieces_full)
        self.bwd_compute(reuse, softmax_scale)
        self._mark("bwd_compute")
        yield 3
        self._mark("bwd_barrier_out")
        res = self.bwd_finish()
        self._mark("bwd_finish")
        if not reuse:
            self._staged_for = None     # the mirrors now hold this backward's inputs, owned by no forward
        return res

    def backward(self, d_o, q, k, v, o, lse, softmax_scale=None, reuse_inputs: Optional[bool] = None):
        return self._drive(self.backward_steps(d_o, q, k, v, o, lse, softmax_scale, reuse_inputs))
