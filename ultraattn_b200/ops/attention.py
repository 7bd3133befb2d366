"""Launch plans and Python entry points for the block-sparse attention kernels.

A *forward plan* is a list of :class:`Row` objects: a block of query tokens plus the key/value
segments it attends to. A *backward plan* is the transposed view: a list of :class:`Col` objects,
a block of key/value tokens plus the query segments that attend to it. Segments name the buffer
they live in by slot number, so one launch can mix this GPU's own tensors, staging buffers filled
from peers and peer memory itself.

Every entry point exists twice: the sm_100a kernel (``*_cuda``) and an fp32 PyTorch restatement of
the same plan semantics (``*_reference``) that runs on CPU and is the oracle of the kernel tests.

Reference behaviour covered: one flash-attention call per scheduled tile with ``causal`` only on
diagonal tiles (orchestrated_attn/orchestrated_attn_impl.py:320-340, 574-597), the LSE-weighted
merge of partial outputs (ring_flash_attn/utils.py:38-52) and the precomputed ``softmax_d``
input of the backward (orchestrated_attn/utils.py:148-188).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from .. import _lib

TILE = 128
CTA_ROWS = 256
KERNEL_HEAD_DIM = 128          # head dim the sm_100a kernels are built for


@dataclass(frozen=True)
class Seg:
    """A run of tokens in source slot ``src`` starting at ``start``.

    ``causal``: key c of the segment is visible to query r of the block iff ``c <= r + diag``
    (both 0-based inside their block / segment).
    """
    src: int
    start: int
    length: int
    causal: bool = False
    diag: int = 0
    wait_flag: int = 0       # 0: in place; f > 0: wait for staging flag f - 1 to reach wait_count
    wait_count: int = 0


@dataclass
class Row:
    """Forward work item: ``q_len`` queries at ``q_start`` of source ``q_src`` attend ``segs``;
    the result goes to rows ``o_start...`` of output slot ``o_slot`` (merged into what is there
    when ``accumulate``)."""
    q_src: int
    q_start: int
    q_len: int
    segs: Sequence[Seg]
    o_slot: int = 0
    o_start: int = 0
    accumulate: bool = False
    q_wait_flag: int = 0
    q_wait_count: int = 0


@dataclass
class Col:
    """Backward work item: ``kv_len`` keys at ``kv_start`` of source ``kv_src`` are attended by the
    query segments ``segs`` (``Seg.src`` indexes the query-side sources; causal condition as in
    :class:`Seg` with r the query index inside the segment and c the key index inside this
    block: visible iff ``c <= r + diag``). dK/dV are accumulated (fp32) at rows ``g_start...`` of
    gradient slot ``g_slot``."""
    kv_src: int
    kv_start: int
    kv_len: int
    segs: Sequence[Seg]
    g_slot: int = 0
    g_start: int = 0
    kv_wait_flag: int = 0
    kv_wait_count: int = 0


@dataclass
class StagePlan:
    """In-kernel staging prologue: ``tasks`` is an int64 device tensor [n, 4] of
    (src pointer, dst pointer, number of 16-byte vectors, flag index); ``flags`` a uint32 device
    tensor of monotonically increasing counters."""
    tasks: torch.Tensor
    n_tasks: int
    n_copy_ctas: int
    flags: torch.Tensor
    epoch: int = 1
    ticket: torch.Tensor | None = None      # one uint32: next unclaimed task of a launch (the launcher zeroes it)


def _launch_order(tiles: list) -> list:
    """Order of the CTAs of a launch. ``tiles``: (cost, group, index) with group = the block row
    (forward) or block column (backward) that the tile belongs to. Tiles of one group walk the SAME
    list of key/value (or query) blocks; started together they stream it in step and a block comes
    out of DRAM once for all of them, whereas a pure heaviest-first order interleaves groups of
    similar cost and every CTA then fetches its blocks from DRAM alone (measured on a global + local
    pattern, whose rows all cost about the same: 15 % of the launch time). So: groups by their
    heaviest tile, heaviest group first (the tail of the launch is then made of light CTAs); inside
    a group heaviest tile first."""
    top = {}
    for cost, g, _ in tiles:
        top[g] = max(top.get(g, 0), cost)
    return sorted(tiles, key=lambda x: (-top[x[1]], x[1], -x[0], x[2]))


def _seg_tiles(seg: Seg, r0: int, rows_here: int) -> int:
    n = (seg.length + TILE - 1) // TILE
    if seg.causal:
        last = r0 + rows_here - 1 + seg.diag
        if last < 0:
            return 0
        n = min(n, last // TILE + 1)
    return n


class FwdPlan:
    """Device-resident tables for one forward launch (rows, segments, tile list in launch order)."""

    def __init__(self, rows: Sequence[Row], device: torch.device | str = "cpu"):
        self.rows = list(rows)
        row_arr = np.zeros((max(len(self.rows), 1), 10), dtype=np.int32)
        segs = []
        tiles = []
        for ri, r in enumerate(self.rows):
            b = len(segs)
            for s in r.segs:
                segs.append((s.src, s.start, s.length, int(s.causal), s.diag, s.wait_flag, s.wait_count, 0))
            row_arr[ri] = (r.q_src, r.q_start, r.q_len, b, len(segs), r.o_slot, r.o_start,
                           int(r.accumulate), r.q_wait_flag, r.q_wait_count)
            for t in range((r.q_len + CTA_ROWS - 1) // CTA_ROWS):
                r0 = t * CTA_ROWS
                rows_here = min(CTA_ROWS, r.q_len - r0)
                cost = sum(_seg_tiles(s, r0, rows_here) for s in r.segs)
                tiles.append((cost, ri, t))
        tiles = _launch_order(tiles)
        self.n_tiles = len(tiles)
        self.total_key_tiles = sum(c for c, _, _ in tiles)
        seg_arr = np.array(segs, dtype=np.int32).reshape(-1, 8) if segs else np.zeros((1, 8), np.int32)
        tile_arr = (np.array([(ri, t) for _, ri, t in tiles], dtype=np.int32).reshape(-1, 2)
                    if tiles else np.zeros((1, 2), np.int32))
        self.device = torch.device(device)
        self.rows_t = torch.from_numpy(row_arr).to(self.device)
        self.segs_t = torch.from_numpy(seg_arr).to(self.device)
        self.tiles_t = torch.from_numpy(tile_arr).to(self.device)


# ---------------------------------------------------------------------------------------------
# Debug mode: bounds of the launch tables. The kernels are table driven: every address they form
# is (source slot, first token, length) from a Row / Col / Seg, so checking the tables against the
# tensors actually passed covers every index the device code will compute. ``UA_DEBUG_BOUNDS=1``
# runs the check before every launch (also on the CPU restatements); it costs host time only.
# ---------------------------------------------------------------------------------------------
def debug_bounds_enabled() -> bool:
    import os
    return os.environ.get("UA_DEBUG_BOUNDS") == "1"


def check_fwd_tables(rows: Sequence["Row"], q_srcs, k_srcs, v_srcs, outs, stage=None) -> list:
    """Problems (strings) in a forward launch's tables; empty = every access is in range."""
    bad = []
    for i, r in enumerate(rows):
        if not 0 <= r.q_src < len(q_srcs):
            bad.append(f"row {i}: query slot {r.q_src} of {len(q_srcs)}")
            continue
        if r.q_start < 0 or r.q_len <= 0 or r.q_start + r.q_len > q_srcs[r.q_src].shape[1]:
            bad.append(f"row {i}: queries {r.q_start}+{r.q_len} exceed {q_srcs[r.q_src].shape[1]} tokens of slot {r.q_src}")
        if not 0 <= r.o_slot < len(outs):
            bad.append(f"row {i}: output slot {r.o_slot} of {len(outs)}")
        else:
            o, lse = outs[r.o_slot]
            if r.o_start < 0 or r.o_start + r.q_len > o.shape[1] or r.o_start + r.q_len > lse.shape[2]:
                bad.append(f"row {i}: output rows {r.o_start}+{r.q_len} exceed slot {r.o_slot} ({o.shape[1]} rows)")
        if stage is not None and r.q_wait_flag and not 0 < r.q_wait_flag <= stage.flags.numel():
            bad.append(f"row {i}: wait flag {r.q_wait_flag} outside {stage.flags.numel()} counters")
        for jx, sg in enumerate(r.segs):
            if not 0 <= sg.src < len(k_srcs):
                bad.append(f"row {i} segment {jx}: key slot {sg.src} of {len(k_srcs)}")
                continue
            for name, t in (("keys", k_srcs[sg.src]), ("values", v_srcs[sg.src])):
                if sg.start < 0 or sg.length <= 0 or sg.start + sg.length > t.shape[1]:
                    bad.append(f"row {i} segment {jx}: {name} {sg.start}+{sg.length} exceed {t.shape[1]} tokens of slot {sg.src}")
            if stage is not None and sg.wait_flag and not 0 < sg.wait_flag <= stage.flags.numel():
                bad.append(f"row {i} segment {jx}: wait flag {sg.wait_flag} outside {stage.flags.numel()} counters")
    return bad


def check_bwd_tables(cols: Sequence["Col"], q_sides, k_srcs, v_srcs, kv_outs, stage=None) -> list:
    """Problems (strings) in a backward launch's tables; empty = every access is in range."""
    bad = []
    for i, c in enumerate(cols):
        if not 0 <= c.kv_src < len(k_srcs):
            bad.append(f"column {i}: key slot {c.kv_src} of {len(k_srcs)}")
            continue
        if c.kv_start < 0 or c.kv_len <= 0 or c.kv_start + c.kv_len > k_srcs[c.kv_src].shape[1] \
                or c.kv_start + c.kv_len > v_srcs[c.kv_src].shape[1]:
            bad.append(f"column {i}: keys {c.kv_start}+{c.kv_len} exceed slot {c.kv_src}")
        if not 0 <= c.g_slot < len(kv_outs):
            bad.append(f"column {i}: gradient slot {c.g_slot} of {len(kv_outs)}")
        elif c.g_start < 0 or c.g_start + c.kv_len > kv_outs[c.g_slot].dk.shape[1]:
            bad.append(f"column {i}: gradient rows {c.g_start}+{c.kv_len} exceed slot {c.g_slot} "
                       f"({kv_outs[c.g_slot].dk.shape[1]} rows)")
        if stage is not None and c.kv_wait_flag and not 0 < c.kv_wait_flag <= stage.flags.numel():
            bad.append(f"column {i}: wait flag {c.kv_wait_flag} outside {stage.flags.numel()} counters")
        for jx, sg in enumerate(c.segs):
            if not 0 <= sg.src < len(q_sides):
                bad.append(f"column {i} segment {jx}: query slot {sg.src} of {len(q_sides)}")
                continue
            side = q_sides[sg.src]
            for name, n in (("q", side.q.shape[1]), ("dO", side.d_o.shape[1]), ("lse", side.lse.shape[2]),
                            ("D", side.dvec.shape[2]), ("dQ", side.dq.shape[1])):
                if sg.start < 0 or sg.length <= 0 or sg.start + sg.length > n:
                    bad.append(f"column {i} segment {jx}: {name} rows {sg.start}+{sg.length} exceed {n} of slot {sg.src}")
            if stage is not None and sg.wait_flag and not 0 < sg.wait_flag <= stage.flags.numel():
                bad.append(f"column {i} segment {jx}: wait flag {sg.wait_flag} outside {stage.flags.numel()} counters")
    return bad


def _raise_if_bad(kind: str, problems: list) -> None:
    if problems:
        raise IndexError(f"{kind} launch tables address memory out of range: " + "; ".join(problems[:8])
                         + (f" (+{len(problems) - 8} more)" if len(problems) > 8 else ""))


_status: dict[int, torch.Tensor] = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """int32[4] per device: [code, where, block, extra]; written by a kernel whose wait ran out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device: torch.device | None = None) -> None:
    """Synchronises and raises if any kernel on ``device`` reported a bounded wait that ran out."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    st = status_buffer(device).cpu().tolist()
    if st[0] != 0:
        status_buffer(device).zero_()
        raise RuntimeError(f"ultraattn kernel error code={st[0]} where={st[1]} block={st[2]} extra={st[3]}")


# ---------------------------------------------------------------------------------------------
# Per-CTA time stamps of the attention launches (normal build; see csrc/attn_common.cuh KernelTrace)
# ---------------------------------------------------------------------------------------------
_traces: dict = {}


def enable_kernel_trace(device: torch.device, max_ctas: int = 1 << 18) -> None:
    """From now on every forward / backward launch on ``device`` records, for each of its first
    ``max_ctas`` CTAs: start, end of its staging copies, end (``globaltimer`` ns), SM id and work
    item. A launch overwrites the record of the previous launch of the same kernel."""
    import ctypes
    lib = _lib.load()
    lib.ua_set_kernel_trace.restype = ctypes.c_int
    lib.ua_set_kernel_trace.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
    idx = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(idx):
        for which in (0, 1):
            buf = torch.zeros(max_ctas, 4, dtype=torch.int64, device=torch.device("cuda", idx))
            _traces[(idx, which)] = buf
            if lib.ua_set_kernel_trace(which, buf.data_ptr(), max_ctas) != 0:
                raise RuntimeError(lib.ua_last_error().decode())


def disable_kernel_trace(device: torch.device) -> None:
    lib = _lib.load()
    idx = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(idx):
        for which in (0, 1):
            if _traces.pop((idx, which), None) is not None:
                lib.ua_set_kernel_trace(which, None, 0)


def read_kernel_trace(device: torch.device, kernel: str = "fwd") -> "np.ndarray":
    """int64 [n_ctas, 4] of the last ``kernel`` ("fwd" / "bwd") launch: start, staged, end, (sm << 32 | item);
    rows of CTAs that did not run are zero and dropped. Synchronises the device."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _traces[(idx, 0 if kernel == "fwd" else 1)]
    torch.cuda.synchronize(idx)
    arr = buf.cpu().numpy()
    out = arr[arr[:, 0] != 0].copy()
    buf.zero_()
    return out


def tensor_map_cache_stats() -> tuple[int, int]:
    """(hits, misses) of the library's host-side cache of encoded TMA tensor maps. A step that
    reuses its buffers (same addresses, shapes and strides) encodes nothing after its first run."""
    import ctypes
    lib = _lib.load()
    lib.ua_tmap_cache_stats.restype = ctypes.c_int
    lib.ua_tmap_cache_stats.argtypes = [ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_ulonglong)]
    h, m = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
    lib.ua_tmap_cache_stats(ctypes.byref(h), ctypes.byref(m))
    return int(h.value), int(m.value)


def _src_struct(t: torch.Tensor) -> _lib.UaTensorSrc:
    assert t.dim() == 4 and t.dtype == torch.bfloat16 and t.stride(3) == 1 and t.shape[3] == 128, \
        "attention sources must be bf16 [batch, tokens, heads, 128] with contiguous head dim"
    return _lib.UaTensorSrc(t.data_ptr(), t.shape[1], t.shape[2], t.shape[0], t.stride(1),
                            t.stride(2), t.stride(0))


def attn_fwd_cuda(q_srcs: Sequence[torch.Tensor], k_srcs: Sequence[torch.Tensor],
                  v_srcs: Sequence[torch.Tensor], outs: Sequence[tuple[torch.Tensor, torch.Tensor]],
                  plan: FwdPlan, softmax_scale: float | None = None,
                  stage: "StagePlan | None" = None) -> None:
    """Run the sm_100a forward. Tensors are ``[batch, tokens, heads, 128]`` bf16; each output is a
    pair ``(O [batch, tokens, heads, 128] bf16, lse [batch, heads, tokens] fp32)`` written in
    place."""
    lib = _lib.load()
    q0 = q_srcs[0]
    n_heads = q0.shape[2]
    n_kv_heads = k_srcs[0].shape[2]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q0.shape[3])
    qs = (_lib.UaTensorSrc * len(q_srcs))(*[_src_struct(t) for t in q_srcs])
    ks = (_lib.UaTensorSrc * len(k_srcs))(*[_src_struct(t) for t in k_srcs])
    vs = (_lib.UaTensorSrc * len(v_srcs))(*[_src_struct(t) for t in v_srcs])
    od = []
    for o, lse in outs:
        assert o.dtype == torch.bfloat16 and lse.dtype == torch.float32 and o.stride(3) == 1
        assert o.stride(2) == 128 and lse.stride(2) == 1
        od.append(_lib.UaOutDst(o.data_ptr(), lse.data_ptr(), o.stride(1), o.stride(0),
                                lse.stride(1), lse.stride(0)))
    ods = (_lib.UaOutDst * len(od))(*od)
    st = status_buffer(q0.device)
    rc = lib.ua_attn_fwd(qs, len(q_srcs), ks, vs, len(k_srcs), ods, len(od),
                         plan.rows_t.data_ptr(), plan.segs_t.data_ptr(), plan.tiles_t.data_ptr(),
                         plan.n_tiles, n_heads, n_kv_heads, q0.shape[0], scale, st.data_ptr(),
                         *_stage_args(stage),
                         torch.cuda.current_stream(q0.device).cuda_stream)
    _lib.check(rc, "ua_attn_fwd")


def _stage_args(stage):
    if stage is None:
        return (None, 0, 0, None, 1, None)
    if stage.ticket is None:
        stage.ticket = torch.zeros(1, dtype=torch.int32, device=stage.flags.device)
    return (stage.tasks.data_ptr() if stage.n_tasks else None, stage.n_tasks, stage.n_copy_ctas,
            stage.flags.data_ptr(), stage.epoch, stage.ticket.data_ptr())


def _mask_for(seg: Seg, q_len: int, device) -> torch.Tensor | None:
    if not seg.causal:
        return None
    r = torch.arange(q_len, device=device)[:, None]
    c = torch.arange(seg.length, device=device)[None, :]
    return c <= r + seg.diag


def attn_fwd_reference(q_srcs, k_srcs, v_srcs, outs, rows: Sequence[Row],
                       softmax_scale: float | None = None) -> None:
    """fp32 PyTorch restatement of :func:`attn_fwd_cuda` (any device, any head dim)."""
    d = q_srcs[0].shape[3]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    group = q_srcs[0].shape[2] // k_srcs[0].shape[2]
    for r in rows:
        q = q_srcs[r.q_src][:, r.q_start:r.q_start + r.q_len].float()       # [B, q, H, D]
        scores = []
        vals = []
        for s in r.segs:
            k = k_srcs[s.src][:, s.start:s.start + s.length].float()
            v = v_srcs[s.src][:, s.start:s.start + s.length].float()
            if group > 1:
                k = k.repeat_interleave(group, dim=2)
                v = v.repeat_interleave(group, dim=2)
            sc = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
            m = _mask_for(s, r.q_len, q.device)
            if m is not None:
                sc = sc.masked_fill(~m[None, None], float("-inf"))
            scores.append(sc)
            vals.append(v)
        o_t, lse_t = outs[r.o_slot]
        osl = slice(r.o_start, r.o_start + r.q_len)
        if scores:
            sc = torch.cat(scores, dim=-1)
            v = torch.cat(vals, dim=1)
            lse = torch.logsumexp(sc, dim=-1)                                # [B, H, q]
            p = torch.exp(sc - lse.masked_fill(lse == float("-inf"), 0.0)[..., None])
            p = torch.where(torch.isfinite(sc), p, torch.zeros_like(p))
            o = torch.einsum("bhqk,bkhd->bqhd", p, v)
        else:
            o = torch.zeros_like(q)
            lse = torch.full((q.shape[0], q.shape[2], r.q_len), float("-inf"), device=q.device)
        if r.accumulate:
            lse_old = lse_t[:, :, osl].float()
            o_old = o_t[:, osl].float()
            tot = torch.logaddexp(lse_old, lse)
            safe = tot.masked_fill(tot == float("-inf"), 0.0)
            w_old = torch.where(torch.isfinite(lse_old), torch.exp(lse_old - safe), torch.zeros_like(tot))
            w_new = torch.where(torch.isfinite(lse), torch.exp(lse - safe), torch.zeros_like(tot))
            o = o_old * w_old.transpose(1, 2)[..., None] + o * w_new.transpose(1, 2)[..., None]
            lse = tot
        o_t[:, osl] = o.to(o_t.dtype)
        lse_t[:, :, osl] = lse.to(lse_t.dtype)


def attn_fwd(q_srcs, k_srcs, v_srcs, outs, plan: FwdPlan, softmax_scale=None, stage=None) -> None:
    """Dispatch on the device of the inputs: CUDA tensors run the sm_100a kernel, CPU tensors the
    fp32 restatement (which expects staged data to be in place already)."""
    if debug_bounds_enabled():
        _raise_if_bad("forward", check_fwd_tables(plan.rows, q_srcs, k_srcs, v_srcs, outs, stage))
    if q_srcs[0].is_cuda:
        attn_fwd_cuda(q_srcs, k_srcs, v_srcs, outs, plan, softmax_scale, stage)
    else:
        attn_fwd_reference(q_srcs, k_srcs, v_srcs, outs, plan.rows, softmax_scale)


def rows_from_block_table(table: np.ndarray, block: int, kv_block: int | None = None) -> list[Row]:
    """Single-buffer forward rows for a square block table (0 empty, 1 full, 2 causal)."""
    kv_block = kv_block or block
    rows = []
    for i in range(table.shape[0]):
        segs = []
        for j in range(table.shape[1]):
            t = int(table[i, j])
            if t == 0:
                continue
            # merge with the previous segment when both are full and contiguous
            if t == 1 and segs and not segs[-1].causal and segs[-1].start + segs[-1].length == j * kv_block:
                p = segs[-1]
                segs[-1] = Seg(0, p.start, p.length + kv_block, False, 0)
            else:
                segs.append(Seg(0, j * kv_block, kv_block, t == 2, 0))
        rows.append(Row(0, i * block, block, tuple(segs), 0, i * block, False))
    return rows


# =================================================================================================
# backward
# =================================================================================================
BWD_QT = 128


def _col_steps(c: Col, c0: int) -> int:
    n = 0
    for s in c.segs:
        nq = (s.length + BWD_QT - 1) // BWD_QT
        first = 0
        if s.causal:
            r_min = c0 - s.diag
            first = 0 if r_min <= 0 else r_min // BWD_QT
        n += max(0, nq - first)
    return n


class BwdPlan:
    """Device-resident tables for one backward launch (columns, query segments, tile list)."""

    def __init__(self, cols: Sequence[Col], device: torch.device | str = "cpu"):
        self.cols = list(cols)
        col_arr = np.zeros((max(len(self.cols), 1), 10), dtype=np.int32)
        segs = []
        tiles = []
        for ci, c in enumerate(self.cols):
            b = len(segs)
            for s in c.segs:
                segs.append((s.src, s.start, s.length, int(s.causal), s.diag, s.wait_flag, s.wait_count, 0))
            col_arr[ci] = (c.kv_src, c.kv_start, c.kv_len, b, len(segs), c.g_slot, c.g_start, 0,
                           c.kv_wait_flag, c.kv_wait_count)
            for t in range((c.kv_len + TILE - 1) // TILE):
                tiles.append((_col_steps(c, t * TILE), ci, t))
        tiles = _launch_order(tiles)
        self.n_tiles = len(tiles)
        self.total_steps = sum(c for c, _, _ in tiles)
        seg_arr = np.array(segs, dtype=np.int32).reshape(-1, 8) if segs else np.zeros((1, 8), np.int32)
        tile_arr = (np.array([(ci, t) for _, ci, t in tiles], dtype=np.int32).reshape(-1, 2)
                    if tiles else np.zeros((1, 2), np.int32))
        self.device = torch.device(device)
        self.cols_t = torch.from_numpy(col_arr).to(self.device)
        self.segs_t = torch.from_numpy(seg_arr).to(self.device)
        self.tiles_t = torch.from_numpy(tile_arr).to(self.device)


@dataclass
class BwdQSide:
    """Query-side tensors of one source: q, dO ``[B, T, H, 128]`` bf16; lse, dvec ``[B, H, T]``
    fp32; dq ``[B, T, H, 128]`` fp32 accumulator (added into)."""
    q: torch.Tensor
    d_o: torch.Tensor
    lse: torch.Tensor
    dvec: torch.Tensor
    dq: torch.Tensor


@dataclass
class BwdKvOut:
    """dK / dV destination ``[B, T, Hkv, 128]``: bf16 (overwritten) or fp32 (added into)."""
    dk: torch.Tensor
    dv: torch.Tensor

    @property
    def add_f32(self) -> bool:
        return self.dk.dtype == torch.float32


def attn_bwd_cuda(q_sides: Sequence[BwdQSide], k_srcs, v_srcs, kv_outs: Sequence[BwdKvOut],
                  plan: BwdPlan, softmax_scale: float | None = None, stage=None) -> None:
    lib = _lib.load()
    q0 = q_sides[0].q
    n_heads = q0.shape[2]
    n_kv_heads = k_srcs[0].shape[2]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q0.shape[3])
    nq = len(q_sides)
    qs = (_lib.UaTensorSrc * nq)(*[_src_struct(s.q) for s in q_sides])
    dos = (_lib.UaTensorSrc * nq)(*[_src_struct(s.d_o) for s in q_sides])
    side = []
    for s in q_sides:
        assert s.lse.dtype == torch.float32 and s.dvec.dtype == torch.float32 and s.dq.dtype == torch.float32
        assert s.lse.stride(2) == 1 and s.lse.stride() == s.dvec.stride()
        assert s.dq.stride(3) == 1 and s.dq.stride(2) == 128
        side.append(_lib.UaBwdQSide(s.lse.data_ptr(), s.dvec.data_ptr(), s.lse.stride(1),
                                    s.lse.stride(0), s.dq.data_ptr(), s.dq.stride(1), s.dq.stride(0)))
    sides = (_lib.UaBwdQSide * nq)(*side)
    ks = (_lib.UaTensorSrc * len(k_srcs))(*[_src_struct(t) for t in k_srcs])
    vs = (_lib.UaTensorSrc * len(v_srcs))(*[_src_struct(t) for t in v_srcs])
    ko = []
    for o in kv_outs:
        assert o.dk.stride(3) == 1 and o.dk.stride(2) == 128 and o.dk.stride() == o.dv.stride()
        ko.append(_lib.UaBwdKvOut(o.dk.data_ptr(), o.dv.data_ptr(), o.dk.stride(1), o.dk.stride(0),
                                  int(o.add_f32), 0))
    kos = (_lib.UaBwdKvOut * len(ko))(*ko)
    st = status_buffer(q0.device)
    rc = lib.ua_attn_bwd(qs, dos, sides, nq, ks, vs, len(k_srcs), kos, len(ko),
                         plan.cols_t.data_ptr(), plan.segs_t.data_ptr(), plan.tiles_t.data_ptr(),
                         plan.n_tiles, n_heads, n_kv_heads, q0.shape[0], scale, st.data_ptr(),
                         *_stage_args(stage),
                         torch.cuda.current_stream(q0.device).cuda_stream)
    _lib.check(rc, "ua_attn_bwd")


def attn_bwd_reference(q_sides: Sequence[BwdQSide], k_srcs, v_srcs, kv_outs: Sequence[BwdKvOut],
                       cols: Sequence[Col], softmax_scale: float | None = None) -> None:
    """fp32 PyTorch restatement of :func:`attn_bwd_cuda` (uses lse and D exactly like the kernel)."""
    d = q_sides[0].q.shape[3]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    group = q_sides[0].q.shape[2] // k_srcs[0].shape[2]
    for c in cols:
        k = k_srcs[c.kv_src][:, c.kv_start:c.kv_start + c.kv_len].float()
        v = v_srcs[c.kv_src][:, c.kv_start:c.kv_start + c.kv_len].float()
        kk = k.repeat_interleave(group, dim=2) if group > 1 else k
        vv = v.repeat_interleave(group, dim=2) if group > 1 else v
        dk = torch.zeros_like(kk)
        dv = torch.zeros_like(vv)
        for s in c.segs:
            qs = q_sides[s.src]
            sl = slice(s.start, s.start + s.length)
            q = qs.q[:, sl].float()
            do = qs.d_o[:, sl].float()
            lse = qs.lse[:, :, sl].float()
            dvec = qs.dvec[:, :, sl].float()
            sc = torch.einsum("bqhd,bkhd->bhqk", q, kk) * scale
            lse_safe = torch.where(torch.isfinite(lse), lse, torch.full_like(lse, float("inf")))
            p = torch.exp(sc - lse_safe[..., None])
            if s.causal:
                r = torch.arange(s.length, device=q.device)[:, None]
                cc = torch.arange(c.kv_len, device=q.device)[None, :]
                p = p * (cc <= r + s.diag)[None, None].to(p.dtype)
            dp = torch.einsum("bqhd,bkhd->bhqk", do, vv)
            ds = p * (dp - dvec[..., None])
            dv += torch.einsum("bhqk,bqhd->bkhd", p, do)
            dk += torch.einsum("bhqk,bqhd->bkhd", ds, q) * scale
            qs.dq[:, sl] += (torch.einsum("bhqk,bkhd->bqhd", ds, kk) * scale).to(qs.dq.dtype)
        if group > 1:
            B, T, H, D = dk.shape
            dk = dk.view(B, T, H // group, group, D).sum(3)
            dv = dv.view(B, T, H // group, group, D).sum(3)
        out = kv_outs[c.g_slot]
        gsl = slice(c.g_start, c.g_start + c.kv_len)
        if out.add_f32:
            out.dk[:, gsl] += dk
            out.dv[:, gsl] += dv
        else:
            out.dk[:, gsl] = dk.to(out.dk.dtype)
            out.dv[:, gsl] = dv.to(out.dv.dtype)


def attn_bwd(q_sides, k_srcs, v_srcs, kv_outs, plan: BwdPlan, softmax_scale=None, stage=None) -> None:
    if debug_bounds_enabled():
        _raise_if_bad("backward", check_bwd_tables(plan.cols, q_sides, k_srcs, v_srcs, kv_outs, stage))
    if q_sides[0].q.is_cuda:
        attn_bwd_cuda(q_sides, k_srcs, v_srcs, kv_outs, plan, softmax_scale, stage)
    else:
        attn_bwd_reference(q_sides, k_srcs, v_srcs, kv_outs, plan.cols, softmax_scale)


def cols_from_block_table(table: np.ndarray, block: int, kv_block: int | None = None) -> list[Col]:
    """Single-buffer backward columns for a block table (0 empty, 1 full, 2 causal)."""
    kv_block = kv_block or block
    cols = []
    for j in range(table.shape[1]):
        segs = []
        for i in range(table.shape[0]):
            t = int(table[i, j])
            if t == 0:
                continue
            if t == 1 and segs and not segs[-1].causal and segs[-1].start + segs[-1].length == i * block:
                p = segs[-1]
                segs[-1] = Seg(0, p.start, p.length + block, False, 0)
            else:
                segs.append(Seg(0, i * block, block, t == 2, 0))
        cols.append(Col(0, j * kv_block, kv_block, tuple(segs), 0, j * kv_block))
    return cols
