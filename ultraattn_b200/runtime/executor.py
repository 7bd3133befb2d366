"""Plan executor: runs an :class:`~ultraattn_b200.planner.schedule.Execution_Plan` on real ranks.

The same walker serves two back ends:
  * CPU ranks over ``gloo`` in fp32 — the numerically exact reference executor that checks
    plan -> execution -> result against the dense oracle without a GPU;
  * CUDA ranks over NCCL point-to-point — the "NCCL path", i.e. the reference's design done
    correctly: three streams per rank (compute / send / receive), the rank launches its kernels in
    plan order, cross-stream ordering comes from events on the graph edges, whole-tile bundles per
    message. It is the baseline that the fused path is compared against.

What the reference's runtime does (orchestrated_attn/orchestrated_attn_impl.py:62-130, 300-350) is
kept: plan-order launch, per-kernel events, NVTX ranges named by kernel key. What it leaves out
(orchestrated_attn/utils.py:119-134, 260-262, 296-298 are stubs) is supplied: partial (O, lse)
are merged with the log-sum-exp rule, partial dQ / dK / dV are accumulated in fp32, each tile
has its own buffers.

Data bundles per message (one flat buffer each, like the reference's carriers):
  forward   input row  Q            input col  K|V        output row  O|lse
  backward  input row  Q|dO|lse|D   input col  K|V        output row  dQ(fp32)   output col  dK|dV(fp32)
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..ops import attention as A
from ..ops import elementwise as E
from ..parallel.comm import count_comm, set_comm_phase
from ..patterns.blocks import CAUSAL


class FaultInjector:
    """Host-side fault injection for tests: drop or delay chosen messages, or make a rank raise
    before a chosen kernel. Nothing here touches a GPU."""

    def __init__(self, drop_keys=(), raise_before=None, delay_s: float = 0.0):
        self.drop_keys = set(drop_keys)
        self.raise_before = raise_before
        self.delay_s = delay_s

    def before(self, kernel) -> bool:
        """Returns False if the kernel must be skipped (message dropped)."""
        if self.raise_before is not None and kernel.key == self.raise_before:
            raise RuntimeError(f"injected failure before kernel {kernel.key}")
        if kernel.key in self.drop_keys:
            return False
        if self.delay_s:
            import time
            time.sleep(self.delay_s)
        return True


class PlanExecutor:
    """Executes forward and backward plans of one intra-node CP group.

    ``group``: the process group of the CP ranks (plan rank g = group rank g).
    ``recv_timeout_s``: how long a receive may wait before the step fails with an error instead
    of hanging (host-side failure detection).
    """

    def __init__(self, plan_fwd, plan_bwd=None, group=None, device: Optional[torch.device] = None,
                 recv_timeout_s: float = 60.0, fault: Optional[FaultInjector] = None,
                 p2p_groups=None):
        self.plan_fwd = plan_fwd
        self.plan_bwd = plan_bwd
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = device or torch.device("cpu")
        self.cuda = self.device.type == "cuda"
        self.recv_timeout_s = recv_timeout_s
        self.fault = fault
        self.p2p_groups = p2p_groups        # (low->high group, high->low group) for full duplex on NCCL
        da = plan_fwd.da_config
        self.da = da
        self.par_d = plan_fwd.split_degrees[0]
        self.cp = plan_fwd.hierarchy_sp
        assert self.cp == self.world, f"plan is for {self.cp} ranks, group has {self.world}"
        self.smap = np.asarray(plan_fwd.d_graph.schedule.S_map)[0]
        self.my_blocks = [i for i in range(self.par_d) if self.smap[i] == self.rank]
        self.blk = da.S[0] // self.par_d
        self.table_int = da.bsa_config.bsa_repr.refined(self.par_d) if self.par_d >= da.bsa_config.table.shape[0] \
            else None
        if self.cuda:
            self.streams = [torch.cuda.Stream(device=self.device) for _ in range(3)]
        self.bytes_sent = 0
        self.bytes_recv = 0
        self._done: set = set()
        self._done_keep: list = []

    # -------------------------------------------------------------------------------------------
    def _global_rank(self, g: int) -> int:
        return dist.get_global_rank(self.group, g) if self.group is not None else g

    def _tile_type(self, r: int, c: int) -> int:
        assert self.table_int is not None, "the schedule must be at least as fine as the pattern"
        return int(self.table_int[r, c])

    def _local_block(self, t: torch.Tensor, blk_id: int) -> torch.Tensor:
        """View of block ``blk_id`` inside this rank's shard [B, S_local, ...]."""
        k = self.my_blocks.index(blk_id)
        return t[:, k * self.blk:(k + 1) * self.blk]

    def _pg_for(self, src: int, dst: int):
        if self.p2p_groups is None:
            return self.group
        return self.p2p_groups[0] if src < dst else self.p2p_groups[1]

    def _walk_order(self, kernel_list):
        """Launch order. On CUDA it is the plan's order (launches are asynchronous). A CPU rank
        executes compute synchronously, so it first posts every message that needs no compute
        result — all input messages and the receives of output messages — and then walks the
        plan; otherwise two ranks could each block in a compute kernel whose input the other
        would only send later in its list."""
        if self.cuda:
            return list(kernel_list)
        g = self.rank
        early = [k for k in kernel_list if k.type == "comm" and (k.key[5] == "i" or k.key[4] == g)]
        early_ids = {id(k) for k in early}
        return early + [k for k in kernel_list if id(k) not in early_ids]

    # ------------------------------- message passing --------------------------------------------
    def _send(self, buf: torch.Tensor, kernel, stream_idx: int, deps):
        dst = self._global_rank(kernel.key[4])
        self.bytes_sent += buf.numel() * buf.element_size()
        count_comm(send_bytes=buf.numel() * buf.element_size())
        if self.cuda:
            st = self.streams[stream_idx]
            for e in deps:
                st.wait_event(e)
            with torch.cuda.stream(st):
                dist.send(buf, dst, group=self._pg_for(kernel.key[3], kernel.key[4]))
                ev = torch.cuda.Event()
                ev.record(st)
            return ev
        return dist.isend(buf, dst, group=self.group, tag=_tag(kernel))

    def _recv(self, buf: torch.Tensor, kernel, stream_idx: int, deps):
        src = self._global_rank(kernel.key[3])
        self.bytes_recv += buf.numel() * buf.element_size()
        count_comm(recv_bytes=buf.numel() * buf.element_size())
        if self.cuda:
            st = self.streams[stream_idx]
            for e in deps:
                st.wait_event(e)
            with torch.cuda.stream(st):
                dist.recv(buf, src, group=self._pg_for(kernel.key[3], kernel.key[4]))
                ev = torch.cuda.Event()
                ev.record(st)
            return ev
        return dist.irecv(buf, src, group=self.group, tag=_tag(kernel))

    def _wait(self, handle, what) -> None:
        """CPU path: wait for an async gloo request with a deadline."""
        if handle is None or self.cuda or isinstance(handle, torch.Tensor):
            return
        if id(handle) in self._done:        # a gloo request must not be waited on twice
            return
        import datetime
        try:
            ok = handle.wait(timeout=datetime.timedelta(seconds=self.recv_timeout_s))
        except RuntimeError as e:       # gloo reports an expired deadline as a RuntimeError
            raise TimeoutError(f"rank {self.rank}: {what} did not complete within "
                               f"{self.recv_timeout_s} s (peer failed or message lost): {e}") from e
        if ok is False:
            raise TimeoutError(f"rank {self.rank}: {what} did not complete within "
                               f"{self.recv_timeout_s} s (peer failed or message lost)")
        self._done.add(id(handle))
        self._done_keep.append(handle)

    # =============================== forward ====================================================
    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale=None):
        """q/k/v: this rank's shard ``[B, S/CP, H, D]`` (blocks in ``my_blocks`` order).
        Returns (O ``[B, S/CP, H, D]``, lse ``[B, H, S/CP]`` fp32)."""
        set_comm_phase("fwd")
        plan, g = self.plan_fwd, self.rank
        B, _, H, D = q.shape
        Hk = k.shape[2]
        dt, dev = q.dtype, q.device
        blk = self.blk
        o = torch.zeros_like(q)
        lse = torch.full((B, H, q.shape[1]), float("-inf"), dtype=torch.float32, device=dev)
        rows: dict = {}      # row id -> dict(q, o, lse, started)
        cols: dict = {}      # col id -> (k, v)
        handles: dict = {}   # kernel -> async handle / event
        pending_merge = []
        for i in self.my_blocks:
            rows[i] = {"q": self._local_block(q, i), "o": self._local_block(o, i),
                       "lse": self._local_block_lse(lse, i), "started": False}
            cols[i] = (self._local_block(k, i), self._local_block(v, i))
        main_ev = None
        if self.cuda:
            main_ev = torch.cuda.Event()
            main_ev.record(torch.cuda.current_stream(dev))
            for st in self.streams:
                st.wait_event(main_ev)

        def deps_of(kern):
            return [handles[p] for p in kern.precursors if p in handles and self.cuda]

        for kern in self._walk_order(plan.gpu_kernel_lists[g]):
            if self.fault is not None and not self.fault.before(kern):
                continue
            if self.cuda:
                torch.cuda.nvtx.range_push(str(kern.key))
            if kern.type == "comm":
                _, _, x, src, dst, io, rc = kern.key
                if io == "i" and rc == "r":
                    if src == g:
                        handles[kern] = self._send(_flat(rows[x]["q"]), kern, 1, deps_of(kern))
                    else:
                        buf = torch.empty(B, blk, H, D, dtype=dt, device=dev)
                        rows[x] = {"q": buf, "o": torch.zeros(B, blk, H, D, dtype=dt, device=dev),
                                   "lse": torch.full((B, H, blk), float("-inf"), dtype=torch.float32, device=dev),
                                   "started": False}
                        handles[kern] = self._recv(buf, kern, 2, deps_of(kern))
                elif io == "i" and rc == "c":
                    if src == g:
                        bundle = torch.stack([cols[x][0], cols[x][1]]).contiguous()
                        handles[kern] = self._send(bundle, kern, 1, deps_of(kern))
                        handles[("keep", kern)] = bundle
                    else:
                        buf = torch.empty(2, B, blk, Hk, D, dtype=dt, device=dev)
                        cols[x] = (buf[0], buf[1])
                        handles[kern] = self._recv(buf, kern, 2, deps_of(kern))
                elif io == "o" and rc == "r":
                    if src == g:     # my partial (O, lse) of a foreign row goes home
                        for p in kern.precursors:
                            self._wait(handles.get(p), f"precursor of {kern.key}")
                        bundle = _pack_bytes([rows[x]["o"], rows[x]["lse"]])
                        handles[kern] = self._send(bundle, kern, 1, deps_of(kern))
                        handles[("keep", kern)] = bundle
                    else:            # I own the row: receive a partial and merge it later
                        buf = torch.empty(_nbytes(_o_lse_specs(B, blk, H, D, dt)), dtype=torch.uint8, device=dev)
                        handles[kern] = self._recv(buf, kern, 2, deps_of(kern))
                        pending_merge.append((kern, x, buf))
                else:
                    raise RuntimeError(f"unexpected forward message {kern.key}")
            else:
                b_, h_, rs, cs, _ = kern.key
                rs = rs if isinstance(rs, tuple) else (rs,)
                cs = cs if isinstance(cs, tuple) else (cs,)
                for p in kern.precursors:
                    self._wait(handles.get(p), f"input of {kern.key}")
                ctx = torch.cuda.stream(self.streams[0]) if self.cuda else _null()
                if self.cuda:
                    for e in deps_of(kern):
                        self.streams[0].wait_event(e)
                with ctx:
                    for r in rs:
                        row = rows[r]
                        k_list = [cols[c][0] for c in cs]
                        v_list = [cols[c][1] for c in cs]
                        segs = [A.Seg(i, 0, blk, self._tile_type(r, c) == CAUSAL, 0)
                                for i, c in enumerate(cs)]
                        work = [A.Row(0, 0, blk, tuple(segs), 0, 0, row["started"])]
                        fplan = A.FwdPlan(work, dev)
                        A.attn_fwd([row["q"]], k_list, v_list, [(row["o"], row["lse"])], fplan, softmax_scale)
                        row["started"] = True
                    if self.cuda:
                        ev = torch.cuda.Event()
                        ev.record(self.streams[0])
                        handles[kern] = ev
            if self.cuda:
                torch.cuda.nvtx.range_pop()

        # receiver-side merge of partial outputs (the "reduce" of the output-row messages)
        for kern, x, buf in pending_merge:
            self._wait(handles.get(kern), f"partial output {kern.key}")
            if self.cuda:
                self.streams[0].wait_event(handles[kern])
            ctx = torch.cuda.stream(self.streams[0]) if self.cuda else _null()
            with ctx:
                po, pl = _unpack_bytes(buf, _o_lse_specs(B, blk, H, D, dt))
                row = rows[x]
                for b in range(B):
                    E.lse_merge([(row["o"][b], row["lse"][b]), (po[b], pl[b])], (row["o"][b], row["lse"][b]))
        for h in list(handles.values()):
            if not isinstance(h, torch.Tensor):
                self._wait(h, "outstanding send")
        if self.cuda:
            cur = torch.cuda.current_stream(dev)
            for st in self.streams:
                ev = torch.cuda.Event()
                ev.record(st)
                cur.wait_event(ev)
            self._keep = handles
        return o, lse

    def _local_block_lse(self, lse: torch.Tensor, blk_id: int) -> torch.Tensor:
        k = self.my_blocks.index(blk_id)
        return lse[:, :, k * self.blk:(k + 1) * self.blk]

    # =============================== backward ===================================================
    def backward(self, d_o, q, k, v, o, lse, softmax_scale=None):
        """Returns (dQ, dK, dV) shards in the dtype of q. ``o`` and ``lse`` are the forward's."""
        set_comm_phase("bwd")
        plan, g = self.plan_bwd, self.rank
        assert plan is not None, "no backward plan was given"
        B, S_loc, H, D = q.shape
        Hk = k.shape[2]
        dt, dev = q.dtype, q.device
        blk = self.blk
        # D = rowsum(dO * O): computed by the owner, travels with the row bundle (O never does)
        dvec = torch.empty(B, H, S_loc, dtype=torch.float32, device=dev)
        for b in range(B):
            E.rowdot(o[b], d_o[b], dvec[b])
        dq_acc = torch.zeros(B, S_loc, H, D, dtype=torch.float32, device=dev)
        dk_acc = torch.zeros(B, S_loc, Hk, D, dtype=torch.float32, device=dev)
        dv_acc = torch.zeros(B, S_loc, Hk, D, dtype=torch.float32, device=dev)
        rows: dict = {}
        cols: dict = {}
        handles: dict = {}
        pending_add = []
        for i in self.my_blocks:
            rows[i] = {"q": self._local_block(q, i), "do": self._local_block(d_o, i),
                       "lse": self._local_block_lse(lse, i), "dvec": self._local_block_lse(dvec, i),
                       "dq": self._local_block(dq_acc, i)}
            cols[i] = {"k": self._local_block(k, i), "v": self._local_block(v, i),
                       "dk": self._local_block(dk_acc, i), "dv": self._local_block(dv_acc, i)}
        if self.cuda:
            main_ev = torch.cuda.Event()
            main_ev.record(torch.cuda.current_stream(dev))
            for st in self.streams:
                st.wait_event(main_ev)

        def deps_of(kern):
            return [handles[p] for p in kern.precursors if p in handles and self.cuda]

        for kern in self._walk_order(plan.gpu_kernel_lists[g]):
            if self.fault is not None and not self.fault.before(kern):
                continue
            if self.cuda:
                torch.cuda.nvtx.range_push(str(kern.key))
            if kern.type == "comm":
                _, _, x, src, dst, io, rc = kern.key
                if io == "i" and rc == "r":
                    if src == g:
                        r = rows[x]
                        bundle = _pack_bytes([r["q"], r["do"], r["lse"], r["dvec"]])
                        handles[kern] = self._send(bundle, kern, 1, deps_of(kern))
                        handles[("keep", kern)] = bundle
                    else:
                        buf = torch.empty(_nbytes(_row_bwd_specs(B, blk, H, D, dt)), dtype=torch.uint8, device=dev)
                        handles[kern] = self._recv(buf, kern, 2, deps_of(kern))
                        rows[x] = {"bundle": buf, "dq": torch.zeros(B, blk, H, D, dtype=torch.float32, device=dev)}
                elif io == "i" and rc == "c":
                    if src == g:
                        bundle = torch.stack([cols[x]["k"], cols[x]["v"]]).contiguous()
                        handles[kern] = self._send(bundle, kern, 1, deps_of(kern))
                        handles[("keep", kern)] = bundle
                    else:
                        buf = torch.empty(2, B, blk, Hk, D, dtype=dt, device=dev)
                        cols[x] = {"k": buf[0], "v": buf[1],
                                   "dk": torch.zeros(B, blk, Hk, D, dtype=torch.float32, device=dev),
                                   "dv": torch.zeros(B, blk, Hk, D, dtype=torch.float32, device=dev)}
                        handles[kern] = self._recv(buf, kern, 2, deps_of(kern))
                elif io == "o":
                    if src == g:
                        for p in kern.precursors:
                            self._wait(handles.get(p), f"precursor of {kern.key}")
                        if rc == "r":
                            bundle = rows[x]["dq"]
                        else:
                            bundle = torch.stack([cols[x]["dk"], cols[x]["dv"]])
                        handles[kern] = self._send(bundle.contiguous(), kern, 1, deps_of(kern))
                        handles[("keep", kern)] = bundle
                    else:
                        shape = (B, blk, H, D) if rc == "r" else (2, B, blk, Hk, D)
                        buf = torch.empty(shape, dtype=torch.float32, device=dev)
                        handles[kern] = self._recv(buf, kern, 2, deps_of(kern))
                        pending_add.append((kern, x, rc, buf))
            else:
                _, _, rs, cs, _ = kern.key
                rs = rs if isinstance(rs, tuple) else (rs,)
                cs = cs if isinstance(cs, tuple) else (cs,)
                for p in kern.precursors:
                    self._wait(handles.get(p), f"input of {kern.key}")
                if self.cuda:
                    for e in deps_of(kern):
                        self.streams[0].wait_event(e)
                ctx = torch.cuda.stream(self.streams[0]) if self.cuda else _null()
                with ctx:
                    sides = []
                    for r in rs:
                        row = rows[r]
                        if "q" not in row:      # unpack a received bundle once
                            qv, dov, lv, dvv = _unpack_bytes(row["bundle"], _row_bwd_specs(B, blk, H, D, dt))
                            row.update({"q": qv, "do": dov, "lse": lv, "dvec": dvv})
                        sides.append(A.BwdQSide(row["q"], row["do"], row["lse"], row["dvec"], row["dq"]))
                    for ci, c in enumerate(cs):
                        col = cols[c]
                        segs = tuple(A.Seg(i, 0, blk, self._tile_type(r, c) == CAUSAL, 0)
                                     for i, r in enumerate(rs))
                        bplan = A.BwdPlan([A.Col(0, 0, blk, segs, 0, 0)], dev)
                        A.attn_bwd(sides, [col["k"]], [col["v"]], [A.BwdKvOut(col["dk"], col["dv"])],
                                   bplan, softmax_scale)
                    if self.cuda:
                        ev = torch.cuda.Event()
                        ev.record(self.streams[0])
                        handles[kern] = ev
            if self.cuda:
                torch.cuda.nvtx.range_pop()

        for kern, x, rc, buf in pending_add:
            self._wait(handles.get(kern), f"partial gradient {kern.key}")
            if self.cuda:
                self.streams[0].wait_event(handles[kern])
            ctx = torch.cuda.stream(self.streams[0]) if self.cuda else _null()
            with ctx:
                if rc == "r":
                    rows[x]["dq"].add_(buf)
                else:
                    cols[x]["dk"].add_(buf[0])
                    cols[x]["dv"].add_(buf[1])
        for h in list(handles.values()):
            if not isinstance(h, torch.Tensor):
                self._wait(h, "outstanding send")
        if self.cuda:
            cur = torch.cuda.current_stream(dev)
            for st in self.streams:
                ev = torch.cuda.Event()
                ev.record(st)
                cur.wait_event(ev)
            self._keep_b = handles
        return dq_acc.to(dt), dk_acc.to(dt), dv_acc.to(dt)


# ------------------------------- bundles ----------------------------------------------------------
class _null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


def _tag(kernel) -> int:
    return kernel.id % 30000


def _flat(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def _pack_bytes(tensors) -> torch.Tensor:
    """Several tensors (any dtypes) as one flat byte buffer: one message moves the whole bundle."""
    return torch.cat([t.contiguous().view(torch.uint8).reshape(-1) for t in tensors])


def _unpack_bytes(buf: torch.Tensor, specs):
    """specs: list of (dtype, shape); returns views into ``buf`` (16-byte aligned offsets)."""
    out, off = [], 0
    for dtype, shape in specs:
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        out.append(buf[off:off + n].view(dtype).view(*shape))
        off += n
    return out


def _nbytes(specs) -> int:
    return sum(int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size() for dtype, shape in specs)


def _o_lse_specs(B, blk, H, D, dt):
    return [(dt, (B, blk, H, D)), (torch.float32, (B, H, blk))]


def _row_bwd_specs(B, blk, H, D, dt):
    return [(dt, (B, blk, H, D)), (dt, (B, blk, H, D)), (torch.float32, (B, H, blk)),
            (torch.float32, (B, H, blk))]
