"""Single-device attention whose forward and backward replay from CUDA graphs.

A step with small tiles is bound by the host: every launch crosses ctypes, looks its tensor maps
up and enqueues one kernel (25-40 us; a 2k x 2k tile computes in less). The kernels themselves
take all of their tables from device memory and their tensor maps as launch parameters, so a
fixed (pattern, shape) step can be captured once and replayed with one host call per pass. This
module makes that a runtime mode instead of a recipe: :class:`GraphedAttention` owns static input
and output buffers, captures one graph for the forward and one for the backward (D = rowsum(dO o O),
clearing of the fp32 dQ accumulator, the backward kernel, the cast), and exposes the differentiable
call. On CPU (no graphs there) it runs the same steps eagerly, which keeps the bookkeeping testable.

The reference checks that its flash-attention call can be captured (tests/test_cuda_graph.py:48-164)
and its communicator takes explicit streams for the same purpose; it has no replay mode of its own.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..api import local_plans
from ..ops import attention as A
from ..ops import elementwise as E
from ..patterns.blocks import BSA_Repr


class GraphedAttention:
    """``o = attention(q, k, v, pattern)`` for one fixed shape, replayed from CUDA graphs.

    ``inputs()`` hands out the static q / k / v / dO buffers: a caller that writes its tensors
    there (e.g. as the ``out=`` of the producing kernel) pays no copy; ``forward(q, k, v)`` and
    ``backward(d_o)`` copy their arguments in unless they already are those buffers. Results are
    views of static buffers, valid until the next call of the same pass."""

    def __init__(self, pattern: BSA_Repr, seq_len: int, n_heads: int, head_dim: int = 128,
                 n_kv_heads: Optional[int] = None, batch: int = 1, device="cuda",
                 dtype: torch.dtype = torch.bfloat16, softmax_scale: Optional[float] = None):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        hk = n_kv_heads or n_heads
        self.scale = softmax_scale
        self.fplan, self.bplan = local_plans(pattern, seq_len, self.device)
        new = lambda *shape, dt=dtype: torch.zeros(*shape, dtype=dt, device=self.device)
        B, S, H, D = batch, seq_len, n_heads, head_dim
        self.q, self.d_o, self.o = new(B, S, H, D), new(B, S, H, D), new(B, S, H, D)
        self.k, self.v = new(B, S, hk, D), new(B, S, hk, D)
        self.lse, self.dvec = new(B, H, S, dt=torch.float32), new(B, H, S, dt=torch.float32)
        self.dq32 = new(B, S, H, D, dt=torch.float32)
        grad_dt = dtype if self.cuda else torch.float32
        self.dq = new(B, S, H, D)
        self.dk, self.dv = new(B, S, hk, D, dt=grad_dt), new(B, S, hk, D, dt=grad_dt)
        self.replays = {"fwd": 0, "bwd": 0}
        self._graphs: dict = {}
        if self.cuda:
            self._capture()

    # ---- the two passes, as they are captured ---------------------------------------------------
    def _fwd_step(self) -> None:
        A.attn_fwd([self.q], [self.k], [self.v], [(self.o, self.lse)], self.fplan, self.scale)

    def _bwd_step(self) -> None:
        for b in range(self.q.shape[0]):
            E.rowdot(self.o[b], self.d_o[b], self.dvec[b])
        self.dq32.zero_()
        if not self.cuda:               # the CPU restatement adds into dK / dV, the kernel overwrites them
            self.dk.zero_()
            self.dv.zero_()
        A.attn_bwd([A.BwdQSide(self.q, self.d_o, self.lse, self.dvec, self.dq32)], [self.k], [self.v],
                   [A.BwdKvOut(self.dk, self.dv)], self.bplan, self.scale)
        if self.cuda:
            E.cast_scale(self.dq32, self.dq)
        else:
            self.dq.copy_(self.dq32)

    def _capture(self) -> None:
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            # one eager run first: library load, shared-memory attributes of the kernels, and the
            # tensor maps of these buffers enter the host-side cache outside the capture
            self._fwd_step()
            self._bwd_step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        for name, step in (("fwd", self._fwd_step), ("bwd", self._bwd_step)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                step()
            self._graphs[name] = g

    # ---- public ---------------------------------------------------------------------------------
    def inputs(self) -> dict:
        return {"q": self.q, "k": self.k, "v": self.v, "d_o": self.d_o}

    @staticmethod
    def _fill(dst: torch.Tensor, src: torch.Tensor) -> None:
        if src.data_ptr() != dst.data_ptr():
            assert src.shape == dst.shape, f"graphed attention was built for {tuple(dst.shape)}, got {tuple(src.shape)}"
            dst.copy_(src)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        """Returns (o, lse): views of static buffers."""
        self._fill(self.q, q), self._fill(self.k, k), self._fill(self.v, v)
        if self.cuda:
            self._graphs["fwd"].replay()
        else:
            self._fwd_step()
        self.replays["fwd"] += 1
        return self.o, self.lse

    def backward(self, d_o: torch.Tensor):
        """Gradients of the last :meth:`forward` (whose inputs and outputs still sit in the static
        buffers): (dq, dk, dv), views of static buffers."""
        self._fill(self.d_o, d_o)
        if self.cuda:
            self._graphs["bwd"].replay()
        else:
            self._bwd_step()
        self.replays["bwd"] += 1
        return self.dq, self.dk, self.dv

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """Differentiable form. The output is a copy (autograd keeps it), the gradients are copies
        too; between this call and its backward no other call of this object may run."""
        return _GraphedFunction.apply(q, k, v, self)


class _GraphedFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, runner: GraphedAttention):
        o, _ = runner.forward(q, k, v)
        ctx.runner = runner
        ctx.serial = runner.replays["fwd"]
        return o.clone()

    @staticmethod
    def backward(ctx, d_o):
        r = ctx.runner
        if r.replays["fwd"] != ctx.serial:
            raise RuntimeError("GraphedAttention: another forward ran before this call's backward; "
                               "its static buffers no longer hold this call's inputs")
        dq, dk, dv = r.backward(d_o.contiguous())
        return dq.clone(), dk.to(d_o.dtype).clone(), dv.to(d_o.dtype).clone(), None
