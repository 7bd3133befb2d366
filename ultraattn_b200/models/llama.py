"""A Llama-2 style decoder built on this framework's kernels, for the end-to-end training step.

The reference has no model, trainer or optimizer: its "end-to-end Llama2-7B" numbers are attention
time times the layer count plus a hard-coded constant for everything else (plot/e2e_pick.py:13-31,
144-177), and its model glue only patches HuggingFace attention modules
(easy_context/zigzag_ring_attn/monkey_patch.py:9-113). This module is the real thing at the same
architecture: RMSNorm -> QKV projection -> RoPE -> block-sparse (optionally context-parallel)
attention -> output projection -> RMSNorm -> SwiGLU FFN, tied together with

  * tcgen05 GEMMs for every projection (forward, dX and dW without transposes),
  * hand-written RMSNorm / RoPE / SwiGLU kernels,
  * attention-aware activation checkpointing: a layer keeps only its input and the attention
    output (O, lse); the backward recomputes the cheap projections but never the attention
    forward (the idea of the reference's CheckpointFunctionEndWithFlashAttention,
    easy_context/dist_flash_attn/monkey_patch.py:78-207),
  * fp32 Adam on a flat master copy, sharded over the context-parallel ranks (ZeRO-1: gradients
    reduce-scattered, parameters all-gathered),
  * a chunked cross-entropy so that the [tokens, vocab] logits never exist at once.

On CPU tensors every op falls back to its fp32 PyTorch restatement, which is how small-shape
parity against a plain PyTorch model is tested without a GPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import api
from ..ops import elementwise as E
from ..ops import gemm as G
from ..patterns.blocks import BSA_Repr


@dataclass
class LlamaConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    vocab: int = 32000
    n_kv_heads: Optional[int] = None
    rope_base: float = 10000.0
    eps: float = 1e-5
    init_std: float = 0.02
    sliding_window: Optional[int] = None     # Mistral: every query sees itself and the sliding_window - 1 tokens before it
    sink_tokens: int = 0                     # with a sliding window: leading tokens that stay visible (streaming)

    @property
    def kv_heads(self) -> int:
        return self.n_kv_heads or self.n_heads

    @classmethod
    def llama2_7b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def mistral_7b(cls) -> "LlamaConfig":
        """Mistral-7B-v0.1: the Llama block with grouped-query attention (8 key/value heads), a
        14336-wide FFN and a 4096-token sliding window."""
        return cls(ffn=14336, n_kv_heads=8, sliding_window=4096)


# ------------------------------- differentiable ops over the kernels -----------------------------
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return G.gemm(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = G.gemm(dy, w, b_is_kn=True)                       # dy[M,N] @ w[N,K]
        dw = G.gemm(dy, x, a_is_km=True, b_is_kn=True)          # dy^T[N,M] @ x[M,K]
        return dx, dw


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        y, rstd = E.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, g):
        x, w, rstd = ctx.saved_tensors
        dx, dw = E.rmsnorm_bwd(x, w, g.contiguous(), rstd)
        return dx, dw.to(w.dtype), None


class _AddRMSNorm(torch.autograd.Function):
    """(x, a) -> (x + a, RMSNorm(x + a) * w) in one kernel; in the backward the gradient that
    reaches x + a through the residual branch is added inside the norm's backward kernel."""

    @staticmethod
    def forward(ctx, x, a, w, eps):
        xsum, y, rstd = E.add_rmsnorm_fwd(x, a.contiguous(), w, eps)
        ctx.save_for_backward(xsum, w, rstd)
        return xsum, y

    @staticmethod
    def backward(ctx, dxsum, dy):
        xsum, w, rstd = ctx.saved_tensors
        dx, dw = E.rmsnorm_bwd(xsum, w, dy.contiguous(), rstd, dres=dxsum.contiguous())
        return dx, dx, dw.to(w.dtype), None


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, pos):
        ctx.save_for_backward(cos, sin, pos)
        return E.rope(x, cos, sin, pos)

    @staticmethod
    def backward(ctx, g):
        cos, sin, pos = ctx.saved_tensors
        return E.rope(g.contiguous(), cos, sin, pos, inverse=True), None, None, None


class _QkvRope(torch.autograd.Function):
    """qkv [T, (H + 2 Hk) * 128] -> q [T, H, 128], k [T, Hk, 128] with rotary embedding applied and
    v [T, Hk, 128]. The split is done by the RoPE kernel itself: it reads the q and k column
    ranges of the projection's output through strided views (no copies, v stays a view), and in
    the backward the inverse rotation writes dq and dk straight into their column ranges of one
    dqkv buffer, next to a single copy of dv."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, pos, n_heads, n_kv_heads):
        T, D = qkv.shape[0], 128
        nq, nk = n_heads * D, n_kv_heads * D
        ctx.save_for_backward(cos, sin, pos)
        ctx.dims = (T, n_heads, n_kv_heads, qkv.dtype)
        q = E.rope(qkv[:, :nq].unflatten(1, (n_heads, D)), cos, sin, pos)
        k = E.rope(qkv[:, nq:nq + nk].unflatten(1, (n_kv_heads, D)), cos, sin, pos)
        v = qkv[:, nq + nk:].unflatten(1, (n_kv_heads, D))
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cos, sin, pos = ctx.saved_tensors
        T, H, Hk, dtype = ctx.dims
        D = 128
        nq, nk = H * D, Hk * D
        dqkv = torch.empty(T, nq + 2 * nk, dtype=dtype, device=dq.device)
        E.rope(dq.contiguous(), cos, sin, pos, inverse=True, out=dqkv[:, :nq].unflatten(1, (H, D)))
        E.rope(dk.contiguous(), cos, sin, pos, inverse=True, out=dqkv[:, nq:nq + nk].unflatten(1, (Hk, D)))
        dqkv[:, nq + nk:].unflatten(1, (Hk, D)).copy_(dv)
        return dqkv, None, None, None, None, None


class _Swiglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return E.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        return E.swiglu_bwd(gu, dy.contiguous())


def _rope_any(x, cos, sin, pos, head_dim):
    """RoPE on [T, H, D]; the kernel handles D = 128, other head dims use the fp32 restatement."""
    if x.is_cuda and head_dim == 128:
        return _Rope.apply(x, cos, sin, pos)
    half = head_dim // 2
    c = cos[pos.long()][:, None, :]
    s = sin[pos.long()][:, None, :]
    lo, hi = x[..., :half].float(), x[..., half:].float()
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1).to(x.dtype)


class _Layer(torch.autograd.Function):
    """One decoder layer with attention-aware checkpointing: the layer input, the attention output
    and its lse are kept (optionally in pinned host memory, reference:
    easy_context/unsloth_offloaded_gradient_checkpoint/monkey_patch.py:20-94), the projections and
    the MLP are recomputed in the backward, the attention forward is not."""

    @staticmethod
    def forward(ctx, x, model, li):
        ctx.model, ctx.li = model, li
        if model.ulysses is not None:
            # head-parallel attention: both all-to-alls live inside the projection GEMMs
            c, p = model.cfg, model.p
            with torch.no_grad():
                h = _RMSNorm.apply(x, p[f"l{li}.norm1"], c.eps)
                cos, sin = model._tables(model.ulysses.S)
                a, o, lse = model.ulysses.forward(h, p[f"l{li}.wqkv"], p[f"l{li}.wo"], cos, sin, return_state=True)
                y = model._seg_ffn(x, li, a)
            ctx.offloaded = None
            ctx.save_for_backward(x, o, lse)
            return y
        with torch.no_grad():
            q, k, v = model._seg_qkv(x, li)
            o, lse = model._attn_fwd(q, k, v)
            y = model._seg_out(x, o, li)
        if model.offload_checkpoints and x.is_cuda:
            ctx.offloaded = (model._offload(x, li, 0), model._offload(o, li, 1))
            ctx.save_for_backward(lse)
        else:
            ctx.offloaded = None
            ctx.save_for_backward(x, o, lse)
        return y

    @staticmethod
    def backward(ctx, dy):
        model, li = ctx.model, ctx.li
        if ctx.offloaded is not None:
            (lse,) = ctx.saved_tensors
            x, o = (model._reload(h) for h in ctx.offloaded)
        else:
            x, o, lse = ctx.saved_tensors
        if model.ulysses is not None:
            c, p, ul = model.cfg, model.p, model.ulysses
            wqkv, wo = p[f"l{li}.wqkv"], p[f"l{li}.wo"]
            cos, sin = model._tables(ul.S)
            with torch.enable_grad():
                x1 = x.detach().requires_grad_()
                h = _RMSNorm.apply(x1, p[f"l{li}.norm1"], c.eps)            # recomputed
                with torch.no_grad():
                    a = ul.recompute_out(o, wo)                              # projection only, attention is NOT recomputed
                a2 = a.requires_grad_()
                x2 = x.detach().requires_grad_()
                y = model._seg_ffn(x2, li, a2)
                torch.autograd.backward([y], [dy])
                with torch.no_grad():
                    dh, dwqkv, dwo = ul.backward(a2.grad, h.detach(), wqkv, wo, o, lse, cos, sin, attn_in_place=True)
                    wqkv.grad.add_(dwqkv)
                    wo.grad.add_(dwo)
                torch.autograd.backward([h], [dh])
            return x1.grad + x2.grad, None, None
        with torch.enable_grad():
            x1 = x.detach().requires_grad_()
            q, k, v = model._seg_qkv(x1, li)                    # recomputed (cheap)
            x2 = x.detach().requires_grad_()
            o2 = o.detach().requires_grad_()
            y = model._seg_out(x2, o2, li)                      # recomputed, attention is NOT
            torch.autograd.backward([y], [dy])
            dq, dk, dv = model._attn_bwd(o2.grad, q.detach(), k.detach(), v.detach(), o, lse)
            torch.autograd.backward([q, k, v], [dq, dk, dv])
        return x1.grad + x2.grad, None, None


class LlamaModel:
    """Parameters live in one flat bf16 buffer (fp32 on CPU) so that the optimizer and the
    gradient collectives work on a single tensor."""

    # ---- activation checkpoints in pinned host memory (optional) --------------------------------
    def _offload(self, t: torch.Tensor, li: int, slot: int):
        """Start copying a checkpoint to its pinned host buffer on the copy stream; returns the
        handle ``_reload`` takes. The device tensor may be freed as soon as the copy has run."""
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=t.device)
        key = (li, slot)
        h = self._host_ckpt.get(key)
        if h is None or h.shape != t.shape or h.dtype != t.dtype:
            h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            self._host_ckpt[key] = h
        cur = torch.cuda.current_stream(t.device)
        self._copy_stream.wait_stream(cur)
        with torch.cuda.stream(self._copy_stream):
            h.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._copy_stream)
        t.record_stream(self._copy_stream)
        return h, ev

    def _reload(self, handle) -> torch.Tensor:
        h, ev = handle
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(ev)
        return h.to(self.device, non_blocking=True)

    def __init__(self, cfg: LlamaConfig, device=None, pattern: Optional[BSA_Repr] = None,
                 runtime=None, group=None, dtype=None, seed: int = 0, lr: float = 1e-4,
                 betas=(0.9, 0.95), weight_decay: float = 0.0, max_pos: int = 1 << 20,
                 offload_checkpoints: bool = False, nvls_optimizer: Optional[bool] = None,
                 seq_algo: str = "cp", seq_len: Optional[int] = None):
        """``seq_algo``: how the sequence is parallelised over ``group``. ``"cp"``: context-parallel
        attention through ``runtime`` (tokens stay sharded inside the attention). ``"ulysses"``:
        head-parallel attention (``parallel/ulysses_fused.py``: the four all-to-alls fused into the
        projection GEMMs); needs ``seq_len`` (whole sequence), every rank then passes the
        contiguous token range ``[rank * S/world, (rank + 1) * S/world)``, and the rows of every
        ``wqkv`` are stored in destination-rank order (``permute_qkv_weight``)."""
        self.cfg = cfg
        if cfg.sliding_window is not None and (runtime is not None or (seq_algo != "halo" and group is not None)):
            raise NotImplementedError("a token-exact sliding window runs on one device or with seq_algo='halo' "
                                      "(contiguous shards); in the planner-driven runtimes express it as a block pattern")
        if seq_algo == "halo":
            assert cfg.sliding_window is not None and not cfg.sink_tokens, \
                "seq_algo='halo' is the strategy of a sliding window (without sink tokens)"
        self.seq_algo = seq_algo
        self.ulysses = None
        self.offload_checkpoints = offload_checkpoints
        self._host_ckpt: dict = {}          # (layer, slot) -> pinned host buffer, reused every step
        self._copy_stream = None
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.pattern = pattern
        self.runtime = runtime          # ContextParallelAttention or None
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.lr, self.betas, self.wd = lr, betas, weight_decay
        self.step_no = 0
        H, D, Hk, Fd, V = cfg.hidden, cfg.head_dim, cfg.kv_heads, cfg.ffn, cfg.vocab
        shapes = [("embed", (V, H))]
        for i in range(cfg.n_layers):
            shapes += [(f"l{i}.norm1", (H,)), (f"l{i}.wqkv", ((cfg.n_heads + 2 * Hk) * D, H)),
                       (f"l{i}.wo", (H, cfg.n_heads * D)), (f"l{i}.norm2", (H,)),
                       (f"l{i}.wgu", (2 * Fd, H)), (f"l{i}.wdown", (H, Fd))]
        shapes += [("norm_f", (H,)), ("lm_head", (V, H))]
        total = sum(math.prod(s) for _, s in shapes)
        pad = (-total) % (8 * max(self.world, 1))
        # Parameters and gradients of a multi-GPU job live in symmetric memory when the machine has
        # NVSwitch multicast: the sharded optimizer then sums the gradients of its shard inside
        # the switch (multimem.ld_reduce) and stores the updated shard into every rank's copy with
        # one multimem.st, instead of NCCL reduce-scatter + all-gather.
        self.space = None
        want_nvls = nvls_optimizer if nvls_optimizer is not None else True
        if want_nvls and self.world > 1 and self.device.type == "cuda" and self.dtype == torch.bfloat16:
            from ..runtime.fused import SymmMemSpace
            sp = SymmMemSpace(group, self.device)
            sp.alloc("params", (total + pad,), self.dtype)
            sp.alloc("grads", (total + pad,), self.dtype)
            sp.finalize()
            if sp.has_multicast():
                self.space = sp
            elif nvls_optimizer:
                raise RuntimeError("nvls_optimizer requested but symmetric memory has no multicast address")
        if self.space is not None:
            self.flat = self.space.local("params")
            self.flat_grad = self.space.local("grads")
            self.flat.zero_()
            self.flat_grad.zero_()
        else:
            self.flat = torch.zeros(total + pad, dtype=self.dtype, device=self.device)
            self.flat_grad = torch.zeros_like(self.flat)
        self.p: dict = {}
        gen = torch.Generator(device=self.device).manual_seed(seed)
        off = 0
        for name, shape in shapes:
            n = math.prod(shape)
            view = self.flat[off:off + n].view(*shape)
            if "norm" in name:
                view.fill_(1.0)
            else:
                chunk = 1 << 26
                fl = view.view(-1)
                for a in range(0, n, chunk):        # generated on the device, bounded temporaries
                    m = min(chunk, n - a)
                    fl[a:a + m] = (torch.randn(m, generator=gen, device=self.device) * cfg.init_std).to(self.dtype)
            view.requires_grad_()
            view.grad = self.flat_grad[off:off + n].view(*shape)
            self.p[name] = view
            off += n
        # optimizer state for this rank's shard
        self.shard = self.flat.numel() // max(self.world, 1)
        sl = slice(self.rank * self.shard, (self.rank + 1) * self.shard)
        self.master = self.flat[sl].detach().float().clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.cos, self.sin = None, None
        self.max_pos = max_pos
        if seq_algo == "ulysses" and self.world > 1:
            from ..parallel.ulysses_fused import FusedUlyssesAttention
            assert seq_len is not None, "seq_algo='ulysses' needs seq_len"
            self.ulysses = FusedUlyssesAttention(group, self.device, seq_len, cfg.hidden, cfg.n_heads, cfg.kv_heads,
                                                 cfg.head_dim, pattern=pattern)
        elif seq_algo not in ("cp", "ulysses", "halo"):
            raise ValueError(f"unknown seq_algo {seq_algo!r}")

    # ------------------------------- segments of a layer ---------------------------------------
    def _tables(self, n_pos: int):
        if self.cos is None or self.cos.shape[0] < n_pos:
            self.cos, self.sin = E.rope_tables(n_pos, self.cfg.head_dim, self.cfg.rope_base, self.device)
        return self.cos, self.sin

    def _seg_qkv(self, x, li):
        c, p = self.cfg, self.p
        h = _RMSNorm.apply(x, p[f"l{li}.norm1"], c.eps)
        qkv = _Linear.apply(h, p[f"l{li}.wqkv"])
        T = x.shape[0]
        nq, nk = c.n_heads * c.head_dim, c.kv_heads * c.head_dim
        if qkv.is_cuda and c.head_dim == 128:
            cos, sin = self._tables(self._n_pos)
            q, k, v = _QkvRope.apply(qkv, cos, sin, self._pos, c.n_heads, c.kv_heads)
            return q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
        q = qkv[:, :nq].reshape(T, c.n_heads, c.head_dim)
        k = qkv[:, nq:nq + nk].reshape(T, c.kv_heads, c.head_dim)
        v = qkv[:, nq + nk:].reshape(T, c.kv_heads, c.head_dim)
        cos, sin = self._tables(self._n_pos)
        q = _rope_any(q.contiguous(), cos, sin, self._pos, c.head_dim)
        k = _rope_any(k.contiguous(), cos, sin, self._pos, c.head_dim)
        return q.unsqueeze(0), k.unsqueeze(0), v.contiguous().unsqueeze(0)

    def _seg_out(self, x, o, li):
        c, p = self.cfg, self.p
        a = _Linear.apply(o.reshape(x.shape[0], c.n_heads * c.head_dim), p[f"l{li}.wo"])
        return self._seg_ffn(x, li, a)

    def _seg_ffn(self, x, li, a=None):
        """Second half of a layer on x (+ a, the attention block's output, added inside the norm
        kernel): x' + W_down(SwiGLU(W_gate,up(RMSNorm(x')))) with x' = x + a."""
        c, p = self.cfg, self.p
        if a is not None:
            x, h = _AddRMSNorm.apply(x, a, p[f"l{li}.norm2"], c.eps)
        else:
            h = _RMSNorm.apply(x, p[f"l{li}.norm2"], c.eps)
        gu = _Linear.apply(h, p[f"l{li}.wgu"])
        return x + _Linear.apply(_Swiglu.apply(gu), p[f"l{li}.wdown"])

    def _window(self):
        w = self.cfg.sliding_window
        return None if w is None else (int(w) - 1, 0)

    def _attn_fwd(self, q, k, v):
        if self._window() is not None:
            if self.world > 1:              # contiguous shards: the window's keys come from the preceding ranks
                from ..parallel.halo import halo_window_attn_forward
                o, lse, _, _ = halo_window_attn_forward(self.group, q.contiguous(), k.contiguous(), v.contiguous(),
                                                        self._window()[0])
                return o, lse
            # token-exact causal band (ops/window.py) on the whole sequence
            from ..ops.window import window_forward
            return window_forward(q, k, v, self._window(), True, sink_tokens=self.cfg.sink_tokens)
        if self.runtime is not None:
            # the fused runtime copies into its symmetric buffers anyway (strided views are fine)
            c = (lambda t: t) if getattr(self.runtime, "path", "") == "fused" else (lambda t: t.contiguous())
            return self.runtime.forward(c(q), c(k), c(v))
        from ..ops import attention as A
        fplan, _ = api.local_plans(self.pattern, q.shape[1], q.device)
        o = torch.empty_like(q)
        lse = torch.empty(1, q.shape[2], q.shape[1], dtype=torch.float32, device=q.device)
        A.attn_fwd([q], [k], [v], [(o, lse)], fplan)
        return o, lse

    def _attn_bwd(self, d_o, q, k, v, o, lse):
        if self._window() is not None:
            if self.world > 1:              # the halo is fetched again (recomputation, like q / k / v themselves)
                from ..parallel.halo import halo_extend, halo_window_attn_backward
                left = self._window()[0]
                k_ext, v_ext, _ = halo_extend(self.group, k.contiguous(), v.contiguous(), left)
                return halo_window_attn_backward(self.group, d_o.contiguous(), q.contiguous(), k_ext, v_ext, o, lse, left)
            from ..ops.window import window_backward
            return window_backward(d_o, q, k, v, o, lse, self._window(), True, sink_tokens=self.cfg.sink_tokens)
        if self.runtime is not None:
            c = (lambda t: t) if getattr(self.runtime, "path", "") == "fused" else (lambda t: t.contiguous())
            return self.runtime.backward(d_o.contiguous(), c(q), c(k), c(v), o, lse)
        _, bplan = api.local_plans(self.pattern, q.shape[1], q.device)
        return api.local_backward(q, k, v, o, lse, d_o.contiguous(), bplan)

    # ------------------------------- forward / loss ---------------------------------------------
    def hidden_states(self, ids: torch.Tensor, pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids [T] (this rank's tokens) -> final normalised hidden states [T, hidden]."""
        T = ids.shape[0]
        self._pos = (pos if pos is not None else torch.arange(T, device=ids.device)).to(torch.int32)
        self._n_pos = int(self._pos.max().item()) + 1 if pos is not None else T
        x = F.embedding(ids, self.p["embed"])
        for li in range(self.cfg.n_layers):
            x = _Layer.apply(x, self, li)
        return _RMSNorm.apply(x, self.p["norm_f"], self.cfg.eps)

    def loss(self, ids, targets, pos=None, chunk: int = 8192, n_total_tokens: Optional[int] = None):
        """Mean next-token cross-entropy over all tokens of the (global) sequence; logits are
        produced and consumed ``chunk`` tokens at a time."""
        h = self.hidden_states(ids, pos)
        n_total = n_total_tokens or ids.shape[0] * self.world
        total = h.new_zeros((), dtype=torch.float32)
        for a in range(0, h.shape[0], chunk):
            total = total + _ChunkLoss.apply(h[a:a + chunk], self.p["lm_head"], targets[a:a + chunk])
        return total / n_total

    # ------------------------------- optimizer --------------------------------------------------
    def optimizer_step(self) -> None:
        self.step_no += 1
        sl = slice(self.rank * self.shard, (self.rank + 1) * self.shard)
        es = self.flat.element_size()
        if self.space is not None:
            # every rank's gradients are complete -> in-switch sum of this rank's shard
            self.space.barrier(0)
            shard_grad = torch.empty(self.shard, dtype=self.dtype, device=self.device)
            E.multimem_reduce(self.space.multicast_ptr("grads") + sl.start * es, shard_grad, self.shard * es,
                              self.dtype, self.device)
        elif self.world > 1:
            shard_grad = torch.empty(self.shard, dtype=self.dtype, device=self.device)
            dist.reduce_scatter_tensor(shard_grad, self.flat_grad, group=self.group)
        else:
            shard_grad = self.flat_grad
        with torch.no_grad():
            E.adam_step(self.master, self.m, self.v, shard_grad, self.flat[sl], self.lr, self.betas[0],
                        self.betas[1], 1e-8, self.wd, self.step_no)
            if self.space is not None:
                # the updated shard goes into every rank's parameter buffer with one multicast store
                E.multimem_bcast_(self.space.multicast_ptr("params") + sl.start * es, self.flat[sl])
                self.space.barrier(1)      # all shards have landed; all ranks have read my gradients
            elif self.world > 1:
                dist.all_gather_into_tensor(self.flat, self.flat[sl].clone(), group=self.group)
            self.flat_grad.zero_()

    def train_step(self, ids, targets, pos=None, n_total_tokens=None) -> float:
        loss = self.loss(ids, targets, pos, n_total_tokens=n_total_tokens)
        loss.backward()
        self.optimizer_step()
        lv = loss.detach()
        if self.world > 1:
            dist.all_reduce(lv, group=self.group)
        return float(lv)


class _ChunkLoss(torch.autograd.Function):
    """Sum of token cross-entropies of one chunk; logits live only inside this function."""

    @staticmethod
    def forward(ctx, h, w, targets):
        lse, rows = E.xent_fwd(G.gemm(h, w), targets)        # one pass over the bf16 logits
        ctx.save_for_backward(h, w, targets, lse)
        return rows.sum()

    @staticmethod
    def backward(ctx, g):
        h, w, targets, lse = ctx.saved_tensors
        dl = E.xent_bwd_(G.gemm(h, w), targets, lse, g)     # logits again, turned into their gradient in place
        dh = G.gemm(dl, w, b_is_kn=True)
        dw = G.gemm(dl, h, a_is_km=True, b_is_kn=True)
        return dh, dw, None


def estimate_memory(cfg: LlamaConfig, seq_len: int, cp: int = 1, offload_checkpoints: bool = False,
                    loss_chunk_tokens: int = 4096, staged_row_tokens: Optional[int] = None,
                    staged_col_tokens: Optional[int] = None) -> dict:
    """Per-GPU memory plan of a training step (GiB), by what holds it: replicated bf16 parameters
    and gradients, the 1/cp shard of the fp32 optimizer state (master, m, v), the activation
    checkpoints (layer input and attention output of every layer, plus lse; in pinned host memory
    with ``offload_checkpoints``), the context-parallel runtime's buffers (symmetric shards of
    Q/K/V/dO, mailboxes, fp32 gradient accumulators, mirrors of the peers it reads from), the
    working set of one layer's backward and one chunk of logits. A planning aid: it tells whether
    a (model, sequence, CP) fits 180 GB before anything is launched."""
    GiB = float(1 << 30)
    H, D, Hk, Fd, V, L = cfg.hidden, cfg.head_dim, cfg.kv_heads, cfg.ffn, cfg.vocab, cfg.n_layers
    per_layer = 2 * H + (cfg.n_heads + 2 * Hk) * D * H + H * cfg.n_heads * D + 2 * Fd * H + H * Fd
    n_params = 2 * V * H + H + L * per_layer
    s_loc = seq_len // cp
    q_bytes = s_loc * cfg.n_heads * D * 2
    kv_bytes = s_loc * Hk * D * 2
    lse_bytes = cfg.n_heads * s_loc * 4
    ckpt_per_layer = s_loc * H * 2 + q_bytes + lse_bytes
    # staging mirrors hold only the foreign blocks a rank's tiles read (``FusedContextParallel.
    # mirror_bytes`` is the exact figure of a plan); default: as many foreign tokens as own ones
    row_tok = s_loc if staged_row_tokens is None else staged_row_tokens
    col_tok = s_loc if staged_col_tokens is None else staged_col_tokens
    runtime = 0.0
    if cp > 1:
        runtime = (2 * q_bytes + 2 * kv_bytes + 2 * lse_bytes           # symmetric q, do, k, v, lse, dvec
                   + q_bytes + lse_bytes                                # mailboxes (one slot per foreign row block: bounded by a shard)
                   + 2 * q_bytes + 2 * 2 * kv_bytes                     # fp32 dq / dk / dv accumulators
                   + row_tok * cfg.n_heads * (D * (2 + 2 + 4) + 8)      # mirrors of foreign rows: q, do, fp32 dq, lse, dvec
                   + col_tok * Hk * D * 4)                              # mirrors of foreign columns: k, v
    layer_work = (s_loc * ((cfg.n_heads + 2 * Hk) * D + 2 * Fd + Fd + 3 * H) * 2) * 2     # activations + their gradients of one layer
    out = {
        "parameters": n_params * 2 / GiB,
        "gradients": n_params * 2 / GiB,
        "optimizer_shard": n_params * 12 / cp / GiB,
        "checkpoints_device": 0.0 if offload_checkpoints else L * ckpt_per_layer / GiB,
        "checkpoints_host": L * ckpt_per_layer / GiB if offload_checkpoints else 0.0,
        "attention_runtime": runtime / GiB,
        "layer_working_set": layer_work / GiB,
        "logits_chunk": loss_chunk_tokens * V * (2 + 4) / GiB,
        "n_params": n_params,
    }
    out["device_total"] = sum(v for k, v in out.items() if k not in ("checkpoints_host", "n_params"))
    return out
