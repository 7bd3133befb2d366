"""Python entry points of the memory-bound kernels (merge, rowdot, casts, RMSNorm, RoPE, SwiGLU,
Adam). CUDA tensors run the sm_100a library; CPU tensors run an fp32 PyTorch restatement that is
also the oracle of the kernel tests."""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from .. import _lib


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


# ---------------------------------------------------------------------------------------------
# online-softmax merge (reference: ring_flash_attn/utils.py:38-52 update_out_and_lse)
# ---------------------------------------------------------------------------------------------
def lse_merge_reference(parts: Sequence[tuple[torch.Tensor, torch.Tensor]]):
    """parts: (O [tokens, heads, D], lse [heads, tokens]) -> merged pair (fp32 math)."""
    lses = torch.stack([l.float() for _, l in parts])                     # [k, H, T]
    tot = torch.logsumexp(lses, dim=0)
    safe = tot.masked_fill(tot == float("-inf"), 0.0)
    w = torch.where(torch.isfinite(lses), torch.exp(lses - safe), torch.zeros_like(lses))
    o = sum(p[0].float() * w[i].t()[..., None] for i, p in enumerate(parts))
    return o, tot


def lse_merge(parts: Sequence[tuple[torch.Tensor, torch.Tensor]], out: tuple[torch.Tensor, torch.Tensor]):
    """Merge k partial (O [tokens, heads, 128] bf16, lse [heads, tokens] fp32) pairs into ``out``
    (which may alias ``parts[0]``)."""
    o_dst, lse_dst = out
    if not o_dst.is_cuda:
        o, l = lse_merge_reference(parts)
        o_dst.copy_(o.to(o_dst.dtype))
        lse_dst.copy_(l)
        return out
    k = len(parts)
    lib = _lib.load()
    vp = ctypes.c_void_p
    o_ptrs = (vp * k)(*[p[0].data_ptr() for p in parts])
    l_ptrs = (vp * k)(*[p[1].data_ptr() for p in parts])
    o_str = (ctypes.c_long * k)(*[p[0].stride(0) for p in parts])
    l_str = (ctypes.c_long * k)(*[p[1].stride(0) for p in parts])
    tokens, heads = o_dst.shape[0], o_dst.shape[1]
    rc = lib.ua_lse_merge(o_ptrs, l_ptrs, o_str, l_str, k, o_dst.data_ptr(), lse_dst.data_ptr(),
                          o_dst.stride(0), lse_dst.stride(0), tokens, heads, _stream(o_dst))
    _lib.check(rc, "ua_lse_merge")
    return out


def rowdot(o: torch.Tensor, d_o: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """D[head, token] = sum_d dO * O for ``[tokens, heads, 128]`` inputs."""
    tokens, heads = o.shape[0], o.shape[1]
    if out is None:
        out = torch.empty(heads, tokens, dtype=torch.float32, device=o.device)
    if not o.is_cuda:
        out.copy_((o.float() * d_o.float()).sum(-1).t())
        return out
    rc = _lib.load().ua_rowdot(o.data_ptr(), d_o.data_ptr(), out.data_ptr(), o.stride(0),
                               d_o.stride(0), out.stride(0), tokens, heads, _stream(o))
    _lib.check(rc, "ua_rowdot")
    return out


def cast_scale(src: torch.Tensor, dst: torch.Tensor, scale: float = 1.0, accumulate: bool = False):
    """dst(bf16) (+)= scale * src(fp32); both contiguous."""
    if not src.is_cuda:
        v = src.float() * scale
        dst.copy_((dst.float() + v if accumulate else v).to(dst.dtype))
        return dst
    rc = _lib.load().ua_cast_scale(src.data_ptr(), dst.data_ptr(), src.numel(), scale,
                                   int(accumulate), _stream(src))
    _lib.check(rc, "ua_cast_scale")
    return dst


# ---------------------------------------------------------------------------------------------
# model-side ops
# ---------------------------------------------------------------------------------------------
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5):
    """x [rows, H] -> (y, rstd)."""
    rows, H = x.shape
    if not x.is_cuda:
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        return (xf * rstd[:, None] * w.float()).to(x.dtype), rstd
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = _lib.load().ua_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows,
                                    H, eps, _stream(x))
    _lib.check(rc, "ua_rmsnorm_fwd")
    return y, rstd


def add_rmsnorm_fwd(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor, eps: float = 1e-5):
    """xsum = x + res and y = RMSNorm(xsum) * w in one pass -> (xsum, y, rstd)."""
    rows, H = x.shape
    if not x.is_cuda:
        xsum = (x.float() + res.float()).to(x.dtype)
        y, rstd = rmsnorm_fwd(xsum, w, eps)
        return xsum, y, rstd
    xsum, y = torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = _lib.load().ua_add_rmsnorm_fwd(x.data_ptr(), res.data_ptr(), w.data_ptr(), xsum.data_ptr(),
                                        y.data_ptr(), rstd.data_ptr(), rows, H, eps, _stream(x))
    _lib.check(rc, "ua_add_rmsnorm_fwd")
    return xsum, y, rstd


def rmsnorm_bwd(x, w, g, rstd, dres=None):
    """-> (dx [rows, H] like x, dw fp32 [H]). ``dres``: a gradient added to dx in the same pass
    (what reaches x through a residual branch next to the norm)."""
    rows, H = x.shape
    if not x.is_cuda:
        xf, gf, wf = x.float(), g.float(), w.float()
        gw = gf * wf
        c = (gw * xf).sum(-1, keepdim=True) * (rstd[:, None] ** 2) / H
        dx = rstd[:, None] * (gw - xf * c)
        if dres is not None:
            dx = dx + dres.float()
        dw = (gf * xf * rstd[:, None]).sum(0)
        return dx.to(x.dtype), dw
    dx = torch.empty_like(x)
    dw = torch.zeros(H, dtype=torch.float32, device=x.device)
    if dres is None:
        rc = _lib.load().ua_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), g.data_ptr(), rstd.data_ptr(),
                                        dx.data_ptr(), dw.data_ptr(), rows, H, _stream(x))
    else:
        rc = _lib.load().ua_rmsnorm_bwd_res(x.data_ptr(), w.data_ptr(), g.data_ptr(), rstd.data_ptr(),
                                            dres.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, H, _stream(x))
    _lib.check(rc, "ua_rmsnorm_bwd")
    return dx, dw


def rope_tables(max_pos: int, dim: int = 128, base: float = 10000.0, device="cpu"):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor,
         inverse: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate-half rotary embedding on ``x [tokens, heads, 128]`` (heads contiguous per token);
    ``pos`` int32 [tokens] selects the table row per token. ``inverse`` applies the transpose
    rotation (the backward)."""
    if out is None:
        out = torch.empty_like(x)
    if not x.is_cuda:
        c = cos[pos.long()][:, None, :]
        s = sin[pos.long()][:, None, :]
        if inverse:
            s = -s
        lo, hi = x[..., :64].float(), x[..., 64:].float()
        out.copy_(torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1).to(x.dtype))
        return out
    assert x.stride(2) == 1 and x.stride(1) == 128 and out.stride(1) == 128
    rc = _lib.load().ua_rope(x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                             pos.data_ptr(), x.shape[0], x.shape[1], x.stride(0), out.stride(0),
                             int(inverse), _stream(x))
    _lib.check(rc, "ua_rope")
    return out


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    """gu [rows, 2F] (gate | up) -> silu(gate) * up [rows, F]."""
    rows, F2 = gu.shape
    F = F2 // 2
    if not gu.is_cuda:
        g, u = gu[:, :F].float(), gu[:, F:].float()
        return (torch.nn.functional.silu(g) * u).to(gu.dtype)
    y = torch.empty(rows, F, dtype=gu.dtype, device=gu.device)
    rc = _lib.load().ua_swiglu_fwd(gu.data_ptr(), y.data_ptr(), rows, F, _stream(gu))
    _lib.check(rc, "ua_swiglu_fwd")
    return y


def swiglu_bwd(gu: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    rows, F2 = gu.shape
    F = F2 // 2
    if not gu.is_cuda:
        g, u, d = gu[:, :F].float(), gu[:, F:].float(), dy.float()
        sig = torch.sigmoid(g)
        dg = d * u * sig * (1 + g * (1 - sig))
        du = d * g * sig
        return torch.cat([dg, du], dim=1).to(gu.dtype)
    dgu = torch.empty_like(gu)
    rc = _lib.load().ua_swiglu_bwd(gu.data_ptr(), dy.data_ptr(), dgu.data_ptr(), rows, F, _stream(gu))
    _lib.check(rc, "ua_swiglu_bwd")
    return dgu


def adam_step(master, m, v, grad, param, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    """Fused Adam(W) on flat fp32 state with a bf16 gradient; rewrites the bf16 ``param``."""
    if not master.is_cuda:
        g = grad.float() * grad_scale
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        upd = (m / bc1) / ((v / bc2).sqrt() + eps)
        master.sub_(lr * (upd + wd * master))
        param.copy_(master.to(param.dtype))
        return
    rc = _lib.load().ua_adam(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(),
                             param.data_ptr(), master.numel(), lr, beta1, beta2, eps, wd, step,
                             grad_scale, _stream(master))
    _lib.check(rc, "ua_adam")


def xent_fwd(logits: torch.Tensor, targets: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Token cross-entropy over ``logits [T, V]``: (lse [T], loss [T]) in fp32, loss =
    lse - logit[target] (0 where the target is outside ``[0, V)``). bf16 logits on CUDA are read
    once by this framework's kernel; anything else runs in PyTorch."""
    T, V = logits.shape
    if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(1) == 1:
        tg = targets.to(torch.int32).contiguous()
        lse = torch.empty(T, dtype=torch.float32, device=logits.device)
        loss = torch.empty(T, dtype=torch.float32, device=logits.device)
        rc = _lib.load().ua_xent_fwd(logits.data_ptr(), tg.data_ptr(), lse.data_ptr(), loss.data_ptr(), T,
                                     logits.stride(0), V, _stream(logits))
        _lib.check(rc, "ua_xent_fwd")
        return lse, loss
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    ok = (targets >= 0) & (targets < V)
    picked = lf.gather(1, targets.clamp(0, V - 1)[:, None].long()).squeeze(1)
    return lse, torch.where(ok, lse - picked, torch.zeros_like(lse))


def xent_bwd_(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """In place: ``logits`` becomes ``g * (softmax(logits) - one_hot(targets))`` (``g``: scalar
    tensor, the gradient of the summed loss); rows with a target outside ``[0, V)`` become zero.
    Returns ``logits``."""
    T, V = logits.shape
    if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(1) == 1:
        tg = targets.to(torch.int32).contiguous()
        gs = g.detach().to(torch.float32).reshape(1).contiguous()
        rc = _lib.load().ua_xent_bwd(logits.data_ptr(), tg.data_ptr(), lse.data_ptr(), gs.data_ptr(), T,
                                     logits.stride(0), V, _stream(logits))
        _lib.check(rc, "ua_xent_bwd")
        return logits
    p = torch.exp(logits.float() - lse[:, None])
    ok = (targets >= 0) & (targets < V)
    p.scatter_add_(1, targets.clamp(0, V - 1)[:, None].long(), -torch.ones_like(lse)[:, None])
    logits.copy_((p * g.float() * ok[:, None]).to(logits.dtype))
    return logits


def peer_add_(dst: torch.Tensor, src: torch.Tensor, zero_src: bool = False) -> None:
    """dst += src for contiguous fp32 tensors; ``dst`` may be a view of a peer GPU's memory
    (this framework's own kernel does the adds — library kernels never touch peer memory)."""
    assert dst.dtype == torch.float32 and src.dtype == torch.float32
    assert dst.is_contiguous() and src.is_contiguous() and dst.numel() == src.numel()
    if not dst.is_cuda:
        dst.add_(src)
        if zero_src:
            src.zero_()
        return
    sms = torch.cuda.get_device_properties(src.device).multi_processor_count
    rc = _lib.load().ua_peer_add_f32(dst.data_ptr(), src.data_ptr(), src.numel(), int(zero_src), sms,
                                     _stream(src))
    _lib.check(rc, "ua_peer_add_f32")


def peer_pull_(dst: torch.Tensor, src: torch.Tensor, n_ctas: int = 0) -> None:
    """dst = src for contiguous tensors of equal byte size (a multiple of 16); ``src`` is usually a
    view of a peer GPU's memory, read with plain peer loads by this framework's copy kernel
    (``n_ctas`` CTAs, default one per SM)."""
    assert dst.is_contiguous() and src.is_contiguous()
    nbytes = dst.numel() * dst.element_size()
    assert nbytes == src.numel() * src.element_size()
    if not dst.is_cuda:
        dst.view(torch.uint8).copy_(src.view(torch.uint8))
        return
    n = n_ctas or torch.cuda.get_device_properties(dst.device).multi_processor_count
    rc = _lib.load().ua_peer_pull(dst.data_ptr(), src.data_ptr(), nbytes, n, _stream(dst))
    _lib.check(rc, "ua_peer_pull")


def multimem_bcast_(mc_ptr: int, src: torch.Tensor) -> None:
    """Store ``src`` (contiguous, size a multiple of 16 bytes) into every rank's replica of a
    symmetric buffer through its NVSwitch multicast address ``mc_ptr`` (``multimem.st``): the
    bytes leave this GPU once however many ranks receive them. The caller orders it against the
    readers with the device barrier."""
    assert src.is_cuda and src.is_contiguous()
    sms = torch.cuda.get_device_properties(src.device).multi_processor_count
    rc = _lib.load().ua_multimem_bcast(mc_ptr, src.data_ptr(), src.numel() * src.element_size(), sms,
                                       _stream(src))
    _lib.check(rc, "ua_multimem_bcast")


def multimem_reduce(mc_ptr: int, dst, nbytes: int, dtype: torch.dtype, device,
                    mc_out: int = 0) -> None:
    """Sum the replicas of a symmetric buffer inside the switch (``multimem.ld_reduce``): the sum of
    ``nbytes`` at multicast address ``mc_ptr`` goes to the local tensor ``dst`` (or nowhere when
    None) and, when ``mc_out`` is given, back into every replica at that multicast address (ranks
    covering disjoint slices with ``mc_out == mc_ptr`` make a one-shot all-reduce). fp32 or bf16
    (bf16 accumulates in fp32)."""
    assert dtype in (torch.float32, torch.bfloat16)
    if dst is not None:
        assert dst.is_contiguous() and dst.dtype == dtype and dst.numel() * dst.element_size() == nbytes
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    rc = _lib.load().ua_multimem_reduce(dst.data_ptr() if dst is not None else 0, mc_ptr, mc_out, nbytes,
                                        int(dtype == torch.bfloat16), sms,
                                        torch.cuda.current_stream(device).cuda_stream)
    _lib.check(rc, "ua_multimem_reduce")
