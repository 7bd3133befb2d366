"""Head-parallel (Ulysses) attention with all four all-to-alls fused into the projection GEMMs.

Unfused (reference: head_parallel_attn/deepspeed_ulysses_attn.py:10-198, comm_lib/comm_utils.py:32-45):
    qkv = x @ Wqkv^T            ->  all-to-all (sequence shard -> head shard)  ->  attention
    attention                   ->  all-to-all (head shard -> sequence shard)  ->  y = o @ Wo^T
    and the mirror image in the backward (dO to head shards, dQ/dK/dV back to sequence shards).
Fused (this module), forward:
    the QKV GEMM's epilogue stores every head group's output tile directly into the receive
    buffer of the rank that owns those heads (peer stores over NVLink, ``gemm_scatter``);
    the output projection's TMA producer loads its A operand K-group by K-group, one group per
    owning rank (``gemm_gather``).
Backward, through the same two fusions:
    dO of every head group:  dy @ Wo  with the scatter epilogue (rank g receives its heads' dO for
    all tokens);  block-sparse attention backward on the local heads over the whole sequence;
    dx = dQKV @ Wqkv  with the gather prologue (this rank's tokens of every head group).  The
    weight gradients are per-group GEMMs on the same gathered operands (dWo: O of head group g,
    dWqkv: dQKV of group g).
No all-to-all kernel exists on this path.

Where the gathered operand comes from (``gather="staged"``, default): a GEMM reads its A operand
once per tile column, i.e. N / 256 times, and peer memory is not cached in the reader's L2, so a
gather prologue that points TMA at the owners' buffers sends every byte over NVLink 16 times for a
4096-wide output (measured on 8 GPUs, S = 256k: the block took 345 ms against 256 ms for the
all-to-all form). So this rank's token rows of every peer's buffer are first pulled ONCE into a
local staging buffer by this framework's copy kernel (plain peer loads, all SMs, about 640 GB/s)
and the gather prologue and the weight-gradient GEMMs read the local copy. ``gather="peer"`` keeps
the direct form (unicast TMA over the peer mappings), which is the right one when the output is
narrow (one tile column).

Weights: ``wqkv`` rows must be ordered by destination rank — for rank g the rows
``[q heads of g | k heads of g | v heads of g]`` — :func:`permute_qkv_weight` produces that order
from the usual ``[q | k | v]`` layout (:func:`unpermute_qkv_weight` is its inverse).
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from ..ops import attention as A
from ..ops import elementwise as E
from ..ops import gemm as G
from ..runtime.fused import SymmMemSpace


def permute_qkv_weight(wqkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, sp: int) -> torch.Tensor:
    """[q | k | v] rows -> for every rank g: [q_g | k_g | v_g]."""
    nq, nk = n_heads * head_dim, n_kv_heads * head_dim
    q, k, v = wqkv[:nq], wqkv[nq:nq + nk], wqkv[nq + nk:]
    hq, hk = n_heads // sp * head_dim, n_kv_heads // sp * head_dim
    parts = []
    for g in range(sp):
        parts += [q[g * hq:(g + 1) * hq], k[g * hk:(g + 1) * hk], v[g * hk:(g + 1) * hk]]
    return torch.cat(parts, dim=0).contiguous()


def unpermute_qkv_weight(wperm: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, sp: int) -> torch.Tensor:
    """Inverse of :func:`permute_qkv_weight`: per-rank ``[q_g | k_g | v_g]`` rows -> ``[q | k | v]``."""
    hq, hk = n_heads // sp * head_dim, n_kv_heads // sp * head_dim
    per = hq + 2 * hk
    qs, ks, vs = [], [], []
    for g in range(sp):
        blk = wperm[g * per:(g + 1) * per]
        qs.append(blk[:hq])
        ks.append(blk[hq:hq + hk])
        vs.append(blk[hq + hk:])
    return torch.cat(qs + ks + vs, dim=0).contiguous()


class FusedUlyssesAttention:
    """One attention block (QKV projection, RoPE, attention, output projection) over a sequence
    that is sharded by tokens outside and by heads inside. ``pattern``: any block pattern of the
    framework (default dense causal); rank r holds the tokens ``[r * S/sp, (r + 1) * S/sp)``."""

    def __init__(self, group, device, seq_len: int, hidden: int, n_heads: int, n_kv_heads: int = None,
                 head_dim: int = 128, causal: bool = True, pattern=None, gather: str = "staged"):
        self.group, self.device = group, device
        self.sp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.S, self.S_loc = seq_len, seq_len // self.sp
        self.H, self.Hk, self.D = n_heads, n_kv_heads or n_heads, head_dim
        assert self.H % self.sp == 0 and self.Hk % self.sp == 0, "heads must divide over the ranks"
        self.hq, self.hk = self.H // self.sp, self.Hk // self.sp
        self.cols = (self.hq + 2 * self.hk) * head_dim
        self.hidden = hidden
        self.causal = causal
        self.space = SymmMemSpace(group, device)
        self.space.alloc("qkv", (seq_len, self.cols), torch.bfloat16)
        self.space.alloc("attn", (seq_len, self.hq * head_dim), torch.bfloat16)
        self.space.alloc("dattn", (seq_len, self.hq * head_dim), torch.bfloat16)
        self.space.alloc("dqkv", (seq_len, self.cols), torch.bfloat16)
        self.space.finalize()
        assert gather in ("staged", "peer")
        self.gather = gather
        # this rank's token rows of every peer's buffer, pulled once per use (attn: the first
        # hq * D columns of a slot; dqkv: all of it)
        self.stage = (torch.empty(self.sp, self.S_loc, self.cols, dtype=torch.bfloat16, device=device)
                      if gather == "staged" and self.sp > 1 else None)
        from ..api import local_plans
        from ..patterns import named
        if pattern is None:
            pattern = named.causal(1) if causal else named.full(1)
        self.pattern = pattern
        self.fplan, self.bplan = local_plans(pattern, seq_len, device)
        # NVLink bytes this rank moves per call (scatter epilogues; gathers), for reports. Staged
        # gathers move every byte once; the direct form re-reads a gathered operand once per tile
        # column of the GEMM that consumes it (hidden / 256 for the projections).
        es, peers = 2, self.sp - 1
        attn_b, qkv_b = self.S_loc * self.hq * head_dim * peers * es, self.S_loc * self.cols * peers * es
        rereads = 1 if gather == "staged" else max(1, hidden // 256)
        self.traffic = {
            "gather_form": gather,
            "fwd_scatter_bytes": qkv_b,
            "fwd_gather_bytes": attn_b * rereads,
            "bwd_scatter_bytes": qkv_b + attn_b,                       # q/k/v again, dO
            "bwd_gather_bytes": (attn_b + qkv_b) * (1 if gather == "staged" else rereads + 1),
        }

    # ------------------------------------------------------------------------------------------
    def _gathered(self, name: str, width: int):
        """This rank's rows ``[r0, r0 + S/sp)`` of buffer ``name`` on every rank, as a list of
        ``[S/sp, width]`` tensors (one per owner). Staged form: remote ones are pulled into the
        local staging buffer (one pass over NVLink); the own one is a view of the local buffer."""
        sp, r0 = self.space, self.rank * self.S_loc
        out = []
        for g in range(self.sp):
            src = sp.peer(name, g)[r0:r0 + self.S_loc]
            if g == self.rank or self.stage is None:
                out.append(src)
                continue
            dst = self.stage[g].view(-1)[:self.S_loc * width].view(self.S_loc, width)
            E.peer_pull_(dst, src)
            out.append(dst)
        return out

    def _project_qkv(self, x, wqkv_perm, cos, sin):
        """x [S/sp, hidden] -> this rank's head group of q, k, v for all tokens (views of the
        symmetric receive buffer), RoPE applied."""
        sp, D = self.space, self.D
        sp.barrier(4)                       # everyone is done reading the buffers of the last call
        dst = [sp.peer("qkv", r).data_ptr() for r in range(self.sp)]
        G.gemm_scatter(x, wqkv_perm, dst, self.cols, self.rank * self.S_loc)
        sp.barrier(5)                       # all head groups of all tokens have arrived
        buf = sp.local("qkv")
        nq, nk = self.hq * D, self.hk * D
        q = buf[:, :nq].unflatten(1, (self.hq, D))
        k = buf[:, nq:nq + nk].unflatten(1, (self.hk, D))
        v = buf[:, nq + nk:].unflatten(1, (self.hk, D))
        if cos is not None:
            pos = torch.arange(self.S, device=self.device, dtype=torch.int32)
            E.rope(q, cos, sin, pos, out=q)
            E.rope(k, cos, sin, pos, out=k)
        return q, k, v

    def _project_out(self, wo):
        """y [S/sp, hidden] = attention outputs of this rank's tokens (all head groups, read from
        their owners) @ Wo^T."""
        y = torch.empty(self.S_loc, wo.shape[0], dtype=torch.bfloat16, device=self.device)
        hqD = self.hq * self.D
        parts = self._gathered("attn", hqD)
        G.gemm_gather([t.data_ptr() for t in parts], self.S_loc, hqD, 0, self.S_loc, hqD, wo, y)
        return y

    def forward(self, x: torch.Tensor, wqkv_perm: torch.Tensor, wo: torch.Tensor, cos=None, sin=None,
                softmax_scale=None, return_state: bool = False):
        """x [S/sp, hidden] (this rank's tokens) -> y [S/sp, hidden]. With ``return_state`` also
        the attention output of the local heads ``[S, hq, D]`` (a copy) and its lse, which
        :meth:`backward` needs."""
        sp, D = self.space, self.D
        q, k, v = self._project_qkv(x, wqkv_perm, cos, sin)
        o = sp.local("attn").view(1, self.S, self.hq, D)
        lse = torch.empty(1, self.hq, self.S, dtype=torch.float32, device=self.device)
        A.attn_fwd([q.unsqueeze(0)], [k.unsqueeze(0)], [v.unsqueeze(0)], [(o, lse)], self.fplan, softmax_scale)
        sp.barrier(6)                       # every rank's attention output is complete
        y = self._project_out(wo)
        if return_state:
            return y, o[0].clone(), lse
        return y

    def recompute_out(self, o_saved: torch.Tensor, wo: torch.Tensor) -> torch.Tensor:
        """The block's output again from a saved attention output (activation checkpointing: the
        attention itself is not recomputed)."""
        sp = self.space
        sp.barrier(4)
        sp.local("attn").view(self.S, self.hq, self.D).copy_(o_saved)
        sp.barrier(6)
        return self._project_out(wo)

    def backward(self, dy: torch.Tensor, x: torch.Tensor, wqkv_perm: torch.Tensor, wo: torch.Tensor,
                 o_saved: torch.Tensor, lse: torch.Tensor, cos=None, sin=None, softmax_scale=None,
                 attn_in_place: bool = False):
        """Gradients of the block: (dx [S/sp, hidden], dWqkv_perm, dWo). ``o_saved`` / ``lse``:
        the state returned by ``forward(..., return_state=True)``. ``attn_in_place``: the
        symmetric attention buffer still holds ``o_saved`` on every rank (as right after
        :meth:`recompute_out`), so it is not copied in again."""
        sp, D, S, S_loc = self.space, self.D, self.S, self.S_loc
        r0 = self.rank * S_loc
        hqD = self.hq * D
        dy = dy.contiguous()
        # q, k, v of the local heads again (projection + scatter; cheap next to the attention)
        q, k, v = self._project_qkv(x, wqkv_perm, cos, sin)
        if not attn_in_place:
            sp.local("attn").view(S, self.hq, D).copy_(o_saved)
        # dO of every head group: dy @ Wo, group g's columns stored into rank g's buffer
        dst = [sp.peer("dattn", r).data_ptr() for r in range(self.sp)]
        G.gemm_scatter(dy, wo, dst, hqD, r0, b_is_kn=True)
        sp.barrier(7)                       # dO of my heads has arrived from every rank; O is in place everywhere
        # dWo[:, heads of g] = dy^T @ O_g[my tokens]
        dwo = torch.empty(wo.shape, dtype=torch.bfloat16, device=self.device)
        for g, o_g in enumerate(self._gathered("attn", hqD)):
            G.gemm(dy, o_g, a_is_km=True, b_is_kn=True, out=dwo[:, g * hqD:(g + 1) * hqD])
        # attention backward on the local heads over the whole sequence
        d_o = sp.local("dattn").view(1, S, self.hq, D)
        o = sp.local("attn").view(1, S, self.hq, D)
        dvec = torch.empty(1, self.hq, S, dtype=torch.float32, device=self.device)
        E.rowdot(o[0], d_o[0], dvec[0])
        dq32 = torch.zeros(1, S, self.hq, D, dtype=torch.float32, device=self.device)
        dbuf = sp.local("dqkv")
        nq, nk = hqD, self.hk * D
        dq = dbuf[:, :nq].unflatten(1, (self.hq, D))
        dk = dbuf[:, nq:nq + nk].unflatten(1, (self.hk, D))
        dv = dbuf[:, nq + nk:].unflatten(1, (self.hk, D))
        A.attn_bwd([A.BwdQSide(q.unsqueeze(0), d_o, lse, dvec, dq32)], [k.unsqueeze(0)], [v.unsqueeze(0)],
                   [A.BwdKvOut(dk.unsqueeze(0), dv.unsqueeze(0))], self.bplan, softmax_scale)
        dq_c = torch.empty(S, self.hq, D, dtype=torch.bfloat16, device=self.device)
        E.cast_scale(dq32, dq_c)
        del dq32
        if cos is not None:
            pos = torch.arange(S, device=self.device, dtype=torch.int32)
            E.rope(dq_c, cos, sin, pos, inverse=True, out=dq)       # straight into the symmetric buffer
            E.rope(dk, cos, sin, pos, inverse=True, out=dk)
        else:
            dq.copy_(dq_c)
        sp.barrier(8)                       # every rank's dQ / dK / dV of its heads is complete
        # dx = dQKV[my tokens, every head group] @ Wqkv_perm   (A gathered from the owners)
        dx = torch.empty(S_loc, self.hidden, dtype=torch.bfloat16, device=self.device)
        parts = self._gathered("dqkv", self.cols)
        G.gemm_gather([t.data_ptr() for t in parts], S_loc, self.cols, 0, S_loc, self.cols, wqkv_perm, dx,
                      b_is_kn=True)
        # dWqkv_perm[rows of g] = dQKV_g[my tokens]^T @ x
        dwqkv = torch.empty(wqkv_perm.shape, dtype=torch.bfloat16, device=self.device)
        for g, d_g in enumerate(parts):
            G.gemm(d_g, x, a_is_km=True, b_is_kn=True, out=dwqkv[g * self.cols:(g + 1) * self.cols])
        return dx, dwqkv, dwo

    def __call__(self, x, wqkv_perm, wo, cos=None, sin=None, softmax_scale=None):
        """Differentiable form (autograd through the fused forward and backward)."""
        return _UlyssesFunction.apply(x, wqkv_perm, wo, self, cos, sin, softmax_scale)


class _UlyssesFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wqkv_perm, wo, block: FusedUlyssesAttention, cos, sin, softmax_scale):
        y, o, lse = block.forward(x, wqkv_perm, wo, cos, sin, softmax_scale, return_state=True)
        ctx.save_for_backward(x, wqkv_perm, wo, o, lse)
        ctx.block, ctx.rope, ctx.scale = block, (cos, sin), softmax_scale
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wqkv_perm, wo, o, lse = ctx.saved_tensors
        cos, sin = ctx.rope
        dx, dwqkv, dwo = ctx.block.backward(dy, x, wqkv_perm, wo, o, lse, cos, sin, ctx.scale)
        return dx, dwqkv, dwo, None, None, None, None


def unfused_reference(x, wqkv_perm, wo, group, n_heads, n_kv_heads, head_dim, pattern, cos=None, sin=None,
                      softmax_scale=None) -> torch.Tensor:
    """The same block with plain GEMMs and ``all_to_all`` collectives (the reference's structure),
    differentiable through PyTorch autograd: the comparator of the fused path in tests and timings."""
    from .. import api
    from ..models.llama import _Linear
    sp = dist.get_world_size(group)
    hq, hk, D = n_heads // sp, n_kv_heads // sp, head_dim
    cols = (hq + 2 * hk) * D
    S_loc = x.shape[0]
    qkv = _Linear.apply(x, wqkv_perm)                                   # [S_loc, sp * cols]
    recv = _AllToAll.apply(qkv.view(S_loc, sp, cols).transpose(0, 1).contiguous(), group)   # [sp, S_loc, cols]
    buf = recv.reshape(sp * S_loc, cols)
    q = buf[:, :hq * D].reshape(-1, hq, D)
    k = buf[:, hq * D:(hq + hk) * D].reshape(-1, hk, D)
    v = buf[:, (hq + hk) * D:].reshape(-1, hk, D)
    if cos is not None:
        from ..models.llama import _rope_any
        pos = torch.arange(sp * S_loc, device=x.device, dtype=torch.int32)
        q = _rope_any(q.contiguous(), cos, sin, pos, D)
        k = _rope_any(k.contiguous(), cos, sin, pos, D)
    o = api.attention(q.unsqueeze(0).contiguous(), k.unsqueeze(0).contiguous(), v.unsqueeze(0).contiguous(),
                      pattern, softmax_scale=softmax_scale)[0]          # [S, hq, D]
    back = _AllToAll.apply(o.reshape(sp, S_loc, hq * D).contiguous(), group)                # [sp, S_loc, hq*D]
    a = back.transpose(0, 1).reshape(S_loc, sp * hq * D)
    return _Linear.apply(a.contiguous(), wo)


class _AllToAll(torch.autograd.Function):
    """all_to_all over the leading dimension (one slice per rank); its own transpose in backward."""

    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        t = t.contiguous()
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g, group=ctx.group)
        return out, None
