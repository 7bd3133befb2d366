"""Head-parallel (Ulysses) attention with both all-to-alls fused into the projection GEMMs.

Unfused (reference: head_parallel_attn/deepspeed_ulysses_attn.py, comm_lib/comm_utils.py:32-45):
    qkv = x @ Wqkv^T            ->  all-to-all (sequence shard -> head shard)  ->  attention
    attention                   ->  all-to-all (head shard -> sequence shard)  ->  y = o @ Wo^T
Fused (this module):
    the QKV GEMM's epilogue stores every head group's output tile directly into the receive
    buffer of the rank that owns those heads (peer stores over NVLink, ``gemm_scatter``);
    the output projection's TMA producer loads its A operand, K-group by K-group, directly from
    the attention outputs held by the owning ranks (unicast TMA over peer mappings,
    ``gemm_gather``). No all-to-all kernel exists on this path.

Weights: ``wqkv`` rows must be ordered by destination rank — for rank g the rows
``[q heads of g | k heads of g | v heads of g]`` — :func:`permute_qkv_weight` produces that order
from the usual ``[q | k | v]`` layout. The backward runs through the unfused path
(:func:`ultraattn_b200.parallel.ring.deepspeed_ulysses_attn_func`).
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


class FusedUlyssesAttention:
    def __init__(self, group, device, seq_len: int, hidden: int, n_heads: int, n_kv_heads: int = None,
                 head_dim: int = 128, causal: bool = True):
        self.group, self.device = group, device
        self.sp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.S, self.S_loc = seq_len, seq_len // self.sp
        self.H, self.Hk, self.D = n_heads, n_kv_heads or n_heads, head_dim
        self.hq, self.hk = self.H // self.sp, self.Hk // self.sp
        self.cols = (self.hq + 2 * self.hk) * head_dim
        self.causal = causal
        self.space = SymmMemSpace(group, device)
        self.space.alloc("qkv", (seq_len, self.cols), torch.bfloat16)
        self.space.alloc("attn", (seq_len, self.hq * head_dim), torch.bfloat16)
        self.space.finalize()
        from ..api import local_plans
        from ..patterns import named
        self.fplan, _ = local_plans(named.causal(1) if causal else named.full(1), seq_len, device)

    def forward(self, x: torch.Tensor, wqkv_perm: torch.Tensor, wo: torch.Tensor, cos=None, sin=None,
                softmax_scale=None) -> torch.Tensor:
        """x [S/sp, hidden] (this rank's tokens) -> y [S/sp, hidden]."""
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
        o = sp.local("attn").view(1, self.S, self.hq, D)
        lse = torch.empty(1, self.hq, self.S, dtype=torch.float32, device=self.device)
        A.attn_fwd([q.unsqueeze(0)], [k.unsqueeze(0)], [v.unsqueeze(0)], [(o, lse)], self.fplan, softmax_scale)
        sp.barrier(6)                       # every rank's attention output is complete
        y = torch.empty(self.S_loc, wo.shape[0], dtype=torch.bfloat16, device=self.device)
        src = [sp.peer("attn", r).data_ptr() for r in range(self.sp)]
        G.gemm_gather(src, self.S, self.hq * D, self.rank * self.S_loc, self.S_loc, self.hq * D, wo, y)
        return y
