"""Dense masked-softmax attention in fp32: the numerical oracle of every execution path.

The mask comes from the same block table the planner uses, so a plan that executes correctly must
reproduce this output (and, through autograd, these gradients) up to rounding.
"""
from __future__ import annotations

import math

import torch

from .blocks import BSA_Repr


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor,
                    softmax_scale: float | None = None):
    """q [B, Sq, H, D], k/v [B, Sk, Hkv, D], mask bool [Sq, Sk] -> (O [B, Sq, H, D], lse [B, H, Sq]).
    Rows without any visible key give O = 0 and lse = -inf."""
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    group = q.shape[2] // k.shape[2]
    kf, vf = k.float(), v.float()
    if group > 1:
        kf = kf.repeat_interleave(group, dim=2)
        vf = vf.repeat_interleave(group, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) * scale
    s = s.masked_fill(~mask.to(s.device)[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.masked_fill(lse == float("-inf"), 0.0)[..., None])
    p = torch.where(torch.isfinite(s), p, torch.zeros_like(p))
    return torch.einsum("bhqk,bkhd->bqhd", p, vf), lse


def dense_attention_with_grads(q, k, v, d_o, pattern: BSA_Repr, softmax_scale=None):
    """Oracle forward + autograd backward for a block pattern. Returns (O, lse, dQ, dK, dV)."""
    mask = pattern.token_mask(q.shape[1], k.shape[1])
    q_ = q.detach().float().requires_grad_()
    k_ = k.detach().float().requires_grad_()
    v_ = v.detach().float().requires_grad_()
    o, lse = dense_attention(q_, k_, v_, mask, softmax_scale)
    o.backward(d_o.float())
    return o.detach(), lse.detach(), q_.grad, k_.grad, v_.grad
