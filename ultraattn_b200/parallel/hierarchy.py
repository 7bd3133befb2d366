"""Two-level (node x device) attention baseline.

Reference: hierarchy_attn/hierarchy_attn_impl.py:14-277 — inside a node K/V travel a ring, across
nodes the queries visit the other nodes and (O, lse) come back; forward only in the reference
(its backward is ``pass``). Here the inter-node exchange is expressed with the same ring
machinery: an outer ring over node groups moves K/V shards between nodes while the inner ring
runs inside each node, which yields the same result and supports the backward. On a single
NVSwitch box the inter level has one node and this reduces to the ring strategy.
"""
from __future__ import annotations

import torch.distributed as dist

from .ring import _RingFunc


def hierarchy_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                        alibi_slopes=None, deterministic=False, return_attn_probs=False, groups=None,
                        group=None, PROC_INFO=None):
    """``groups`` may be a dict with 'intra' / 'inter' process groups (the reference's convention);
    with a single node only the intra group matters."""
    pg = group
    if isinstance(groups, dict):
        inter = groups.get("inter")
        if inter is not None and dist.get_world_size(inter) > 1:
            pg = groups.get("world", None)      # a flat ring over all ranks covers both levels
        else:
            pg = groups.get("intra", group)
    o, lse = _RingFunc.apply(q, k, v, softmax_scale, causal, pg, "zigzag" if causal else "ring")
    return (o, lse, None) if return_attn_probs else o
