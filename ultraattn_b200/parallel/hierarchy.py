"""Two-level (node x device) attention baseline.

Reference: hierarchy_attn/hierarchy_attn_impl.py:14-277 — inside a node K/V travel a ring, across
nodes the queries visit the other nodes and (O, lse) come back; forward only in the reference
(its backward is ``pass``). Here both levels move K/V: a block makes a full tour of the intra-node
ring and then takes one hop on the inter-node ring, so only every ``tasks_per_node``-th hop
crosses the slow links, the queries and their outputs never leave their rank, and the backward
follows from the same route (dK/dV travel with their block and go home with one exchange per
level). On a single NVSwitch box the inter level has one node and this is the ring strategy.
"""
from __future__ import annotations

import torch.distributed as dist

from .ring import _check_unsupported, _RingFunc

_group_cache: dict = {}


def create_hierarchy_groups(tasks_per_node: int, world_size: int | None = None) -> dict:
    """``{'intra': pg, 'inter': pg}`` for consecutive-rank nodes (reference:
    hierarchy_attn/utils.py:69-117 creates its intra / inter groups the same way, lazily). Every
    rank must call this (``dist.new_group`` is collective); the result is cached."""
    world = world_size or dist.get_world_size()
    key = (tasks_per_node, world)
    if key in _group_cache:
        return _group_cache[key]
    assert world % tasks_per_node == 0
    rank = dist.get_rank()
    groups = {}
    for n in range(world // tasks_per_node):
        ranks = list(range(n * tasks_per_node, (n + 1) * tasks_per_node))
        g = dist.new_group(ranks)
        if rank in ranks:
            groups["intra"] = g
    for loc in range(tasks_per_node):
        ranks = list(range(loc, world, tasks_per_node))
        g = dist.new_group(ranks)
        if rank in ranks:
            groups["inter"] = g
    _group_cache[key] = groups
    return groups


def hierarchy_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                        alibi_slopes=None, deterministic=False, return_attn_probs=False, groups=None,
                        group=None, PROC_INFO=None):
    """``groups``: ``{'intra': pg, 'inter': pg}`` (the reference's convention; see
    :func:`create_hierarchy_groups`). Shards are ordered by ``node * tasks_per_node + local rank``;
    causal inputs use the zigzag layout over that order (``shard_sequence(..., 'zigzag')``)."""
    _check_unsupported(dropout_p, alibi_slopes, window_size)
    route = group
    if isinstance(groups, dict) and groups.get("inter") is not None \
            and dist.get_world_size(groups["inter"]) > 1:
        route = {"intra": groups["intra"], "inter": groups["inter"]}
    elif isinstance(groups, dict):
        route = groups.get("intra", group)
    o, lse = _RingFunc.apply(q, k, v, softmax_scale, causal, route, "zigzag" if causal else "ring")
    return (o, lse, None) if return_attn_probs else o
