"""Two-level (node x device) context tiling, flattened to one allocation over all ranks.

The reference plans in two levels (search_algo/task1_bsa.py:501-547, search_algo/benchmark.py:21-83):
ILP #1 at node granularity assigns *node tiles* to nodes, and every node tile is itself a
block-sparse sub-problem whose device tiles are allocated to the GPUs of that node; at run time an
inter-level compute kernel *is* an intra-level plan (orchestrated_attn/orchestrated_attn_impl.py:
132-213). Here the two allocations are composed into a single tile -> global-rank table, so the
ordinary single-level graph, scheduler and executors run it: messages between ranks of different
nodes are the inter-node traffic, the rest is intra-node.
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from ..patterns.blocks import BSA_Config, BSA_Repr
from .allocate import EMPTY_TILE, Allocation, comm_volumes, comp_volumes, solve_sparse_from_bsa, tile_volumes


def flatten_two_level(bsa_config: BSA_Config, fob: int = 0, time_limit: float = 20.0,
                      node_ParD: Optional[int] = None) -> Allocation:
    """``bsa_config.CP = (intra, inter)``. Returns an allocation over ``intra * inter`` ranks at
    granularity ``ParD = ParD_node * ParD_dev`` where rank = node * intra + local rank and block i
    belongs to rank ``i // (ParD / ranks)`` (nodes own contiguous chunks, devices contiguous
    sub-chunks)."""
    intra, inter = bsa_config.CP
    pat = bsa_config.bsa_repr
    if inter == 1:
        al = solve_sparse_from_bsa(bsa_config, fob=fob, hierarchy=1, time_limit=time_limit)
        return al
    # level 0: node tiles -> nodes
    n_node = node_ParD or inter
    top = solve_sparse_from_bsa(bsa_config, fob=fob, ParD=n_node, hierarchy=0, time_limit=time_limit)
    per_node = n_node // inter
    # level 1: inside every node tile, device tiles -> local ranks. The sub-pattern of node tile
    # (R, C) is planned as an intra-node problem whose rows / columns are owned by the GPUs of
    # the node that holds the Q rows / the K,V columns; tiles computed on a third node are
    # first assigned by the sub-problem's own allocation (local index) and then mapped there.
    sub_size = max(intra, 1)
    # granularity of the flat table
    fine = max(pat.table.shape[0], n_node * sub_size)
    while fine % (n_node * sub_size) != 0 or fine % pat.table.shape[0] != 0:
        fine += 1
    per_tile = fine // n_node
    vol = tile_volumes(pat, fine)
    ranks = intra * inter
    cmap = np.arange(fine) // (fine // ranks)
    table = np.full((fine, fine), EMPTY_TILE, dtype=np.int64)
    cache: dict = {}
    for R in range(n_node):
        for C in range(n_node):
            node = int(top.table[R, C])
            if node < 0:
                continue
            rows = list(range(R * per_tile, (R + 1) * per_tile))
            cols = list(range(C * per_tile, (C + 1) * per_tile))
            sub = BSA_Repr(pat.refined(fine)[np.ix_(rows, cols)])
            key = str(sub)
            if key not in cache:
                cfg = BSA_Config(None, None, {"bsa_repr": sub, "CP": (intra, 1)})
                if sub.check_empty():
                    cache[key] = None
                else:
                    cache[key] = solve_sparse_from_bsa(cfg, fob=fob, ParD=per_tile if per_tile % intra == 0 else None,
                                                       hierarchy=1, time_limit=time_limit)
            sa = cache[key]
            if sa is None:
                continue
            st = np.asarray(sa.table)
            f = per_tile // st.shape[0]
            for i in range(per_tile):
                for j in range(per_tile):
                    if vol[rows[i], cols[j]] > 0:
                        local = int(st[i // f, j // f])
                        if local < 0:
                            local = int(cmap[rows[i]]) % intra
                        table[rows[i], cols[j]] = node * intra + local
    cin, cout = comm_volumes(table, cmap, ranks, fob)
    return Allocation(fine, cmap, table, float(max(cin.max(), cout.max())),
                      float(comp_volumes(table, vol, ranks).max()), "two-level")
