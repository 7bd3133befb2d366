"""Named pattern constructors: full, causal, strided, global+local, star, streaming.

Every constructor returns a :class:`~ultraattn_b200.patterns.blocks.BSA_Repr`. Diagonal blocks
of causal-type patterns are CAUSAL, off-diagonal ones FULL; wording that admits two readings
("window of w blocks": does it count the block itself?) is resolved by explicit parameters:
``window`` always counts the diagonal block, so ``window=1`` is "self only" and ``window=2`` is
"self and the previous block".

Covers the reference's parametric generator (search_algo/custom_sparse_pattern.py:5-89: star,
stream, local_global; its ``stride`` branch is an empty stub) and its six canonical tables
(search_algo/bsa_utils.py:115-150), reproduced by :func:`create_bsa_block_table`.
"""
from __future__ import annotations

import numpy as np

from .blocks import BSA_Repr, CAUSAL, EMPTY, FULL, _to_enum


def full(n_blocks: int = 1) -> BSA_Repr:
    return BSA_Repr(np.full((n_blocks, n_blocks), FULL, dtype=np.int8))


def causal(n_blocks: int = 1) -> BSA_Repr:
    t = np.zeros((n_blocks, n_blocks), dtype=np.int8)
    t[np.tril_indices(n_blocks, -1)] = FULL
    t[np.diag_indices(n_blocks)] = CAUSAL
    return BSA_Repr(t)


def strided(n_blocks: int, stride: int, window: int = 2) -> BSA_Repr:
    """Causal strided attention: query block i sees key block j <= i iff ``i - j < window`` or
    ``(i - j) % stride == 0``."""
    t = np.zeros((n_blocks, n_blocks), dtype=np.int8)
    for i in range(n_blocks):
        for j in range(i + 1):
            if i - j < window or (i - j) % stride == 0:
                t[i, j] = CAUSAL if i == j else FULL
    return BSA_Repr(t)


def global_local(n_blocks: int, n_global: int = 1, window: int = 2, causal_local: bool = True,
                 global_rows_see_all: bool = True) -> BSA_Repr:
    """Global + local attention: the first ``n_global`` blocks are global (every query block sees
    them; with ``global_rows_see_all`` they also see every key block, future ones included), plus
    a local band of ``window`` blocks ending at the diagonal. With ``causal_local`` the band is
    causal (diagonal blocks CAUSAL); otherwise the band is symmetric and FULL."""
    t = np.zeros((n_blocks, n_blocks), dtype=np.int8)
    for i in range(n_blocks):
        for j in range(n_blocks):
            if causal_local:
                if 0 <= i - j < window:
                    t[i, j] = CAUSAL if i == j else FULL
            elif abs(i - j) < window:
                t[i, j] = FULL
    t[:, :n_global] = np.where(t[:, :n_global] == CAUSAL, CAUSAL, FULL)
    if global_rows_see_all:
        t[:n_global, :] = FULL
    else:
        for i in range(n_global):
            t[i, i] = CAUSAL if causal_local else FULL
    return BSA_Repr(t)


def star(n_blocks: int, n_sink: int = 1) -> BSA_Repr:
    """Star attention prefill: every query block sees the first ``n_sink`` key blocks and itself
    (causally)."""
    return streaming(n_blocks, n_sink, window=1)


def streaming(n_blocks: int, n_sink: int = 1, window: int = 1) -> BSA_Repr:
    """Streaming (attention-sink) prefill: ``n_sink`` sink blocks plus a causal local band of
    ``window`` blocks (the diagonal block counts)."""
    t = np.zeros((n_blocks, n_blocks), dtype=np.int8)
    for i in range(n_blocks):
        for j in range(i + 1):
            if j < n_sink or i - j < window:
                t[i, j] = CAUSAL if i == j else FULL
    return BSA_Repr(t)


def document(doc_blocks, causal_docs: bool = True) -> BSA_Repr:
    """Document mask for a packed batch whose documents are whole numbers of blocks long:
    ``doc_blocks[i]`` blocks for document i. Tokens attend only their own document (causally, or
    fully with ``causal_docs=False``), so the table is block-diagonal. The reference lists this
    mask as future work (its README.md:71); as a block table it goes through the same planner and
    runtimes as every other pattern, which gives context parallelism over packed documents."""
    n = int(sum(doc_blocks))
    t = np.zeros((n, n), dtype=np.int8)
    a = 0
    for d in doc_blocks:
        for i in range(a, a + d):
            for j in range(a, (i if causal_docs else a + d - 1) + 1):
                t[i, j] = (CAUSAL if i == j else FULL) if causal_docs else FULL
        a += d
    return BSA_Repr(t)


def by_name(name: str, **kw) -> BSA_Repr:
    table = {"full": full, "causal": causal, "strided": strided, "stride": strided,
             "global_local": global_local, "local_global": global_local, "lg": global_local,
             "star": star, "streaming": streaming, "stream": streaming, "document": document}
    if name not in table:
        raise KeyError(f"unknown pattern {name!r}; choose from {sorted(set(table))}")
    return table[name](**kw)


def create_bsa_block_table(case_id: int) -> np.ndarray:
    """The reference's six canonical tables as enum arrays (search_algo/bsa_utils.py:115-150):
    0 strided(1/16, 4, 3) after remapping, 1 global+local(1/16, 1, 1), 2 star(1/4),
    3 streaming(1/8, 3 local), 4 full, 5 causal."""
    if case_id == 0:
        t = np.zeros((16, 16), dtype=np.int8)
        for r in range(4):
            blk = np.full((4, 4), FULL, dtype=np.int8)
            blk[0, 3] = blk[3, 0] = EMPTY
            t[r * 4:(r + 1) * 4, r * 4:(r + 1) * 4] = blk
    elif case_id == 1:
        t = np.zeros((16, 16), dtype=np.int8)
        t[:, 0] = FULL
        t[0, :] = FULL
        t[np.diag_indices(16)] = FULL
    elif case_id == 2:
        t = star(4, 1).block_table_int
    elif case_id == 3:
        t = streaming(8, 1, 3).block_table_int
    elif case_id == 4:
        t = np.array([[FULL]], dtype=np.int8)
    elif case_id == 5:
        t = np.array([[CAUSAL]], dtype=np.int8)
    else:
        raise ValueError(f"unsupported bsa_block_table case_id={case_id}")
    return _to_enum(t)


# -------------------------------------------------------------------------------------------------
# context remap: block permutations that make a pattern cheaper to tile across ranks
# -------------------------------------------------------------------------------------------------
def cmap_contiguous(n_blocks: int, cp: int) -> np.ndarray:
    """Block i belongs to rank ``i // (n_blocks / cp)`` (the reference's default,
    search_algo/workload_partition.py:320-322)."""
    return np.arange(n_blocks) // (n_blocks // cp)


def cmap_strided(n_blocks: int, cp: int) -> np.ndarray:
    """Residue classes: block i belongs to rank ``i % cp``; groups the blocks that a strided
    pattern couples, and balances causal work."""
    return np.arange(n_blocks) % cp


def cmap_zigzag(n_blocks: int, cp: int) -> np.ndarray:
    """Zigzag: with 2*cp chunks, rank r owns chunks r and 2*cp-1-r (reference input sharding of
    the zigzag ring, easy_context/zigzag_ring_attn/prepare_inputs.py:4-9); generalised to
    ``n_blocks`` a multiple of ``2*cp``."""
    assert n_blocks % (2 * cp) == 0
    per = n_blocks // (2 * cp)
    chunk = np.arange(n_blocks) // per
    return np.where(chunk < cp, chunk, 2 * cp - 1 - chunk)


def remap_permutation(cmap: np.ndarray) -> np.ndarray:
    """Stable permutation of block indices that makes ownership contiguous (rank 0's blocks first).
    Applying it to token ids / position ids at data-loading time realises the remap."""
    return np.argsort(cmap, kind="stable")


def permute_pattern(repr_: BSA_Repr, perm: np.ndarray) -> np.ndarray:
    """Block table after re-ordering both axes by ``perm``. A CAUSAL diagonal block stays on the
    diagonal; FULL/EMPTY blocks move freely. (Token-level causality inside a block is unchanged
    because blocks move whole.)"""
    t = repr_.block_table_int
    return t[np.ix_(perm, perm)]
