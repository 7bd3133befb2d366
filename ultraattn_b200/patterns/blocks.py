"""Block-sparse attention patterns: the CP-agnostic block table and its algebra.

A pattern is a small 2-D table whose entries say how a block of queries attends a block of keys:
EMPTY (not at all), FULL (every pair) or CAUSAL (lower triangle, diagonal included). The same
table serves any context-parallel degree because it can be *coarsened* to its irreducible form
and *refined* on demand: a CAUSAL block refines into a lower-triangular arrangement of
CAUSAL / FULL / EMPTY blocks.

Behaviour follows the reference's ``BSA_Repr`` / ``BSA_Config`` (search_algo/bsa_config.py:10-263,
265-383) and ``Block_Type`` (search_algo/utils.py:135-149): the string form
``[[2000][1200][1020][1002]]`` and ``CP=(a, b)_repr=[[...]]`` are part of the plan-database key
grammar and are reproduced exactly. Tables are held as small integer arrays here; the
``block_table_raw`` attribute exposes enum objects for code written against the reference.
"""
from __future__ import annotations

import enum
import math
from typing import Optional, Sequence

import numpy as np


class Block_Type(enum.Enum):
    EMPTY = 0
    FULL = 1
    CAUSAL = 2


class Block_Table_Type(enum.Enum):
    EMPTY = 0
    FULL = 1
    PARTIAL = 2


Block_Comp_Volume = {Block_Type.EMPTY: 0.0, Block_Type.FULL: 1.0, Block_Type.CAUSAL: 0.5}
_VOLUME = np.array([0.0, 1.0, 0.5])

EMPTY, FULL, CAUSAL = 0, 1, 2


def _prime_factors(n: int) -> list[int]:
    out, p = [], 2
    while p * p <= n:
        while n % p == 0:
            out.append(p)
            n //= p
        p += 1
    if n > 1:
        out.append(n)
    return out


def as_int_table(table) -> np.ndarray:
    """Accept int arrays, nested lists or object arrays of ``Block_Type`` and return int8."""
    arr = np.asarray(table)
    if arr.dtype == object:
        arr = np.vectorize(lambda b: b.value if isinstance(b, Block_Type) else int(b))(arr)
    arr = arr.astype(np.int8)
    assert arr.ndim == 2, "a block table is two-dimensional"
    assert ((arr >= 0) & (arr <= 2)).all(), "block types are 0 (empty), 1 (full), 2 (causal)"
    return arr


def _causal_template(k: int) -> np.ndarray:
    t = np.zeros((k, k), dtype=np.int8)
    t[np.tril_indices(k, -1)] = FULL
    t[np.diag_indices(k)] = CAUSAL
    return t


def coarsen_once(table: np.ndarray, k: int) -> Optional[np.ndarray]:
    """Merge every k x k group of blocks into one block if each group is uniformly EMPTY, uniformly
    FULL or exactly the refined form of a CAUSAL block; otherwise return None."""
    nq, nk = table.shape
    if k <= 1 or nq % k or nk % k:
        return None
    g = table.reshape(nq // k, k, nk // k, k).transpose(0, 2, 1, 3)        # [Q, K, k, k]
    is_empty = (g == EMPTY).all(axis=(2, 3))
    is_full = (g == FULL).all(axis=(2, 3))
    is_causal = (g == _causal_template(k)[None, None]).all(axis=(2, 3))
    if not (is_empty | is_full | is_causal).all():
        return None
    out = np.zeros((nq // k, nk // k), dtype=np.int8)
    out[is_full] = FULL
    out[is_causal] = CAUSAL
    return out


def coarsen(table: np.ndarray) -> np.ndarray:
    """Irreducible form: repeatedly merge by the prime factors of gcd(shape) while possible
    (reference: BSA_Repr.simplify, search_algo/bsa_config.py:160-175)."""
    table = as_int_table(table)
    for p in _prime_factors(math.gcd(*table.shape)):
        nxt = coarsen_once(table, p)
        if nxt is None:
            # the reference stops trying this prime at the first failure and moves to the next
            continue
        table = nxt
    return table


def refine(table: np.ndarray, rate: int) -> np.ndarray:
    """Split every block into rate x rate blocks (reference: BSA_Repr.complicate, :203-224)."""
    table = as_int_table(table)
    if rate == 1:
        return table.copy()
    nq, nk = table.shape
    out = np.repeat(np.repeat(table, rate, axis=0), rate, axis=1)
    tmpl = _causal_template(rate)
    for i, j in zip(*np.nonzero(table == CAUSAL)):
        out[i * rate:(i + 1) * rate, j * rate:(j + 1) * rate] = tmpl
    return out


class BSA_Repr:
    """A block-sparse attention pattern, independent of how many GPUs will run it.

    ``block_table`` is what the caller gave, ``table`` / ``block_table_raw`` the irreducible form.
    ``cmap`` optionally assigns every block row of ``block_table`` to a context-parallel rank (the
    "context remap" hook: which rank owns which chunk of the sequence).
    """

    def __init__(self, block_table, cmap: Optional[Sequence[int]] = None):
        self.block_table_int = as_int_table(block_table)
        self.cmap = None if cmap is None else np.asarray(cmap, dtype=np.int64)
        self.table = coarsen(self.block_table_int)
        self.cmap_raw = self._coarsen_cmap()
        self.minimum_Par_D = self.table.shape[0]

    def __getstate__(self) -> dict:
        """Pickled with the attribute names and value types of the reference's class (tables of
        ``Block_Type``, ``block_table_raw`` / ``cmap_raw``, the two ``*_Par_D`` slots), so that a
        plan written here is usable after the reference loads it; :meth:`__setstate__` rebuilds
        this class's own fields from ``block_table`` and ``cmap``."""
        return {"block_table": self.block_table, "cmap": self.cmap, "block_table_raw": self.block_table_raw,
                "cmap_raw": self.cmap_raw, "block_table_Par_D": None, "cmap_Par_D": None,
                "minimum_Par_D": self.minimum_Par_D}

    def __setstate__(self, state: dict) -> None:
        """A pattern pickled here or by the reference (inside one of its plans): both carry
        ``block_table`` / ``cmap``; everything else is derived again."""
        if "block_table_int" not in state and "block_table" in state:
            self.__init__(state["block_table"], state.get("cmap"))
            return
        self.__dict__.update(state)

    # -- reference-compatible views -------------------------------------------------------------
    @property
    def block_table(self) -> np.ndarray:
        return _to_enum(self.block_table_int)

    @property
    def block_table_raw(self) -> np.ndarray:
        return _to_enum(self.table)

    def _coarsen_cmap(self):
        if self.cmap is None:
            return None
        n0, n1 = self.block_table_int.shape[0], self.table.shape[0]
        if n0 == n1:
            return self.cmap.copy()
        k = n0 // n1
        groups = self.cmap.reshape(n1, k)
        if (groups == groups[:, :1]).all():
            return groups[:, 0].copy()
        return None

    # -- predicates -----------------------------------------------------------------------------
    def check_empty(self) -> bool:
        return bool((self.table == EMPTY).all())

    def check_full(self) -> bool:
        return bool((self.table == FULL).all())

    def check_causal(self) -> bool:
        """True if the pattern is lower-triangular with CAUSAL blocks on the diagonal and only
        EMPTY / FULL below it (reference :44-53)."""
        t = self.table
        if t.shape[0] != t.shape[1]:
            return False
        n = t.shape[0]
        iu = np.triu_indices(n, 1)
        il = np.tril_indices(n, -1)
        return bool((t[iu] == EMPTY).all() and (np.diag(t) == CAUSAL).all()
                    and np.isin(t[il], (EMPTY, FULL)).all())

    # -- algebra --------------------------------------------------------------------------------
    def refined(self, n: int) -> np.ndarray:
        """Integer table at n x n granularity (n a multiple of the irreducible size)."""
        cur = self.table.shape[0]
        assert self.table.shape[0] == self.table.shape[1], "refinement needs a square pattern"
        assert n % cur == 0, f"cannot express a {cur}-block pattern with {n} blocks"
        return refine(self.table, n // cur)

    def complicate_to(self, n: int) -> np.ndarray:
        return _to_enum(self.refined(n))

    def create_sub_bsa_repr(self, split_degrees: Sequence[int], select_ids: Sequence[Sequence[int]]) -> "BSA_Repr":
        """Pattern seen by a subset of row chunks x column chunks when both axes are cut into
        ``split_degrees`` equal chunks (reference :24-42)."""
        assert len(split_degrees) == 2 and split_degrees[0] == split_degrees[1]
        n = split_degrees[0]
        cur = self.table.shape[0]
        if n >= cur:
            tab = self.refined(n) if n > cur else self.table
            rows, cols = list(select_ids[0]), list(select_ids[1])
        else:
            assert cur % n == 0
            f = cur // n
            tab = self.table
            rows = [r * f + x for r in select_ids[0] for x in range(f)]
            cols = [c * f + x for c in select_ids[1] for x in range(f)]
        return BSA_Repr(tab[np.ix_(rows, cols)], None)

    def split_n(self, n: int) -> list["BSA_Repr"]:
        """The distinct sub-patterns of an n x n cut (used to plan each distinct node-level tile
        once; reference :226-246)."""
        cur = self.table.shape[0]
        if cur >= n:
            assert cur % n == 0
            tab, sz = self.table, cur // n
        else:
            tab, sz = self.refined(n), 1
        out: list[BSA_Repr] = []
        for i in range(n):
            for j in range(n):
                sub = BSA_Repr(tab[i * sz:(i + 1) * sz, j * sz:(j + 1) * sz], None)
                if not any(sub == o for o in out):
                    out.append(sub)
        return out

    # -- measures -------------------------------------------------------------------------------
    @property
    def volume(self) -> float:
        """Work in units of one FULL block of the irreducible table."""
        return float(_VOLUME[self.table].sum())

    @property
    def sparsity(self) -> float:
        return self.volume / self.table.size

    # -- identity -------------------------------------------------------------------------------
    def __str__(self) -> str:
        return "[" + "".join("[" + "".join(str(int(v)) for v in row) + "]" for row in self.table) + "]"

    __repr__ = __str__

    def __eq__(self, other) -> bool:
        return isinstance(other, BSA_Repr) and np.array_equal(self.table, other.table)

    def __hash__(self) -> int:
        return hash(str(self))

    @classmethod
    def from_string(cls, s: str) -> "BSA_Repr":
        rows = [r for r in s.strip()[1:-1].replace("][", "],[").split(",")]
        return cls(np.array([[int(c) for c in r.strip("[]")] for r in rows], dtype=np.int8))

    # -- token-level mask (the oracle's view of the same table) ----------------------------------
    def token_mask(self, seq_q: int, seq_k: Optional[int] = None, table: Optional[np.ndarray] = None):
        """Boolean [seq_q, seq_k] mask (True = attend) generated from the block table."""
        import torch
        seq_k = seq_q if seq_k is None else seq_k
        tab = self.block_table_int if table is None else table
        nq, nk = tab.shape
        assert seq_q % nq == 0 and seq_k % nk == 0
        bq, bk = seq_q // nq, seq_k // nk
        mask = torch.zeros(seq_q, seq_k, dtype=torch.bool)
        tri = torch.tril(torch.ones(bq, bk, dtype=torch.bool))
        for i in range(nq):
            for j in range(nk):
                if tab[i, j] == FULL:
                    mask[i * bq:(i + 1) * bq, j * bk:(j + 1) * bk] = True
                elif tab[i, j] == CAUSAL:
                    mask[i * bq:(i + 1) * bq, j * bk:(j + 1) * bk] = tri
        return mask


def _to_enum(table: np.ndarray) -> np.ndarray:
    lut = np.array([Block_Type.EMPTY, Block_Type.FULL, Block_Type.CAUSAL], dtype=object)
    return lut[table]


class BSA_Config:
    """A pattern plus the context-parallel degrees it will run on: ``CP = (intra, inter)``.

    Live constructor of the reference: ``BSA_Config(None, None, {'bsa_repr': ..., 'CP': (a, b)})``
    (search_algo/bsa_config.py:293-300). ``to_string()`` is embedded in every database key.
    """

    def __init__(self, pat_dict=None, pat_s=None, pat_bsa_repr: Optional[dict] = None):
        if pat_bsa_repr is None:
            raise ValueError("BSA_Config is built from {'bsa_repr': BSA_Repr, 'CP': (intra, inter)}; "
                             "use patterns.named.* to create the BSA_Repr")
        self.bsa_repr: BSA_Repr = pat_bsa_repr["bsa_repr"]
        self.CP = tuple(pat_bsa_repr["CP"])
        self.cmap = self.bsa_repr.cmap
        self.pat_dict = None
        self.pat_s = None
        self.causal = self.bsa_repr.check_causal()

    @property
    def block_table_raw(self):
        return self.bsa_repr.block_table_raw

    @property
    def table(self) -> np.ndarray:
        return self.bsa_repr.table

    @classmethod
    def create_full(cls, CP: tuple) -> "BSA_Config":
        return cls(None, None, {"bsa_repr": BSA_Repr(np.array([[FULL]])), "CP": CP})

    @classmethod
    def create_causal(cls, CP: tuple) -> "BSA_Config":
        return cls(None, None, {"bsa_repr": BSA_Repr(np.array([[CAUSAL]])), "CP": CP})

    @property
    def total_sparsity(self) -> float:
        return self.bsa_repr.sparsity

    def to_string(self) -> str:
        return f"CP={self.CP}_repr={self.bsa_repr}"

    __str__ = to_string
    __repr__ = to_string

    def __eq__(self, other) -> bool:
        return isinstance(other, BSA_Config) and self.CP == other.CP and self.bsa_repr == other.bsa_repr

    def __hash__(self) -> int:
        return hash(self.to_string())

    def print_block_table(self) -> None:
        print(f"block_table_raw_value:\n{self.table}")
