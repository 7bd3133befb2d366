"""Small utilities (reference: search_algo/utils.py:21-133, 184-227)."""
from __future__ import annotations

import functools
import heapq
import os

import numpy as np

from ..patterns.blocks import Block_Table_Type, _VOLUME, as_int_table


def print_rank_0(*args, **kw) -> None:
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*args, **kw, flush=True)


def use_all_cpus(fn):
    """Run ``fn`` with the affinity mask widened to every CPU (solver runs under srun/numactl
    otherwise inherit a one-core mask), then restore it."""
    @functools.wraps(fn)
    def wrapped(*a, **kw):
        if not hasattr(os, "sched_getaffinity"):
            return fn(*a, **kw)
        old = os.sched_getaffinity(0)
        try:
            os.sched_setaffinity(0, range(os.cpu_count() or 1))
        except OSError:
            pass
        try:
            return fn(*a, **kw)
        finally:
            try:
                os.sched_setaffinity(0, old)
            except OSError:
                pass
    return wrapped


def report_memory(name: str = "") -> dict:
    """Allocator and device memory in GiB (torch allocator + NVML when available)."""
    import torch
    out = {}
    if torch.cuda.is_available():
        gib = 1024 ** 3
        out = {"allocated": torch.cuda.memory_allocated() / gib,
               "max_allocated": torch.cuda.max_memory_allocated() / gib,
               "reserved": torch.cuda.memory_reserved() / gib}
        try:
            free, total = torch.cuda.mem_get_info()
            out.update(device_used=(total - free) / gib, device_total=total / gib)
        except RuntimeError:
            pass
        print_rank_0(f"[memory] {name} " + " ".join(f"{k}={v:.2f}GiB" for k, v in out.items()))
    return out


def calc_flops(bs: int, S, Nh: int, D: int, causal: bool = False, fob: int = 0, sparsity: float = 1.0):
    """(model FLOPs, hardware FLOPs) of attention: forward 4*Sq*Skv*D per head; the backward is
    2x in model FLOPs and 2.5x in hardware FLOPs (the recomputed S = QK^T)."""
    sq, skv = (S, S) if isinstance(S, int) else S
    f = 4.0 * bs * sq * skv * Nh * D * sparsity * (0.5 if causal else 1.0)
    return (f, f) if fob == 0 else (2.0 * f, 2.5 * f)


def unique_list(items: list) -> list:
    out = []
    for it in items:
        if not any(it == o for o in out):
            out.append(it)
    return out


def calc_table_comp_relative_time(table) -> float:
    return float(_VOLUME[as_int_table(table)].sum())


def get_block_table_type(table) -> Block_Table_Type:
    t = as_int_table(table)
    if (t == 0).all():
        return Block_Table_Type.EMPTY
    if (t == 1).all():
        return Block_Table_Type.FULL
    return Block_Table_Type.PARTIAL


class FinitePriorityQueue:
    """Keeps the ``max_size`` smallest items (by key) seen so far."""

    def __init__(self, max_size: int, pack_func=lambda x: x, unpack_func=lambda x: x):
        self.max_size = max_size
        self.pack, self.unpack = pack_func, unpack_func
        self._heap: list = []
        self._n = 0

    def push(self, item) -> None:
        key = self.pack(item)
        entry = (_Neg(key), self._n, item)
        self._n += 1
        if len(self._heap) < self.max_size:
            heapq.heappush(self._heap, entry)
        elif entry[0] > self._heap[0][0]:
            heapq.heapreplace(self._heap, entry)

    def items(self) -> list:
        return [e[2] for e in sorted(self._heap, key=lambda e: e[0], reverse=True)]

    def __len__(self) -> int:
        return len(self._heap)


class _Neg:
    """Reverses ordering so that heapq's min-heap evicts the largest key."""
    __slots__ = ("k",)

    def __init__(self, k): self.k = k
    def __lt__(self, o): return self.k > o.k
    def __gt__(self, o): return self.k < o.k
    def __eq__(self, o): return self.k == o.k


# -------------------------------------------------------------------------------------------------
# small helpers of the reference's search_algo/utils.py that scripts written against it import
# -------------------------------------------------------------------------------------------------
def all_wait_main_stream(stream_list, main_stream) -> None:
    """Every stream of the list waits for the work queued so far on ``main_stream``
    (reference: search_algo/utils.py:105-108)."""
    for s in stream_list:
        if s.cuda_stream != main_stream.cuda_stream:
            s.wait_stream(main_stream)


def main_stream_wait_all(stream_list, main_stream) -> None:
    """``main_stream`` waits for every stream of the list (reference: search_algo/utils.py:110-113)."""
    for s in stream_list:
        if s.cuda_stream != main_stream.cuda_stream:
            main_stream.wait_stream(s)


def convert_block_table_to_value(block_table):
    """Integer table (0 empty, 1 full, 2 causal) of a table of :class:`Block_Type` members."""
    import numpy as np
    flat = [getattr(v, "value", v) for v in np.asarray(block_table, dtype=object).flatten()]
    return np.array(flat, dtype=np.int64).reshape(np.asarray(block_table).shape)


def combine_list_to_0(l0: list, l1: list) -> list:
    """Append to ``l0`` the items of ``l1`` that it lacks (order kept); returns ``l0``."""
    for x in l1:
        if x not in l0:
            l0.append(x)
    return l0


def closest_fraction(x: float, max_denominator: int = 1000):
    from fractions import Fraction
    return Fraction(x).limit_denominator(max_denominator)


def get_factors(n: int) -> list:
    """All divisors of ``n`` in increasing order."""
    small = [d for d in range(1, int(n ** 0.5) + 1) if n % d == 0]
    return sorted(set(small + [n // d for d in small]))


def find_file_with_regex(directory: str, pattern: str) -> list:
    """Names of the files in ``directory`` that match the regular expression."""
    import os
    import re
    rx = re.compile(pattern)
    return sorted(f for f in os.listdir(directory) if rx.match(f))


def filter_kwargs(func, kwargs: dict) -> dict:
    """The entries of ``kwargs`` that ``func`` accepts."""
    import inspect
    names = inspect.signature(func).parameters
    return {k: v for k, v in kwargs.items() if k in names}


class Block_Attention_Config:
    """Pattern plus partition in the pre-``BSA_Config`` form of the reference
    (search_algo/utils.py:151-178): ``CP`` ranks, ``ParD`` x ``ParD`` table of
    :class:`Block_Type`, ``cmap`` chunk -> rank. ``to_bsa_config`` gives the current form."""

    def __init__(self, CP: int, ParD: int, cmap, block_table):
        import numpy as np
        self.CP, self.ParD = CP, ParD
        self.cmap = np.asarray(cmap)
        self.block_table = block_table

    @classmethod
    def from_causal(cls, CP: int, ParD: int, cmap):
        import numpy as np
        from ..patterns.blocks import Block_Type
        table = np.empty((ParD, ParD), dtype=object)
        for i in range(ParD):
            for j in range(ParD):
                table[i, j] = Block_Type.FULL if j < i else Block_Type.CAUSAL if j == i else Block_Type.EMPTY
        return cls(CP, ParD, cmap, table)

    @property
    def block_table_value(self):
        return convert_block_table_to_value(self.block_table)

    def to_bsa_config(self):
        from ..patterns.blocks import BSA_Config, BSA_Repr
        return BSA_Config(None, None, {"bsa_repr": BSA_Repr(self.block_table_value, self.cmap), "CP": (self.CP, 1)})
