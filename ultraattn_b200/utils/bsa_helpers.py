"""Pattern predicates, node-level decomposition, ablation-suffix maps and the parametric pattern
generator (reference: search_algo/bsa_utils.py:10-113, search_algo/custom_sparse_pattern.py:5-89)."""
from __future__ import annotations

import numpy as np

from ..patterns import named
from ..patterns.blocks import BSA_Config, BSA_Repr, CAUSAL, FULL
from .misc import unique_list


def bsa_repr_is_square_full(r: BSA_Repr) -> bool:
    return r.table.shape == (1, 1) and r.table[0, 0] == FULL


def bsa_repr_is_causal(r: BSA_Repr) -> bool:
    return r.table.shape == (1, 1) and r.table[0, 0] == CAUSAL


def bsa_is_square_full(c: BSA_Config) -> bool: return bsa_repr_is_square_full(c.bsa_repr)
def bsa_is_full(c: BSA_Config) -> bool: return c.bsa_repr.check_full()
def bsa_is_causal(c: BSA_Config) -> bool: return bsa_repr_is_causal(c.bsa_repr)
def bsa_is_dense(c: BSA_Config) -> bool: return bsa_is_causal(c) or bsa_is_full(c)


def split_to_node_configs(global_cfg: BSA_Config) -> list:
    """Distinct per-node sub-patterns of a global pattern, each with ``CP = (intra, 1)``."""
    reprs = global_cfg.bsa_repr.split_n(global_cfg.CP[1])
    return unique_list([BSA_Config(None, None, {"bsa_repr": r, "CP": (global_cfg.CP[0], 1)}) for r in reprs])


_b2f_cache: dict = {}


def get_b2f_suf_map(CP: int) -> dict:
    """Ablation suffix of a block-sparse plan -> the FULL-attention (Y, X) suffixes whose measured
    times may implement its FULL node tiles."""
    if CP not in _b2f_cache:
        xys = [(x, CP // x) for x in range(1, CP + 1) if CP % x == 0]
        wo = [f"_ablation=(w/o_kernel_tile,Y={y},X={x},dim=0)" for x, y in xys]
        w = [f"_ablation=(w_kernel_tile,Y={y},X={x},dim=0)" for x, y in xys]
        _b2f_cache[CP] = {
            "_ablation=(w/o_gpu_tile,w/o_kernel_tile,Flexflow)": [f"_ablation=(w/o_kernel_tile,Y={CP},X=1,dim=0)"],
            "_ablation=(w/o_kernel_tile,Flexflow)": wo,
            "_ablation=(w_kernel_tile,Flexflow)": wo + w,
            "_ablation=(w/o_kernel_tile,ILP)": wo,
            "_ablation=(w_kernel_tile,ILP)": wo + w,
        }
    return _b2f_cache[CP]


def select_best_profile_comp_key(key_prefix: str, suffixes, comp_profile_map, fob: int,
                                 fault_tolerance_func=lambda s: True) -> str:
    best, best_t = None, float("inf")
    for suf in suffixes:
        key = f"{key_prefix}{suf}"
        try:
            t = comp_profile_map.get_comp_time_from_map_key(key)[fob]
        except KeyError:
            if not fault_tolerance_func(suf):
                raise
            continue
        if t < best_t:
            best, best_t = key, t
    if best is None:
        raise KeyError(f"no profiled key with prefix {key_prefix}")
    return best


def convert_intra_profile_key_to_exe_key_or_plan(comp_map_key: str, prof_db=None):
    """What implements an inter-level compute kernel whose cost was looked up under
    ``comp_map_key`` (reference: search_algo/bsa_utils.py:27-51). Block-sparse keys name their plan
    directly. FULL node tiles are profiled per (Y, X) grid: the variant without kernel tile maps to
    the shape-free plan key ``..._shape_config=full_ablation=(Y=..,X=..,dim=0)``, the variant with
    kernel tile to a ``Fused_Execution_Plan(Y, X)`` built on the spot."""
    import re
    if "Y=" not in comp_map_key:
        return comp_map_key
    if "w/o_kernel_tile" in comp_map_key:
        return re.sub(r"shape_config=.*_ablation=\(w/o_kernel_tile,", "shape_config=full_ablation=(", comp_map_key)
    if "w_kernel_tile" in comp_map_key:
        m = re.match(r"^fob=(\d+)_.*Y=(\d+),X=(\d+),", comp_map_key)
        if m is None:
            raise ValueError(f"cannot read (fob, Y, X) from {comp_map_key!r}")
        from ..planner.schedule import Fused_Execution_Plan
        fob, Y, X = (int(g) for g in m.groups())
        return Fused_Execution_Plan(Y, X, None, fob=fob, m_config=getattr(prof_db, "m_config", None))
    raise ValueError(f"unsupported profile key {comp_map_key!r}")


def create_block_sparse_pattern(CP: int, ParD: int, pattern_type: str, pattern_sparsity: float,
                                local_blocks=(1, 1), global_blocks=(0, 0), replicate: int = 1) -> BSA_Repr:
    """Parametric generator: ``star`` / ``stream`` = sink columns + causal local band sized from the
    sparsity; ``local_global`` = global rows/cols + symmetric band, replicated block-diagonally;
    ``stride`` = causal strided pattern (the reference leaves this branch empty)."""
    n = ParD
    if pattern_type == "star":
        return named.star(n, max(1, global_blocks[0] or 1))
    if pattern_type == "stream":
        return named.streaming(n, max(1, global_blocks[0] or 1), max(1, local_blocks[0]))
    if pattern_type in ("local_global", "lg"):
        sub = n // replicate
        t = np.zeros((n, n), dtype=np.int8)
        for r in range(replicate):
            blk = np.zeros((sub, sub), dtype=np.int8)
            for i in range(sub):
                for j in range(sub):
                    if -local_blocks[0] < j - i < local_blocks[1] or i == j:
                        blk[i, j] = FULL
            g = global_blocks[0]
            blk[:g, :] = FULL
            blk[:, :g] = FULL
            t[r * sub:(r + 1) * sub, r * sub:(r + 1) * sub] = blk
        return BSA_Repr(t)
    if pattern_type == "stride":
        stride = max(2, int(round(1.0 / max(pattern_sparsity, 1e-6) ** 0.5)))
        return named.strided(n, stride, max(1, local_blocks[0]))
    raise ValueError(f"unknown pattern_type {pattern_type!r}")
