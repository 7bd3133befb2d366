"""Reference: search_algo/manual_schedules.py.

The reference's functions take ``(split_degrees, S_map, causal, da_config)`` with ``split_degrees =
(Sq_split, Skv_split, bs_split, Nh_split)`` and ``S_map[bs, block]`` = owner of a block, and return
a table ``[bs_split, Nh_split, Sq_split, Skv_split]`` of ranks (-1: no tile). These adapters accept
that form and also this framework's short form ``(n, causal)``, which returns the ``n x n`` table."""
import numpy as np

from ultraattn_b200.planner import dense as _dense


def _lift(make, split_degrees, S_map, causal, **kw):
    if np.isscalar(split_degrees):                       # short form: (n, causal)
        return make(int(split_degrees), bool(S_map) if S_map is not None else False, **kw)
    sq, skv, sb, sh = (int(x) for x in split_degrees)
    assert sq == skv, "square partitions only"
    S_map = np.asarray(S_map)
    assert S_map.shape == (sb, min(sq, skv)), f"S_map must be [bs_split, blocks], got {S_map.shape}"
    base = make(sq, bool(causal), **kw)                  # ranks 0..n-1 as if block i lived on rank i
    out = np.full((sb, sh, sq, skv), -1, dtype=np.int32)
    for b in range(sb):
        mapped = np.where(base >= 0, S_map[b][np.clip(base, 0, None)], -1)
        out[b, :] = mapped
    return out


def get_qo_schedule_table(split_degrees, S_map=None, causal=False, da_config=None):
    """Every tile runs where its keys live (queries travel, outputs come back)."""
    return _lift(_dense.get_qo_schedule_table, split_degrees, S_map, causal)


def get_kv_schedule_table(split_degrees, S_map=None, causal=False, da_config=None):
    """Every tile runs where its queries live (keys / values travel: ring-like)."""
    return _lift(_dense.get_kv_schedule_table, split_degrees, S_map, causal)


def get_cc_optimal_schedule_table(split_degrees, S_map=None, causal=False, da_config=None, fob: int = 0,
                                  time_limit: float = 30.0):
    """Communication-optimal allocation of a dense n x n problem (solved; the reference keeps
    literal tables for the sizes it needs, manual_schedules.py:36-597)."""
    return _lift(_dense.get_cc_optimal_schedule_table, split_degrees, S_map, causal, fob=fob, time_limit=time_limit)
