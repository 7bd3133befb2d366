"""Reference: search_algo/dense_utils.py.

``get_block_schedule_table_for_full`` and ``create_plan_for_full`` accept the reference's argument
lists (``split_degrees, S_map, X, da_config`` / ``da_config, m_config, X, fob, first_dim``) as well
as this framework's short forms (``CP, X[, S_map]`` / ``CP, X, fob, ...``)."""
import numpy as np

from ultraattn_b200.planner import dense as _dense
from ultraattn_b200.planner.cost import CP2ParD_map  # noqa: F401
from ultraattn_b200.planner.dense import (create_plan_key_suffixes_for_full, get_full_ablation_suffix,  # noqa: F401
                                          split_dense_configs, write_plan)
from ultraattn_b200.planner.dense import ablation_dicts_for_full as create_ablation_configs_for_full  # noqa: F401


def get_block_schedule_table_for_full(split_degrees, S_map=None, X=None, da_config=None):
    """FULL attention on a Y x X grid of ranks: the rank of tile (k, l). Reference form returns
    ``[bs_split, Nh_split, Sq_split, Skv_split]``; the short form ``(CP, X[, S_map])`` the CP x CP table."""
    if np.isscalar(split_degrees):
        cp, x = int(split_degrees), int(S_map)           # (CP, X, S_map=None) positionally
        return _dense.get_block_schedule_table_for_full(cp, x, X)
    sq, skv, sb, sh = (int(v) for v in split_degrees)
    S_map = np.asarray(S_map)
    out = np.empty((sb, sh, sq, skv), dtype=np.int32)
    for b in range(sb):
        out[b, :] = _dense.get_block_schedule_table_for_full(sq, int(X), S_map[b])
    return out


def create_plan_for_full(*args, **kw):
    """Manual plan of FULL attention on a Y x X grid. Reference form: ``(da_config, m_config, X, fob,
    first_dim)``; short form: ``(CP, X, fob, m_config=None, shape_config=None, first_dim=0)``."""
    if args and np.isscalar(args[0]):
        return _dense.create_plan_for_full(*args, **kw)
    names = ("da_config", "m_config", "X", "fob", "first_dim")
    given = dict(zip(names, args), **kw)
    da = given["da_config"]
    return _dense.create_plan_for_full(da.hierarchy_sp, int(given["X"]), int(given["fob"]), given.get("m_config"),
                                       shape_config=da.shape_config, first_dim=int(given.get("first_dim", 0)))
