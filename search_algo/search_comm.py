"""Reference: search_algo/search_comm.py (its exhaustive search over tile-to-rank maps, a legacy
tool kept next to the integer program as an optimality oracle for small problems)."""
import numpy as np

from ultraattn_b200.patterns.blocks import BSA_Config
from ultraattn_b200.patterns.named import causal as _causal, full as _full
from ultraattn_b200.planner.allocate import brute_force_allocate
from ultraattn_b200.planner.cost import Dist_Attn_Config, Machine_Config, get_cc_optimal_schedule_from_table


def get_configs() -> Dist_Attn_Config:
    """A small dense causal problem (4 ranks, 4k tokens, 32 heads of 128), as in the reference."""
    cfg = BSA_Config(None, None, {"bsa_repr": _causal(1), "CP": (4, 1)})
    return Dist_Attn_Config.from_bsa_config(cfg, {"S": (4096, 4096), "Nh": (32, 32), "bs": 1, "D": 128}, hierarchy=1)


class Brute_Force_Search_Engine:
    """``search_optimal_schedules()`` -> the communication-optimal schedules of ``da_config`` found by
    trying every assignment (list with the best one first). ``fob`` selects the pass whose traffic
    is minimised. Only for a handful of tiles: the search is exponential."""

    def __init__(self, da_config: Dist_Attn_Config, m_config: Machine_Config = None, init_schedule_list=None,
                 fob: int = 0):
        self.da_config = da_config
        self.m_config = m_config or Machine_Config.b200_default()
        self.init_schedule_list = list(init_schedule_list or [])
        self.fob = fob
        self.tot_sp = int(np.prod(da_config.SP))

    def search_optimal_schedules(self) -> list:
        cfg = self.da_config.bsa_config
        if cfg is None:
            pat = _causal(1) if getattr(self.da_config, "causal", False) else _full(1)
            cfg = BSA_Config(None, None, {"bsa_repr": pat, "CP": tuple(self.da_config.SP[::-1])})
        al = brute_force_allocate(cfg, fob=self.fob, hierarchy=self.da_config.hierarchy)
        best = get_cc_optimal_schedule_from_table(self.da_config, self.m_config, al)
        best.comm_volume = float(al.comm_volume)
        return [best] + self.init_schedule_list
