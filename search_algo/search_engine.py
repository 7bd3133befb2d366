"""Reference: search_algo/search_engine.py."""
from ultraattn_b200.planner.cost import (Comm_Profile_Map, Comp_Profile_Map, Dist_Attn_Config,  # noqa: F401
                                         Dist_Attn_Schedule, Evaluation_Configs,
                                         FlashAttn_Profile_Map, Inter_Comp_Profile_Map,
                                         Machine_Config, get_cc_optimal_schedule_from_table)
from ultraattn_b200.planner.cost import create_schedule  # noqa: F401,E402
