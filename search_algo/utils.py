"""Block types and small utilities (reference: search_algo/utils.py)."""
from ultraattn_b200.patterns.blocks import Block_Comp_Volume, Block_Table_Type, Block_Type  # noqa: F401
from ultraattn_b200.drivers.arguments import parse_args  # noqa: F401
from ultraattn_b200.planner.cost import (convert_node_profile_data_to_comp_map,  # noqa: F401
                                         convert_profile_data_to_comm_map, convert_profile_data_to_map)
from ultraattn_b200.utils.misc import (Block_Attention_Config, all_wait_main_stream,  # noqa: F401
                                       closest_fraction, combine_list_to_0,
                                       convert_block_table_to_value, filter_kwargs,
                                       find_file_with_regex, get_factors, main_stream_wait_all)
from ultraattn_b200.utils.misc import (FinitePriorityQueue, calc_table_comp_relative_time,  # noqa: F401
                                       get_block_table_type, print_rank_0, report_memory,
                                       unique_list, use_all_cpus)
from ultraattn_b200.planner.cost import convert_throughput_to_B  # noqa: F401,E402


def calc_flops(mbs, S, Nh, D, fob=0, total_sparsity=1):
    """(model FLOPs, hardware FLOPs) with the reference's argument order (utils.py:92-103):
    ``fob`` 0 forward, 1 backward (2x / 2.5x the forward), 2 both; ``total_sparsity`` = computed share."""
    from ultraattn_b200.utils.misc import calc_flops as _calc
    if fob == 2:
        (a, b), (c, d) = _calc(mbs, S, Nh, D, False, 0, total_sparsity), _calc(mbs, S, Nh, D, False, 1, total_sparsity)
        return a + c, b + d
    return _calc(mbs, S, Nh, D, False, fob, total_sparsity)
