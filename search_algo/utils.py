"""Block types and small utilities (reference: search_algo/utils.py)."""
from ultraattn_b200.patterns.blocks import Block_Comp_Volume, Block_Table_Type, Block_Type  # noqa: F401
from ultraattn_b200.planner.cost import (convert_profile_data_to_comm_map,  # noqa: F401
                                         convert_profile_data_to_map)
from ultraattn_b200.utils.misc import (FinitePriorityQueue, calc_flops, calc_table_comp_relative_time,  # noqa: F401
                                       get_block_table_type, print_rank_0, report_memory,
                                       unique_list, use_all_cpus)
