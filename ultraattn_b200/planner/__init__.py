from .allocate import (Allocation, brute_force_allocate, comm_volumes, comp_volumes,
                       naive_allocate_strategy, solve_sparse_from_bsa, tile_volumes)
from .cost import (Comm_Profile_Map, Dist_Attn_Config, Dist_Attn_Schedule, Evaluation_Configs,
                   FlashAttn_Profile_Map, Inter_Comp_Profile_Map, Machine_Config,
                   convert_shape_config_to_str, get_cc_optimal_schedule_from_table)
from .fuse import Comp_Fusion_Substitution, Comp_Fusion_Transformation, Graph_Transformation_Engine
from .graph import Comm_Kernel, Comp_Kernel, Cuda_Kernel, Dependent_Graph
from .schedule import Execution_Plan, Fused_Execution_Plan, create_one_node_exe_plan
from .pipeline import make_plan, make_plan_collective
