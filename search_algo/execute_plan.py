"""Reference: search_algo/execute_plan.py."""
from ultraattn_b200.planner.schedule import (Execution_Plan, Fused_Execution_Plan,  # noqa: F401
                                             create_one_node_exe_plan)
