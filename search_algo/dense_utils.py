"""Reference: search_algo/dense_utils.py."""
from ultraattn_b200.planner.cost import CP2ParD_map  # noqa: F401
from ultraattn_b200.planner.dense import (create_plan_for_full, create_plan_key_suffixes_for_full,  # noqa: F401
                                          get_block_schedule_table_for_full, get_full_ablation_suffix,
                                          split_dense_configs, write_plan)
from ultraattn_b200.planner.dense import ablation_dicts_for_full as create_ablation_configs_for_full  # noqa: F401
