"""Reference: search_algo/manual_schedules.py."""
from ultraattn_b200.planner.dense import (get_cc_optimal_schedule_table, get_kv_schedule_table,  # noqa: F401
                                          get_qo_schedule_table)
