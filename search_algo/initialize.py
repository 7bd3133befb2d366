"""Reference: search_algo/initialize.py."""
from ultraattn_b200.parallel.comm import (PROC_INFO, get_proc_info, initialize_distribution,  # noqa: F401
                                          initialize_prof_db, parse_slurm_tasks_per_node)
