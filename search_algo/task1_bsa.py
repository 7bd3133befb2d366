"""Campaign steps 0-3 (reference: search_algo/task1_bsa.py). ``python search_algo/task1_bsa.py --exp-class X``

The step functions are exported under the reference's names; their argument lists are this
framework's (a configuration space and the database instead of the reference's globals). The
per-configuration generators (``generate_*_execution_plans``) take the reference's lists."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ultraattn_b200.drivers.task1 import (generate_bsa_execution_plans, generate_general_full_execution_plans,  # noqa: E402,F401
                                          generate_inter_bsa_execution_plans, generate_intra_bsa_execution_plans,
                                          get_general_bsa_cc_optimal_schedule,
                                          main, profile_all_intra_BSA, profile_all_intra_full, step1_generate_intra_bsa_exe_plans,
                                          step1_generate_intra_full_exe_plans,
                                          step2_profile_intra_bsa_exe_plans,
                                          step2_profile_intra_full_exe_plans,
                                          step3_generate_inter_bsa_exe_plans,
                                          step3_generate_inter_dense_exe_plans)

get_general_bsa_cc_optimal_schedule_old = get_general_bsa_cc_optimal_schedule   # same result, cached

if __name__ == "__main__":
    main()
