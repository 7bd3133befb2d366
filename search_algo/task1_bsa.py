"""Campaign steps 0-3 (reference: search_algo/task1_bsa.py). ``python search_algo/task1_bsa.py --exp-class X``

The step functions are exported under the reference's names; their argument lists are this
framework's (a configuration space and the database instead of the reference's globals)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ultraattn_b200.drivers.task1 import (generate_bsa_execution_plans, get_general_bsa_cc_optimal_schedule,  # noqa: E402,F401
                                          main, step1_generate_intra_bsa_exe_plans,
                                          step1_generate_intra_full_exe_plans,
                                          step2_profile_intra_bsa_exe_plans,
                                          step2_profile_intra_full_exe_plans,
                                          step3_generate_inter_bsa_exe_plans)

if __name__ == "__main__":
    main()
