"""Campaign step 4 (reference: search_algo/task2_bsa.py). ``python search_algo/task2_bsa.py --exp-class X``"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ultraattn_b200.drivers.task2 import (main, prepare_inter_comp_plans,  # noqa: E402,F401
                                          profile_all_inter_BSA, profile_all_inter_full,
                                          step4_profile_inter_bsa_exe_plans, step5_profile_baselines)

step4_profile_inter_full_exe_plans = step4_profile_inter_bsa_exe_plans   # one step covers both here

if __name__ == "__main__":
    main()
