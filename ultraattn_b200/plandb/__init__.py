from .db import (ABLATION_SUFFIXES, Prof_DB, allocation_key, full_plan_key, full_profile_suffix,
                 plan_key_prefix)
