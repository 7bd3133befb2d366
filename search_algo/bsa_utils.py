"""Reference: search_algo/bsa_utils.py."""
from ultraattn_b200.patterns.named import create_bsa_block_table  # noqa: F401
from ultraattn_b200.planner.cost import convert_shape_config_to_str  # noqa: F401
from ultraattn_b200.utils.bsa_helpers import (bsa_is_causal, bsa_is_dense, bsa_is_full,  # noqa: F401
                                              bsa_is_square_full, bsa_repr_is_causal,
                                              bsa_repr_is_square_full,
                                              convert_intra_profile_key_to_exe_key_or_plan, get_b2f_suf_map,
                                              select_best_profile_comp_key, split_to_node_configs)
