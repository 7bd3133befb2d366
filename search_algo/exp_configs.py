"""Reference: search_algo/exp_configs.py."""
from ultraattn_b200.drivers.exp_configs import (get_bsa_infer_configs, get_bsa_train_configs,  # noqa: F401
                                                get_dense_train_configs, get_exp_configs,
                                                get_exp_infer_configs, get_exp_train_configs,
                                                step0_top_down_decompose)
