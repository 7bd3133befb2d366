"""Reference: search_algo/bsa_config.py."""
from ultraattn_b200.patterns.blocks import BSA_Config, BSA_Repr  # noqa: F401
