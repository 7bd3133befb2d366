"""Reference: search_algo/custom_sparse_pattern.py."""
from ultraattn_b200.utils.bsa_helpers import create_block_sparse_pattern  # noqa: F401
