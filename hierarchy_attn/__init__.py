"""Reference: hierarchy_attn/hierarchy_attn_impl.py:415."""
from ultraattn_b200.parallel.hierarchy import hierarchy_attn_func  # noqa: F401
