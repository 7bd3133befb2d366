"""Reference: hierarchy_attn/hierarchy_attn_impl.py."""
from ultraattn_b200.parallel.hierarchy import (HierarchyAttnFunc, hierarchy_attn_backward, hierarchy_attn_forward,  # noqa: F401
                                               hierarchy_attn_func, intra_attn_forward,
                                               overlapped_hierarchy_attn_backward,
                                               overlapped_hierarchy_attn_forward)
