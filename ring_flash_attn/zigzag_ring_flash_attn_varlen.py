"""Reference: ring_flash_attn/zigzag_ring_flash_attn_varlen.py."""
from ultraattn_b200.parallel.ring import (ZigZagRingFlashAttnVarlenFunc, get_half_index, get_half_lse,  # noqa: F401
                                          zigzag_ring_flash_attn_varlen_backward,
                                          zigzag_ring_flash_attn_varlen_forward,
                                          zigzag_ring_flash_attn_varlen_func,
                                          zigzag_ring_flash_attn_varlen_kvpacked_func,
                                          zigzag_ring_flash_attn_varlen_qkvpacked_func)
