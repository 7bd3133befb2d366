"""Reference: ring_flash_attn/zigzag_ring_flash_attn.py."""
from ultraattn_b200.parallel.ring import (ZigZagRingFlashAttnFunc, zigzag_ring_flash_attn_backward,  # noqa: F401
                                          zigzag_ring_flash_attn_forward, zigzag_ring_flash_attn_func,
                                          zigzag_ring_flash_attn_kvpacked_func,
                                          zigzag_ring_flash_attn_qkvpacked_func)

zigzag_ring_flash_attn_forward_old = zigzag_ring_flash_attn_forward     # the reference keeps an older body under this name
