"""Reference: ring_flash_attn/ring_flash_attn.py."""
from ultraattn_b200.parallel.ring import (RingFlashAttnFunc, ring_flash_attn_backward, ring_flash_attn_forward,  # noqa: F401
                                          ring_flash_attn_func, ring_flash_attn_kvpacked_func,
                                          ring_flash_attn_qkvpacked_func)
