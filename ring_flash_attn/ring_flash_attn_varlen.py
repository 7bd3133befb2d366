"""Reference: ring_flash_attn/ring_flash_attn_varlen.py."""
from ultraattn_b200.parallel.ring import (RingFlashAttnVarlenFunc, ring_flash_attn_varlen_backward,  # noqa: F401
                                          ring_flash_attn_varlen_forward, ring_flash_attn_varlen_func,
                                          ring_flash_attn_varlen_kvpacked_func,
                                          ring_flash_attn_varlen_qkvpacked_func)
