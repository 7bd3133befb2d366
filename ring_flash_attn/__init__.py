"""Reference: ring_flash_attn/__init__.py:1-28."""
from ultraattn_b200.parallel.ring import (ring_flash_attn_func, ring_flash_attn_kvpacked_func,  # noqa: F401
                                          ring_flash_attn_qkvpacked_func, ring_flash_attn_varlen_func,
                                          ring_flash_attn_varlen_kvpacked_func,
                                          ring_flash_attn_varlen_qkvpacked_func, stripe_flash_attn_func,
                                          stripe_flash_attn_kvpacked_func,
                                          stripe_flash_attn_qkvpacked_func,
                                          zigzag_ring_flash_attn_func,
                                          zigzag_ring_flash_attn_kvpacked_func,
                                          zigzag_ring_flash_attn_qkvpacked_func,
                                          zigzag_ring_flash_attn_varlen_func,
                                          zigzag_ring_flash_attn_varlen_kvpacked_func,
                                          zigzag_ring_flash_attn_varlen_qkvpacked_func)
from ultraattn_b200.parallel.ring import (RingFlashAttnFunc, RingFlashAttnVarlenFunc, StripeFlashAttnFunc,  # noqa: F401
                                          ZigZagRingFlashAttnFunc, ZigZagRingFlashAttnVarlenFunc,
                                          ring_flash_attn_backward, ring_flash_attn_forward,
                                          stripe_flash_attn_backward, stripe_flash_attn_forward,
                                          zigzag_ring_flash_attn_backward, zigzag_ring_flash_attn_forward)
