"""Reference: ring_flash_attn/stripe_flash_attn.py."""
from ultraattn_b200.parallel.ring import (StripeFlashAttnFunc, stripe_flash_attn_backward, stripe_flash_attn_forward,  # noqa: F401
                                          stripe_flash_attn_func, stripe_flash_attn_kvpacked_func,
                                          stripe_flash_attn_qkvpacked_func)
