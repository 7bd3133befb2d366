"""Reference: easy_context/zigzag_ring_attn/monkey_patch.py."""
from ultraattn_b200.models.glue import (apply_zigzag_ring_attn_monkey_patch_llama,  # noqa: F401
                                        apply_zigzag_ring_attn_monkey_patch_mistral)
