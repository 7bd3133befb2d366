"""Reference: easy_context/zigzag_ring_attn/{prepare_inputs,monkey_patch}.py."""
from ultraattn_b200.models.glue import (apply_zigzag_ring_attn_monkey_patch_llama,  # noqa: F401
                                        apply_zigzag_ring_attn_monkey_patch_mistral,
                                        prepare_zigzag_ring_attn_inputs)
