"""Reference: easy_context/__init__.py:1-48."""
from ultraattn_b200.models.glue import (apply_dist_flash_attn_monkey_patch_llama,  # noqa: F401
                                        apply_seq_parallel_monkey_patch,
                                        apply_unsloth_offloaded_gradient_checkpoint_monkey_patch,
                                        apply_zigzag_ring_attn_monkey_patch_llama,
                                        apply_zigzag_ring_attn_monkey_patch_mistral,
                                        prepare_dataloader, prepare_dist_flash_attn_inputs,
                                        prepare_seq_parallel_inputs, prepare_zigzag_ring_attn_inputs)
