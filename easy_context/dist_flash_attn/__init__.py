"""Reference: easy_context/dist_flash_attn/{prepare_input,monkey_patch}.py."""
from ultraattn_b200.models.glue import (apply_dist_flash_attn_monkey_patch_llama,  # noqa: F401
                                        prepare_dist_flash_attn_inputs)
