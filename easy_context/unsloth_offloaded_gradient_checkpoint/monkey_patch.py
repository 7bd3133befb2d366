"""Reference: easy_context/unsloth_offloaded_gradient_checkpoint/monkey_patch.py."""
from ultraattn_b200.models.glue import OffloadedCheckpoint, apply_unsloth_offloaded_gradient_checkpoint_monkey_patch  # noqa: F401

Unsloth_Offloaded_Gradient_Checkpointer = OffloadedCheckpoint
