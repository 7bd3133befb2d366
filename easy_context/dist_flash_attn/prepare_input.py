"""Reference: easy_context/dist_flash_attn/prepare_input.py."""
from ultraattn_b200.models.glue import prepare_dist_flash_attn_inputs  # noqa: F401
from ultraattn_b200.parallel.lightseq import extract_local  # noqa: F401
