"""Reference: easy_context/dist_flash_attn/monkey_patch.py. Its buffer bookkeeping around the
LightSeq kernels (global out / lse buffers, checkpoint functions that end with attention) has no
counterpart: the attention operators here are ordinary autograd functions that save their own
(O, lse), and ``models.llama`` checkpoints around them."""
from ultraattn_b200.models.glue import apply_dist_flash_attn_monkey_patch_llama  # noqa: F401
