"""Reference: easy_context/dist_flash_attn/lightseq_async_attn.py:437-464."""
from ultraattn_b200.parallel.lightseq import (attention, maybe_reduce_dkv, maybe_repeat_kv_bwd,  # noqa: F401
                                              maybe_repeat_kv_fwd)
