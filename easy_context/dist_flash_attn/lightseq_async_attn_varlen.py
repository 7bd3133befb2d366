"""Reference: easy_context/dist_flash_attn/lightseq_async_attn_varlen.py (same entry point as the
fixed-length module: ``attention(q, k, v, causal, sm_scale)``)."""
from ultraattn_b200.parallel.lightseq import (attention, maybe_reduce_dkv, maybe_repeat_kv_bwd,  # noqa: F401
                                              maybe_repeat_kv_fwd)
