"""Reference: head_parallel_attn/deepspeed_ulysses_attn.py:169."""
from ultraattn_b200.parallel.ring import deepspeed_ulysses_attn_func  # noqa: F401
