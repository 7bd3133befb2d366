"""Reference: head_parallel_attn/deepspeed_ulysses_attn.py."""
from ultraattn_b200.parallel.ring import (DeepSpeedUlyssesAttnFunc, deepspeed_ulysses_attn_backward,  # noqa: F401
                                          deepspeed_ulysses_attn_forward, deepspeed_ulysses_attn_func)
