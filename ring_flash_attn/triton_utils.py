"""Reference: ring_flash_attn/triton_utils.py (its two Triton kernels have no counterpart: the
attention kernels here read and write packed lse directly)."""
from ultraattn_b200.parallel.ring import flatten_varlen_lse, unflatten_varlen_lse  # noqa: F401
