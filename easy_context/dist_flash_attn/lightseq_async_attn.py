"""Reference: easy_context/dist_flash_attn/lightseq_async_attn.py:437-464."""
from ultraattn_b200.parallel.lightseq import attention  # noqa: F401
