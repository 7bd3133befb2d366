"""Reference: easy_context/__init__.py:8-42."""
from ultraattn_b200.models.glue import (apply_seq_parallel_monkey_patch,  # noqa: F401
                                        prepare_seq_parallel_inputs)
