"""Reference: ring_flash_attn/utils.py."""
from ultraattn_b200.parallel.ring import (flatten_varlen_lse, unflatten_varlen_lse,  # noqa: F401
                                          update_out_and_lse)
from ultraattn_b200.utils.misc import print_rank_0  # noqa: F401
from ultraattn_b200.parallel.comm import RingComm  # noqa: F401,E402

update_out_and_lse_old = update_out_and_lse      # the reference keeps an older body under this name
