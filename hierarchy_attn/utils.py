"""Reference: hierarchy_attn/utils.py."""
from ultraattn_b200.parallel.hierarchy import InterComm, IntraComm, OverlappedInterComm, wait_recursively  # noqa: F401
from ultraattn_b200.parallel.ring import update_out_and_lse  # noqa: F401
from ultraattn_b200.utils.misc import print_rank_0  # noqa: F401
