"""Reference: search_algo/arguments.py."""
from ultraattn_b200.drivers.arguments import get_args, parse_args  # noqa: F401
