"""Reference: search_algo/arguments.py."""
from ultraattn_b200.drivers.arguments import (get_args, parse_args, parse_config, parse_experiment_args,  # noqa: F401
                                              parse_parallel_args, parse_pattern_args, parse_shape_args,
                                              print_args, recursive_update)
