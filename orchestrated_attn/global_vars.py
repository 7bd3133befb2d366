"""Reference: orchestrated_attn/global_vars.py:1-17."""
import torch

from ultraattn_b200.parallel.communicator import CommRegistry

FULL_DTYPE = torch.float32
ncclcomm_dict: CommRegistry = CommRegistry()      # communicators by tuple(ranks)
cpu_group_dict: dict = {}
streams: dict = {}
_vars: dict = {}


def get_global_var(name):
    return _vars.get(name)


def set_global_var(name, value):
    _vars[name] = value


def is_exist_global_var(name) -> bool:
    return name in _vars
