"""Reference: orchestrated_attn/global_vars.py:1-17."""
import torch

FULL_DTYPE = torch.float32
ncclcomm_dict: dict = {}
cpu_group_dict: dict = {}
streams: dict = {}
_vars: dict = {}


def get_global_var(name):
    return _vars.get(name)


def set_global_var(name, value):
    _vars[name] = value
