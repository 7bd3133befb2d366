"""Module-level registry (reference: search_algo/global_vars.py:17-22)."""
_vars: dict = {}


def get_global_var(name):
    return _vars.get(name)


def set_global_var(name, value):
    _vars[name] = value
