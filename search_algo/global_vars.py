"""Module-level registry and constants (reference: search_algo/global_vars.py:1-22)."""
import enum


class TASK_STATUS(enum.Enum):
    """Markers in schedule tables: a tile that does not exist / one not yet assigned."""
    EMPTY = -1
    UNSETTLED = -2


BYTE_MULTPLE_UP = 1024
BYTE_MULTPLE_DOWN = 1000

_vars: dict = {}


def get_global_var(name):
    return _vars.get(name)


def set_global_var(name, value):
    _vars[name] = value


def is_exist_global_var(name) -> bool:
    return name in _vars
