"""Reference: search_algo/database.py."""
from ultraattn_b200.plandb import Prof_DB  # noqa: F401
