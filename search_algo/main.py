"""Reference: search_algo/main.py (which does not run there); one configuration end to end."""
from ultraattn_b200.drivers.main import main  # noqa: F401

if __name__ == "__main__":
    import sys
    sys.exit(main())
