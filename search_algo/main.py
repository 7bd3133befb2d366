"""Reference: search_algo/main.py (which does not run there); one configuration end to end."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ultraattn_b200.drivers.main import main  # noqa: E402,F401

if __name__ == "__main__":
    sys.exit(main())
