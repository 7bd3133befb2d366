"""Reference: search_algo/fusion_evaluate.py."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ultraattn_b200.drivers.fusion_evaluate import fusion_table, main  # noqa: E402,F401

if __name__ == "__main__":
    sys.exit(main())
