"""Reference: search_algo/intra_attn_gen.py."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ultraattn_b200.drivers.intra_attn_gen import generate, main  # noqa: E402,F401

if __name__ == "__main__":
    sys.exit(main())
