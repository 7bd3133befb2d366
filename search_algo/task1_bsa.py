"""Campaign steps 0-3 (reference: search_algo/task1_bsa.py). ``python search_algo/task1_bsa.py --exp-class X``"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ultraattn_b200.drivers.task1 import main  # noqa: E402,F401

if __name__ == "__main__":
    main()
