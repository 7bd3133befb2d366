"""Reference: search_algo/fusion_evaluate.py."""
from ultraattn_b200.drivers.fusion_evaluate import fusion_table, main  # noqa: F401

if __name__ == "__main__":
    import sys
    sys.exit(main())
