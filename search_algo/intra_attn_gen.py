"""Reference: search_algo/intra_attn_gen.py."""
from ultraattn_b200.drivers.intra_attn_gen import generate, main  # noqa: F401

if __name__ == "__main__":
    import sys
    sys.exit(main())
