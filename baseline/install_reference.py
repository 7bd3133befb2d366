"""Put an unmodified copy of the reference's source tree under ``baseline/_ref``.

    python baseline/install_reference.py <path to a checkout of oliverYoung2001/UltraAttn>

The reference has neither ``setup.py`` nor ``pyproject.toml``, so ``pip install`` refuses it; it is a
tree of plain ``.py`` files that is used from ``sys.path``. Every file is copied byte for byte.
Figures, plots and bulky measurement logs (no code reads them on the benchmark path) are left out
to keep the copy small; the machine-profile files the reference's planner loads
(``prof_data/fit/time_*.json``, ``cb_8_*.log``, ``cb_16_*.log``) are kept.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SKIP_TOP = {"assets", "plot", "results_exp", ".git"}


def _ignore(src_root: str):
    def fn(directory: str, names: list[str]):
        rel = os.path.relpath(directory, src_root)
        out = []
        for n in names:
            if rel == "." and n in SKIP_TOP:
                out.append(n)
            elif rel.startswith("prof_data") and n.endswith(".log") and not n.startswith("cb_"):
                out.append(n)
            elif n == "__pycache__":
                out.append(n)
        return out
    return fn


def main() -> None:
    if len(sys.argv) != 2 or sys.argv[1].startswith("-"):
        raise SystemExit(__doc__)
    src = os.path.abspath(sys.argv[1])
    if not os.path.isdir(os.path.join(src, "search_algo")) or not os.path.isdir(os.path.join(src, "orchestrated_attn")):
        raise SystemExit(f"{src} is not a checkout of the reference (no search_algo/ and orchestrated_attn/ in it); "
                         "nothing was changed")
    dst = os.path.join(HERE, "_ref")
    tmp = dst + ".new"
    if os.path.isdir(tmp):
        shutil.rmtree(tmp)
    shutil.copytree(src, tmp, ignore=_ignore(src), symlinks=False)     # the old copy goes only once the new one is complete
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.rename(tmp, dst)
    for root, dirs, files in os.walk(dst):          # the source may be read-only; the copy is not
        for d in dirs:
            os.chmod(os.path.join(root, d), 0o755)
        for f in files:
            os.chmod(os.path.join(root, f), 0o644)
    print(f"copied {src} -> {dst}")


if __name__ == "__main__":
    main()
