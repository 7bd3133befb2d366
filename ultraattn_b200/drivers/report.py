"""Turn a profile database into the tables behind the reference's figures (text / CSV).

    python -m ultraattn_b200.drivers.report --db database/<cluster>/<platform> [--level intra|inter]
                                            [--csv out.csv]

Reads ``<level>_bsa_exe_plans_profile.json`` (key -> {"hfu", "time", "sim_time"}), groups the keys
by their prefix (everything before ``_ablation=`` or a baseline suffix) and prints, per
configuration, the measured time of every variant and the speed-up of the best UltraAttn variant
over the ring baseline and over the best baseline. The label mapping is the reference's
(plot/da_bsa_training_pick.py:138-155, plot/common.py:48-53): "Node Tile" =
``(w/o_gpu_tile,w/o_kernel_tile,Flexflow)``, "Node+Device Tile" = ``(w/o_kernel_tile,Flexflow)``,
"+Kernel Tile" = min with ``(w_kernel_tile,Flexflow)``, "UltraAttn" = min over the four
``w/o|w_kernel_tile`` x ``Flexflow|ILP`` variants; baselines carry the suffixes ``_ring``,
``_zigzag``, ``_stripe``. Unlike the reference's plot scripts nothing is substituted when a
baseline wins: the ratio is printed as measured. Figures need matplotlib, which this image does
not ship; ``--csv`` gives the same numbers to any plotting tool.
"""
from __future__ import annotations

import argparse
import csv
import json
import re
import sys
from pathlib import Path

BASELINES = ("_ring", "_zigzag", "_stripe")
ULTRA = ("_ablation=(w/o_kernel_tile,Flexflow)", "_ablation=(w_kernel_tile,Flexflow)",
         "_ablation=(w/o_kernel_tile,ILP)", "_ablation=(w_kernel_tile,ILP)")
NODE_TILE = "_ablation=(w/o_gpu_tile,w/o_kernel_tile,Flexflow)"


def split_key(key: str):
    """(prefix, suffix) of a profile key."""
    i = key.find("_ablation=")
    if i >= 0:
        return key[:i], key[i:]
    for b in BASELINES + ("_ultra",):
        if key.endswith(b):
            return key[:-len(b)], b
    return key, ""


def _time(entry) -> float:
    return float(entry["time"]) if isinstance(entry, dict) else float(entry)


def build_rows(profile: dict) -> list:
    groups: dict = {}
    for key, entry in profile.items():
        prefix, suffix = split_key(key)
        groups.setdefault(prefix, {})[suffix] = _time(entry)
    rows = []
    for prefix, variants in sorted(groups.items()):
        m = re.match(r"fob=(\d)_CP=\((\d+), (\d+)\)_shape_config=\{?(.*?)\}?(_bsa_config=.*)?$", prefix)
        ultra = [variants[s] for s in ULTRA if s in variants]
        full = {s: t for s, t in variants.items() if "Y=" in s}
        if full:
            ultra += list(full.values())
        base = {b: variants[b] for b in BASELINES if b in variants}
        row = {"key": prefix, "fob": m.group(1) if m else "", "CP": f"({m.group(2)}, {m.group(3)})" if m else "",
               "shape": m.group(4) if m else "",
               "ring": base.get("_ring"), "zigzag": base.get("_zigzag"), "stripe": base.get("_stripe"),
               "node_tile": variants.get(NODE_TILE),
               "node_device_tile": variants.get(ULTRA[0]),
               "kernel_tile": min((variants[s] for s in ULTRA[:2] if s in variants), default=None),
               "ultraattn": min(ultra) if ultra else None}
        if row["ultraattn"] is not None:
            if row["ring"]:
                row["speedup_vs_ring"] = row["ring"] / row["ultraattn"]
            if base:
                row["speedup_vs_best_baseline"] = min(base.values()) / row["ultraattn"]
        rows.append(row)
    return rows


COLS = ["fob", "CP", "shape", "ring", "zigzag", "stripe", "node_tile", "node_device_tile", "kernel_tile",
        "ultraattn", "speedup_vs_ring", "speedup_vs_best_baseline"]


def _fmt(v):
    if v is None:
        return "-"
    if isinstance(v, float):
        return f"{v:.3e}" if v < 1e-2 or v >= 1e3 else f"{v:.3f}"
    return str(v)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--db", required=True, help="database/<cluster>/<platform> directory")
    ap.add_argument("--level", default="inter", choices=["intra", "inter"])
    ap.add_argument("--csv", default=None)
    a = ap.parse_args(argv)
    path = Path(a.db) / f"{a.level}_bsa_exe_plans_profile.json"
    if not path.exists():
        print(f"no profile file {path}", file=sys.stderr)
        return 1
    rows = build_rows(json.loads(path.read_text()))
    print("| " + " | ".join(COLS) + " |")
    print("|" + "---|" * len(COLS))
    for r in rows:
        print("| " + " | ".join(_fmt(r.get(c)) for c in COLS) + " |")
    if a.csv:
        with open(a.csv, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=["key"] + COLS, extrasaction="ignore")
            w.writeheader()
            w.writerows(rows)
    return 0


if __name__ == "__main__":
    sys.exit(main())
