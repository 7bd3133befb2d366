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
baseline wins: the ratio is printed as measured. ``--svg`` draws the speed-ups as a grouped bar chart without any plotting library (this image
has no matplotlib); ``--csv`` gives the same numbers to any plotting tool.

    python -m ultraattn_b200.drivers.report --bench-jsonl lines.jsonl [--svg out.svg] [--csv out.csv]

reads the JSON lines that ``drivers/bench_configs.py`` prints (one per configuration and path)
instead of a database and prints the same table: ``ring`` / ``zigzag`` are the baselines, the
``nccl`` path (the launch plan executed with NCCL messages) fills the "Node+Device Tile" column it
corresponds to, and "UltraAttn" is the best of the fused path and the NCCL path.
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


def sim_accuracy(profile: dict, tolerance: float = 0.3) -> dict:
    """How well the planner's predicted time (``sim_time``) matches the measured ``time`` over all
    entries that carry both: share of outliers beyond ``tolerance`` relative error (the reference
    uses 0.3 at the intra level and 0.5 at the inter level) and R^2 of predicted against measured
    (reference: plot/sim_accuracy.py:26-66)."""
    pairs = []
    for entry in profile.values():
        if isinstance(entry, dict) and "sim_time" in entry and "time" in entry:
            t, s = float(entry["time"]), float(entry["sim_time"])
            if t > 0 and s > 0:
                pairs.append((t, s))
    if not pairs:
        return {"n": 0, "outlier_pct": 0.0, "r2": float("nan"), "mean_abs_rel_err": float("nan")}
    rel = [abs(s - t) / t for t, s in pairs]
    mean_t = sum(t for t, _ in pairs) / len(pairs)
    ss_res = sum((t - s) ** 2 for t, s in pairs)
    ss_tot = sum((t - mean_t) ** 2 for t, _ in pairs)
    return {"n": len(pairs), "outlier_pct": 100.0 * sum(r > tolerance for r in rel) / len(pairs),
            "r2": 1.0 - ss_res / ss_tot if ss_tot > 0 else float("nan"),
            "mean_abs_rel_err": sum(rel) / len(rel)}


def e2e_rows(rows: list, n_layers: int, time_wo_attn: float) -> list:
    """End-to-end step time the way the reference's figure derives it (plot/e2e_pick.py:144-177):
    forward + backward attention time of one layer times ``n_layers`` plus a constant for
    everything else. Rows are joined on (CP, shape, pattern); returns one row per configuration
    with the baselines' and UltraAttn's step time and the speed-up over the best baseline."""
    by_cfg: dict = {}
    for r in rows:
        cfg = re.sub(r"^fob=\d_", "", r["key"])
        by_cfg.setdefault(cfg, {})[r["fob"]] = r
    out = []
    for cfg, fobs in sorted(by_cfg.items()):
        if "0" not in fobs:
            continue
        def total(col):
            ts = [fobs[f].get(col) for f in sorted(fobs)]
            return None if any(t is None for t in ts) else n_layers * sum(ts) + time_wo_attn
        row = {"key": cfg, "CP": fobs["0"]["CP"], "shape": fobs["0"]["shape"]}
        for col in ("ring", "zigzag", "stripe", "ultraattn"):
            row[col] = total(col)
        base = [row[c] for c in ("ring", "zigzag", "stripe") if row[c] is not None]
        if base and row["ultraattn"]:
            row["speedup_vs_best_baseline"] = min(base) / row["ultraattn"]
        out.append(row)
    return out


SYSTEMS = ("ring", "zigzag", "stripe", "ultraattn")


def scalability_rows(rows: list, mode: str = "strong") -> list:
    """Relative performance across rank counts, the way the reference's scalability figures
    normalise it. ``strong`` (plot/strong_scalability_training_pick.py:105-142): one pattern, pass
    and shape on several rank counts; every system's GPU time (seconds x ranks) is divided into the
    smallest GPU time of the group, so 1.0 marks the most efficient point and a flat line is perfect
    scaling. ``weak`` (plot/weak_scalability_training.py:136-180): the work per GPU is fixed, which
    for attention means S^2 / ranks (S doubles while the ranks quadruple); the smallest time of the
    group is divided by each time. Rows are the figure rows of :func:`build_rows` or
    :func:`rows_from_bench_lines`; groups seen on a single rank count are left out."""
    assert mode in ("strong", "weak"), mode
    groups: dict = {}
    for r in rows:
        cp = re.match(r"\((\d+), (\d+)\)", r.get("CP") or "")
        sm = re.search(r"S=\((\d+), ?(\d+)\)", r.get("shape") or "")
        if not cp or not sm:
            continue
        ranks, S = int(cp.group(1)) * int(cp.group(2)), int(sm.group(1))
        pm = re.search(r"_repr=(.*?)\}?$", r["key"])
        pattern = r.get("config") or (pm.group(1) if pm else r["key"])
        rest = re.sub(r"S=\(\d+, ?\d+\)_?", "", r["shape"])
        ident = (r.get("fob", ""), pattern, rest) + ((S,) if mode == "strong" else (S * S // ranks,))
        groups.setdefault(ident, []).append((ranks, S, r))
    out = []
    for ident, members in sorted(groups.items(), key=lambda kv: tuple(str(x) for x in kv[0])):
        if len({m[0] for m in members}) < 2:
            continue
        weight = (lambda n: n) if mode == "strong" else (lambda n: 1)
        costs = [r[c] * weight(n) for n, _, r in members for c in SYSTEMS if r.get(c)]
        if not costs:
            continue
        best = min(costs)
        for n, S, r in sorted(members, key=lambda m: m[0]):
            row = {"fob": ident[0], "pattern": ident[1] if len(str(ident[1])) <= 24 else str(ident[1])[:21] + "...",
                   "shape": r["shape"], "ranks": n, "S": S}
            for c in SYSTEMS:
                row[c] = best / (r[c] * weight(n)) if r.get(c) else None
            out.append(row)
    return out


def rows_from_bench_lines(lines) -> list:
    """Figure rows from ``bench_configs`` JSON lines (dicts or strings); times become seconds."""
    groups: dict = {}
    for ln in lines:
        rec = json.loads(ln) if isinstance(ln, str) else ln
        if "config" not in rec or "path" not in rec:
            continue
        groups.setdefault((rec["config"], rec["n_gpus"], rec["S"]), {})[rec["path"]] = rec["ms"] / 1e3
    rows = []
    for (config, n, S), t in sorted(groups.items(), key=lambda kv: (kv[0][1], kv[0][0])):
        ultra = [t[p] for p in ("fused", "nccl", "nccl-ilp") if p in t]
        base = {b: t[b] for b in ("ring", "zigzag", "stripe") if b in t}
        row = {"key": config, "config": config, "fob": "", "CP": f"({n}, 1)",
               "shape": f"S=({S},{S})_Nh=(32,32)_bs=1_D=128",
               "ring": t.get("ring"), "zigzag": t.get("zigzag"), "stripe": t.get("stripe"), "node_tile": None,
               "node_device_tile": t.get("nccl"), "kernel_tile": None, "fused": t.get("fused"),
               "ultraattn": min(ultra) if ultra else None}
        if row["ultraattn"] is not None:
            if row["ring"]:
                row["speedup_vs_ring"] = row["ring"] / row["ultraattn"]
            if base:
                row["speedup_vs_best_baseline"] = min(base.values()) / row["ultraattn"]
        rows.append(row)
    return rows


SERIES = [("ring", "#9e9e9e"), ("zigzag", "#64b5f6"), ("stripe", "#4db6ac"), ("node_tile", "#ffcc80"),
          ("node_device_tile", "#ffa726"), ("ultraattn", "#e53935")]


def bar_chart_svg(rows: list, title: str = "", baseline: str = "ring", width_per_group: int = 150,
                  height: int = 260) -> str:
    """Grouped bar chart of speed-ups over ``baseline`` (one group per configuration, one bar per
    variant that was measured), as a self-contained SVG string. The reference draws its figures
    with matplotlib (plot/*.py), which this image does not have; the chart carries the same
    content as its per-configuration panels: bars labelled with the speed-up, baselines in cool
    colours, the tiling ablations in orange, the full system in red."""
    groups = []
    for r in rows:
        base = r.get(baseline) or next((r[k] for k, _ in SERIES if r.get(k)), None)
        if not base:
            continue
        bars = [(k, colour, base / r[k]) for k, colour in SERIES if r.get(k)]
        label = f"{r['config']} CP={r.get('CP', '')}" if r.get("config") else f"fob={r.get('fob', '')} CP={r.get('CP', '')}"
        m = re.search(r"S=\((\d+)", r.get("shape", "") or "")
        if m:
            label += f" S={int(m.group(1)) // 1024}k"
        groups.append((label, bars))
    top = max([v for _, bars in groups for _, _, v in bars] + [1.0]) * 1.15
    left, bottom, head = 46, 46, 30
    plot_h = height - bottom - head
    total_w = left + max(1, len(groups)) * width_per_group + 10
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{total_w}" height="{height}" '
           f'font-family="sans-serif" font-size="10">',
           f'<rect width="{total_w}" height="{height}" fill="white"/>',
           f'<text x="{total_w / 2:.0f}" y="16" text-anchor="middle" font-size="12">{title}</text>']
    y_of = lambda v: head + plot_h * (1 - v / top)
    for tick in range(0, int(top) + 1):
        y = y_of(tick)
        out.append(f'<line x1="{left}" y1="{y:.1f}" x2="{total_w - 10}" y2="{y:.1f}" stroke="#ddd"/>')
        out.append(f'<text x="{left - 6}" y="{y + 3:.1f}" text-anchor="end">{tick}x</text>')
    for gi, (label, bars) in enumerate(groups):
        x0 = left + gi * width_per_group + 8
        bw = (width_per_group - 16) / max(1, len(bars))
        for bi, (name, colour, v) in enumerate(bars):
            x, y = x0 + bi * bw, y_of(v)
            out.append(f'<rect class="bar" x="{x:.1f}" y="{y:.1f}" width="{bw - 2:.1f}" '
                       f'height="{head + plot_h - y:.1f}" fill="{colour}"><title>{name}</title></rect>')
            out.append(f'<text x="{x + bw / 2 - 1:.1f}" y="{y - 2:.1f}" text-anchor="middle" font-size="8">{v:.2f}</text>')
        out.append(f'<text x="{x0 + (width_per_group - 16) / 2:.1f}" y="{height - bottom + 14}" '
                   f'text-anchor="middle">{label}</text>')
    lx = left
    for name, colour in SERIES:
        out.append(f'<rect x="{lx}" y="{height - 14}" width="9" height="9" fill="{colour}"/>')
        out.append(f'<text x="{lx + 12}" y="{height - 6}">{name}</text>')
        lx += 16 + 6 * len(name) + 10
    out.append("</svg>")
    return "\n".join(out)


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
    ap.add_argument("--db", default=None, help="database/<cluster>/<platform> directory")
    ap.add_argument("--bench-jsonl", default=None,
                    help="JSON lines printed by drivers/bench_configs.py, instead of a database")
    ap.add_argument("--level", default="inter", choices=["intra", "inter"])
    ap.add_argument("--csv", default=None)
    ap.add_argument("--svg", default=None, help="also draw the speed-ups over the ring baseline as a bar chart")
    ap.add_argument("--sim-accuracy", action="store_true",
                    help="print predicted-vs-measured statistics instead of the table")
    ap.add_argument("--scalability", default=None, choices=["strong", "weak"],
                    help="print relative performance across rank counts (strong: fixed shape, GPU time; weak: "
                         "fixed S^2 / ranks, time) instead of the table")
    ap.add_argument("--e2e-layers", type=int, default=0,
                    help="print end-to-end step times: layers x (fwd + bwd) + --e2e-const")
    ap.add_argument("--e2e-const", type=float, default=0.0, help="seconds per step outside attention")
    a = ap.parse_args(argv)
    if a.bench_jsonl:
        rows = rows_from_bench_lines(l for l in Path(a.bench_jsonl).read_text().splitlines() if l.startswith("{"))
        title = "measured paths, speed-up over the ring"
    else:
        if not a.db:
            ap.error("one of --db / --bench-jsonl is needed")
        path = Path(a.db) / f"{a.level}_bsa_exe_plans_profile.json"
        if not path.exists():
            print(f"no profile file {path}", file=sys.stderr)
            return 1
        profile = json.loads(path.read_text())
        if a.sim_accuracy:
            print(json.dumps(sim_accuracy(profile, 0.3 if a.level == "intra" else 0.5)))
            return 0
        rows = build_rows(profile)
        title = f"{a.level}-level plans, speed-up over ring"
    if a.scalability:
        cols = ["fob", "pattern", "shape", "ranks"] + list(SYSTEMS)
        print("| " + " | ".join(cols) + " |")
        print("|" + "---|" * len(cols))
        for r in scalability_rows(rows, a.scalability):
            print("| " + " | ".join(_fmt(r.get(c)) for c in cols) + " |")
        return 0
    if a.e2e_layers:
        cols = ["CP", "shape", "ring", "zigzag", "stripe", "ultraattn", "speedup_vs_best_baseline"]
        print("| " + " | ".join(cols) + " |")
        print("|" + "---|" * len(cols))
        for r in e2e_rows(rows, a.e2e_layers, a.e2e_const):
            print("| " + " | ".join(_fmt(r.get(c)) for c in cols) + " |")
        return 0
    cols = (["config"] if a.bench_jsonl else []) + [c for c in COLS if not (a.bench_jsonl and c == "fob")]
    if a.bench_jsonl:
        cols.insert(cols.index("ultraattn"), "fused")
    print("| " + " | ".join(cols) + " |")
    print("|" + "---|" * len(cols))
    for r in rows:
        print("| " + " | ".join(_fmt(r.get(c)) for c in cols) + " |")
    if a.svg:
        Path(a.svg).write_text(bar_chart_svg(rows, title=title))
    if a.csv:
        with open(a.csv, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=["key"] + COLS + (["fused"] if a.bench_jsonl else []), extrasaction="ignore")
            w.writeheader()
            w.writerows(rows)
    return 0


if __name__ == "__main__":
    sys.exit(main())
