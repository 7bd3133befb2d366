"""Tile-fusion table: how much faster is ONE kernel over x query blocks and y key blocks than
x * y kernels over single blocks?

    python -m ultraattn_b200.drivers.fusion_evaluate [--m-config DIR] [--nh 1,32] [--smin 256] [--smax 16384]

Reference: search_algo/fusion_evaluate.py:10-56 (prints the same table from its profile map). The
numbers decide which rectangle shapes the kernel-tiling pass tries first: on a GPU with 148 SMs a
small tile leaves most of the machine idle, so fusing pays until the fused kernel fills whole
waves. Times come from the measured kernel profile in ``--m-config`` (``time*.json`` written by
``cluster_profile --kernels``) where a shape was profiled, else from the analytic B200 model.
"""
from __future__ import annotations

import argparse
import math
import sys

from ..planner.cost import FlashAttn_Profile_Map, load_flash_profile

BATCH_DEGREES = [(1, 2), (2, 1), (1, 3), (3, 1), (1, 4), (2, 2), (4, 1), (2, 4), (4, 2), (4, 4)]


def fusion_table(pmap: FlashAttn_Profile_Map, nhs, s_values, D: int = 128, degrees=BATCH_DEGREES) -> list:
    """Rows ``{Nh, S, fob, bd, t_base, t_fused, speedup}``; speedup = x*y*t_base / t_fused."""
    rows = []
    for nh in nhs:
        for S in s_values:
            base = pmap.get_comp_time_from_map_key((S, 1, nh, D, "1/1", False))
            for bd in degrees:
                sq, skv = S * bd[0], S * bd[1]
                g = math.gcd(sq, skv)
                fused = pmap.get_comp_time_from_map_key((min(sq, skv), 1, nh, D, f"{sq // g}/{skv // g}", False))
                for fob in (0, 1):
                    rows.append({"Nh": nh, "S": S, "fob": fob, "bd": bd, "t_base": float(base[fob]),
                                 "t_fused": float(fused[fob]),
                                 "speedup": bd[0] * bd[1] * float(base[fob]) / float(fused[fob])})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m-config", default=None, help="directory with time*.json (measured kernel grid)")
    ap.add_argument("--nh", default="1,32")
    ap.add_argument("--smin", type=int, default=256)
    ap.add_argument("--smax", type=int, default=16384)
    a = ap.parse_args(argv)
    prof = {}
    if a.m_config:
        from pathlib import Path
        for f in sorted(Path(a.m_config).glob("time*.json")):
            prof.update(load_flash_profile(f))
    pmap = FlashAttn_Profile_Map(prof)
    s_values = [1 << p for p in range(int(math.log2(a.smin)), int(math.log2(a.smax)) + 1)]
    rows = fusion_table(pmap, [int(x) for x in a.nh.split(",")], s_values)
    print("| Nh | S | pass | x,y | base (us) | fused (us) | speed-up |")
    print("|---|---|---|---|---|---|---|")
    for r in rows:
        print(f"| {r['Nh']} | {r['S']} | {'fwd' if r['fob'] == 0 else 'bwd'} | {r['bd'][0]},{r['bd'][1]} | "
              f"{r['t_base'] * 1e6:.1f} | {r['t_fused'] * 1e6:.1f} | {r['speedup']:.2f} |")
    return 0


if __name__ == "__main__":
    sys.exit(main())
