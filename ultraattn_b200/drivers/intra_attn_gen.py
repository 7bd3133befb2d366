"""Write the manual Y x X plans of FULL attention for one CP degree into the plan database.

    python -m ultraattn_b200.drivers.intra_attn_gen --cp 8 [--fobs 0,1]

Reference: search_algo/intra_attn_gen.py:40-64 (pickles one plan per factorisation X * Y = CP and
pass into ``execution_plans/<cluster>/<platform>/``). Here the plans go into the profile database
under the shape-free keys ``fob=..._CP=(cp, 1)_shape_config=full_ablation=(Y=..,X=..,dim=0)`` that
the campaign and the inter-level planner look up, so they need not be generated twice.
"""
from __future__ import annotations

import argparse
import os
import sys

from ..plandb import Prof_DB, full_plan_key
from ..planner.dense import create_ablation_configs_for_full, create_plan_for_full


def full_plan_keys(cp: int, fobs=(0, 1), hierarchy: int = 1) -> list:
    CP = (cp, 1) if hierarchy else (1, cp)
    return [full_plan_key(fob, CP, Y, X) for fob in fobs for Y, X in create_ablation_configs_for_full(cp)]


def generate(prof_db: Prof_DB, cp: int, fobs=(0, 1), hierarchy: int = 1) -> list:
    """Store every missing (Y, X) plan of one level (1: the ``cp`` ranks of a node, 0: ``cp`` nodes);
    returns the keys that are present afterwards."""
    keys = []
    CP = (cp, 1) if hierarchy else (1, cp)
    for fob in fobs:
        for Y, X in create_ablation_configs_for_full(cp):
            key = full_plan_key(fob, CP, Y, X)
            if not prof_db.has_plan(key, hierarchy):
                prof_db.put_plan(key, create_plan_for_full(cp, X, fob, prof_db.m_config, hierarchy=hierarchy),
                                 hierarchy)
            keys.append(key)
    return keys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cp", type=int, default=8)
    ap.add_argument("--fobs", default="0,1")
    a = ap.parse_args(argv)
    db = Prof_DB(os.environ.get("CLUSTER_NAME"), os.environ.get("PLATFORM"))
    for k in generate(db, a.cp, [int(x) for x in a.fobs.split(",")]):
        print(k)
    return 0


if __name__ == "__main__":
    sys.exit(main())
