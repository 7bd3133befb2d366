"""Solve the tile-allocation program for the named benchmark patterns ahead of time.

    python -m ultraattn_b200.drivers.precompute_allocations --out ultraattn_b200/data/allocations.json \\
           [--cp 2,4,8] [--time-limit 60] [--configs causal128k,strided512k,...]

A job on GPUs should not spend its first minute in a CPU solver, and a time-limited solver may
return different incumbents on different runs. The answers for the configurations of
``drivers/bench_configs.py`` on 2 / 4 / 8 ranks are therefore solved once with a long time limit and
shipped in ``ultraattn_b200/data/allocations.json``, where ``planner.allocate.solve_sparse_from_bsa``
finds them (any other pattern is solved on demand). The reference does the same with its plan
database (``*_bsa_allocation.json``, search_algo/task1_bsa.py:106-143) and with the literal tables
of search_algo/manual_schedules.py.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
from pathlib import Path


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--cp", default="2,4,8")
    ap.add_argument("--time-limit", type=float, default=60.0)
    ap.add_argument("--configs", default=None)
    ap.add_argument("--resolve", action="store_true",
                    help="solve again even where the shipped file has an answer (e.g. with a longer --time-limit)")
    a = ap.parse_args(argv)
    work = tempfile.mkdtemp(prefix="ua_alloc_")
    before = os.environ.get("UA_PLAN_CACHE")
    os.environ["UA_PLAN_CACHE"] = work
    from ..planner import allocate
    shipped = allocate._SHIPPED
    try:
        _run(a, work)
    finally:                                    # a caller in the same process keeps its own cache setting
        allocate._SHIPPED = shipped
        if before is None:
            os.environ.pop("UA_PLAN_CACHE", None)
        else:
            os.environ["UA_PLAN_CACHE"] = before


def _run(a, work: str) -> None:
    from ..patterns.blocks import BSA_Config
    from ..planner import allocate
    from ..planner.allocate import solve_sparse_from_bsa
    if a.resolve:
        allocate._SHIPPED = {}                  # the lookup then sees only what this run solves
    from ..runtime.context_parallel import plan_allocation
    from .bench_configs import CONFIGS
    names = a.configs.split(",") if a.configs else list(CONFIGS)
    for name in names:
        pattern = CONFIGS[name][0]()
        for cp in (int(x) for x in a.cp.split(",")):
            # what the runtimes ask for: backward weights with refinement, then the forward plan
            # of the NCCL executor at the partition the refinement settled on
            table, _ = plan_allocation(pattern, cp, 1, "ilp", a.time_limit)
            cfg = BSA_Config(None, None, {"bsa_repr": pattern, "CP": (cp, 1)})
            al = solve_sparse_from_bsa(cfg, fob=0, ParD=table.shape[0], time_limit=a.time_limit)
            print(f"{name} cp={cp}: ParD={table.shape[0]} fwd comm {al.comm_volume} ({al.status})", flush=True)
    out = Path(a.out)
    data = json.loads(out.read_text()) if out.exists() else {}
    solved = Path(work) / "allocations.json"
    fresh = json.loads(solved.read_text()) if solved.exists() else {}     # absent: every answer was shipped already
    data.update(fresh)
    out.write_text(json.dumps(data, indent=0, sort_keys=True))
    print(f"{len(data)} allocations in {out} ({len(fresh)} solved now)")


if __name__ == "__main__":
    main()
