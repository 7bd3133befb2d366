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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--cp", default="2,4,8")
    ap.add_argument("--time-limit", type=float, default=60.0)
    ap.add_argument("--configs", default=None)
    a = ap.parse_args()
    work = tempfile.mkdtemp(prefix="ua_alloc_")
    os.environ["UA_PLAN_CACHE"] = work
    from ..patterns.blocks import BSA_Config
    from ..planner.allocate import solve_sparse_from_bsa
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
    data.update(json.loads((Path(work) / "allocations.json").read_text()))
    out.write_text(json.dumps(data, indent=0, sort_keys=True))
    print(f"{len(data)} allocations in {out}")


if __name__ == "__main__":
    main()
