"""Predicted times of the fused runtime and of the ring baselines for the named configurations,
from the machine profile (kernel grid + link curve): what the cost model expects before anything
is measured, and the table to hold measurements against afterwards.

    python -m ultraattn_b200.drivers.predict [--cps 2,4,8] [--m-config DIR] [--configs strided512k,...]

Per configuration and rank count: forward / backward time of the fused runtime under the planner's
allocation (``planner.cost.fused_step_time``), of the K/V ring with contiguous shards that skips
excluded block pairs (``ring_step_time``), of the zigzag ring for dense causal attention, and the
ratios. The reference publishes such ratios as its headline (speed-up over ring attention,
its README.md:31-67); these are the model's values for one NVSwitch box of B200s.
"""
from __future__ import annotations

import argparse
import json
import sys

from .. import patterns as P
from ..planner.cost import Machine_Config, fused_step_time, ring_step_time

CONFIGS = {
    "causal128k": (lambda: P.causal(1), 131072, True),
    "strided512k": (lambda: P.strided(32, 4, 2), 524288, True),
    "gl512k": (lambda: P.global_local(32, 1, 2), 524288, True),
    "star512k": (lambda: P.star(32, 1), 524288, False),
    "streaming512k": (lambda: P.streaming(32, 1, 2), 524288, False),
}


def predict(name: str, cp: int, m_config=None, n_heads: int = 32, time_limit: float = 8.0) -> dict:
    from ..runtime.context_parallel import plan_allocation
    mk, S, train = CONFIGS[name]
    pat = mk()
    table, cmap = plan_allocation(pat, cp, 1, "ilp", time_limit=time_limit)
    f = fused_step_time(table, cmap, pat, S, n_heads, m_config=m_config)
    r = ring_step_time(pat, cp, S, n_heads, m_config=m_config)
    rec = {"config": name, "n_gpus": cp, "fused_fwd_ms": f["fwd_s"] * 1e3, "ring_fwd_ms": r["fwd_s"] * 1e3,
           "speedup_fwd": r["fwd_s"] / f["fwd_s"]}
    if train:
        rec.update(fused_bwd_ms=f["bwd_s"] * 1e3, ring_bwd_ms=r["bwd_s"] * 1e3, speedup_bwd=r["bwd_s"] / f["bwd_s"])
    if pat.check_causal() and pat.table.shape[0] == 1:
        z = ring_step_time(pat, cp, S, n_heads, m_config=m_config, kind="zigzag")
        rec.update(zigzag_fwd_ms=z["fwd_s"] * 1e3, zigzag_bwd_ms=z["bwd_s"] * 1e3)
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cps", default="2,4,8")
    ap.add_argument("--configs", default=",".join(CONFIGS))
    ap.add_argument("--m-config", default=None, help="directory with time*.json / cb_*.log (default: the shipped B200 profile)")
    a = ap.parse_args(argv)
    m = Machine_Config.from_dir(a.m_config) if a.m_config else None
    for name in a.configs.split(","):
        for cp in (int(c) for c in a.cps.split(",")):
            rec = predict(name, cp, m)
            print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in rec.items()}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
