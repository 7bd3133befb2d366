"""One configuration, end to end: pattern -> allocation -> dependent graph -> (kernel tiling) ->
schedule -> predicted time, and, when launched on the ranks the configuration names, execution and
measurement.

    python -m ultraattn_b200.drivers.main --config configs/stride.yaml [--plan-only] [--fob 0|1|2]
                                          [--path fused|nccl] [--save-plan DIR] [--iters 3]
    torchrun --nproc-per-node 8 -m ultraattn_b200.drivers.main --config configs/stride.yaml

The YAML files and flags are the reference's (configs/*.yaml, search_algo/arguments.py:18-67); its
own ``main.py`` that was meant to consume them does not run. ``Parallel.SP = [inter, intra]`` gives
the number of nodes and of ranks per node; ``Experiment.lowering_mode`` picks the scheduler (ILP /
Flexflow), ``Experiment.transform_mode`` the kernel-tiling search (greedy / bf; "none" disables it).
Without a launcher (world size 1) or with ``--plan-only`` the plan is made and described but not
run. Output: one JSON line per pass.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

from .arguments import load_yaml, RunConfig


def describe(plan) -> dict:
    """Counts and predicted time of a launch plan."""
    kernels = plan.valid_kernels
    comp = [k for k in kernels if k.type == "comp"]
    comm = [k for k in kernels if k.type == "comm"]
    al = getattr(plan, "allocation", None)
    return {"comp_kernels": len(comp), "comm_kernels": len(comm),
            "fused_comp_kernels": sum(isinstance(k.key[2], tuple) or isinstance(k.key[3], tuple) for k in comp),
            "sim_time_ms": float(plan.end_time) * 1e3,
            "comm_volume_units": None if al is None else float(al.comm_volume),
            "comp_max_tiles": None if al is None else float(al.comp_max),
            "problems": plan.verify()}


def plan_config(cfg: RunConfig, fob: int, time_limit: float = 20.0):
    from ..planner import make_plan
    inter, intra = (cfg.SP if len(cfg.SP) == 2 else (1, cfg.SP[0]))
    return make_plan(pattern=cfg.pattern(), cp=intra, cp_inter=inter, seq_len=cfg.Sq, n_heads=cfg.Nhq,
                     head_dim=cfg.D, n_kv_heads=cfg.Nhkv, batch=cfg.BS, fob=fob,
                     plan_type=cfg.lowering_type if cfg.lowering_type in ("ILP", "Flexflow") else "Flexflow",
                     kernel_tile=cfg.transform_mode in ("greedy", "bf") and inter == 1, time_limit=time_limit)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, help="YAML file (configs/*.yaml)")
    ap.add_argument("--fob", type=int, default=2, choices=[0, 1, 2], help="0 forward, 1 backward, 2 both")
    ap.add_argument("--plan-only", action="store_true")
    ap.add_argument("--path", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--save-plan", default=None, metavar="DIR", help="write <plan name>.pkl / .json here")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--time-limit", type=float, default=20.0, help="seconds per solver call")
    a = ap.parse_args(argv)
    cfg = load_yaml(a.config)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    ranks_needed = cfg.SP[0] * cfg.SP[1]
    run = not a.plan_only and world == ranks_needed and world > 1
    fobs = [0, 1] if a.fob == 2 else [a.fob]
    if rank == 0:
        for fob in fobs:
            plan = plan_config(cfg, fob, a.time_limit)
            rec = {"config": os.path.basename(a.config), "fob": fob, "SP": list(cfg.SP), "S": cfg.Sq,
                   "pattern": cfg.pattern_type, "plan": plan.get_plan_name(), **describe(plan)}
            if a.save_plan:
                from ..planner.dense import write_plan
                rec["plan_file"] = write_plan(plan, a.save_plan)
            print(json.dumps(rec), flush=True)
    if not run:
        if rank == 0 and not a.plan_only and world != ranks_needed:
            print(json.dumps({"note": f"not run: the configuration needs {ranks_needed} ranks, this job has {world}"}))
        return 0
    import torch
    import torch.distributed as dist
    from ..runtime import ContextParallelAttention
    from .benchmark import benchmark_ops
    from ..utils.misc import calc_flops
    use_cuda = torch.cuda.is_available()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl" if use_cuda else "gloo", **({"device_id": dev} if use_cuda else {}))
    dtype = torch.bfloat16 if use_cuda else torch.float32
    rt = ContextParallelAttention(cfg.pattern(), cfg.Sq, cfg.Nhq, cfg.D, device=dev, n_kv_heads=cfg.Nhkv,
                                  batch=cfg.BS, path=a.path if use_cuda else "nccl", dtype=dtype,
                                  plan_time_limit=a.time_limit)
    g = torch.Generator().manual_seed(rank)
    S_loc = cfg.Sq // world
    mk = lambda h: torch.randn(cfg.BS, S_loc, h, cfg.D, generator=g).to(dtype).to(dev)
    q, k, v, d_o = mk(cfg.Nhq), mk(cfg.Nhkv), mk(cfg.Nhkv), mk(cfg.Nhq)
    o, lse = rt.forward(q, k, v)
    for fob in fobs:
        fn = (lambda: rt.forward(q, k, v)) if fob == 0 else (lambda: rt.backward(d_o, q, k, v, o, lse))
        t = benchmark_ops(fn, warmup=2, num_iter=a.iters, repeats=2, device=dev)
        _, hw = calc_flops(cfg.BS, (cfg.Sq, cfg.Skv), cfg.Nhq, cfg.D, False, fob, cfg.pattern().total_sparsity
                           if hasattr(cfg.pattern(), "total_sparsity") else 1.0)
        if rank == 0:
            print(json.dumps({"config": os.path.basename(a.config), "fob": fob, "path": rt.path, "n_ranks": world,
                              "time_ms": t * 1e3, "hfu_tflops_per_rank": hw / t / world / 1e12}), flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
