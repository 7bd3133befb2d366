"""Campaign step 4: measure the inter-node plans (reference: search_algo/task2_bsa.py:38-387).

Each compute kernel of an inter-node plan is a whole intra-node plan; ``prepare_inter_comp_plans``
binds them (reference: search_algo/benchmark.py:21-83). On one node the inter level has a single
compute kernel, so the measured time of a single-node configuration is the time of its best
intra-node plan and is copied into the inter profile under the reference's key.
"""
from __future__ import annotations

import os

import torch.distributed as dist

from ..parallel.comm import initialize_distribution
from ..plandb import ABLATION_SUFFIXES, Prof_DB, plan_key_prefix
from ..utils.misc import print_rank_0
from .arguments import parse_args
from .exp_configs import step0_top_down_decompose


def prepare_inter_comp_plans(inter_plan, prof_db, da_config=None, node_id: int = 0) -> dict:
    """Attach to every inter-level compute kernel of ``node_id`` the intra-level plan that
    implements it; returns ``{(batch degrees, profile key): intra plan}`` so that kernels with the
    same workload share one plan object. A kernel-tile inter plan (``Fused_Execution_Plan``) has
    one compute kernel per node and gets ``kernel_execution_plan``."""
    from ..planner.schedule import Fused_Execution_Plan
    from ..utils.bsa_helpers import convert_intra_profile_key_to_exe_key_or_plan
    if da_config is not None and hasattr(inter_plan, "materialize") and (
            isinstance(inter_plan, Fused_Execution_Plan)
            or getattr(getattr(inter_plan, "d_graph", None), "seqlen_variable_graph", False)):
        inter_plan.materialize(da_config)
    plans: dict = {}

    def resolve(key, degrees):
        ident = (degrees, key)
        if ident not in plans:
            what = convert_intra_profile_key_to_exe_key_or_plan(key, prof_db)
            plans[ident] = prof_db.get_plan(what, 1) if isinstance(what, str) else what
            if plans[ident] is None:
                raise KeyError(f"no intra-level plan is stored under {what!r}")
        return plans[ident]

    if isinstance(inter_plan, Fused_Execution_Plan):
        key = getattr(inter_plan, "comp_map_key", None)
        if isinstance(key, str):
            inter_plan.kernel_execution_plan = resolve(key, (inter_plan.X, inter_plan.Y))
        return plans
    lists = inter_plan.gpu_kernel_lists
    kernels = lists.get(node_id, []) if isinstance(lists, dict) else lists[node_id]
    for k in kernels:
        if k.type == "comp" and isinstance(k.comp_map_key, str):
            r, c = k.key[2], k.key[3]
            degrees = (len(r) if isinstance(r, tuple) else 1, len(c) if isinstance(c, tuple) else 1)
            k.execution_plan = resolve(k.comp_map_key, degrees)
    return plans


def _profile_inter_one(fob, cfg, shape, prof_db) -> list:
    """Inter-level profiles of one (pass, pattern, shape) on a single node: the inter plan has one
    compute kernel, so each ablation's time is that of its intra plan (for FULL attention, of the
    best grid the ablation may use). Returns the keys written."""
    written = []
    if cfg.CP[1] != 1:
        return written          # several nodes: measured by running the inter plan on all of them
    prefix = plan_key_prefix(fob, cfg.CP, shape, cfg)
    for suf in ABLATION_SUFFIXES:
        intra = prof_db.get_profile(prefix + suf, 1)
        if intra is None and cfg.bsa_repr.check_full():
            # FULL attention is measured per (Y, X) grid: an ablation level stands for
            # the best grid it may use (reference: search_algo/bsa_utils.py:53-70)
            from ..utils.bsa_helpers import get_b2f_suf_map
            cands = [prof_db.get_profile(prefix + s, 1) for s in get_b2f_suf_map(cfg.CP[0])[suf]]
            cands = [c for c in cands if c is not None]
            intra = min(cands, key=lambda c: float(c["time"])) if cands else None
        if intra is not None:
            prof_db.put_profile(prefix + suf, intra["hfu"], float(intra["time"]), float(intra["sim_time"]), 0)
            written.append(prefix + suf)
    return written


def step4_profile_inter_bsa_exe_plans(space, prof_db, world: int) -> None:
    if dist.is_initialized() and dist.get_rank() != 0:
        return
    for fob in space.fobs:
        for cfg in space.inter_bsa_configs:
            if cfg.CP[0] * cfg.CP[1] != world:
                continue
            for shape in space.shape_configs(world):
                _profile_inter_one(fob, cfg, shape, prof_db)


def profile_all_inter_BSA(args, exp_config, da_config, ncclcomm_global=None, gloo_global_group=None,
                          tensor_buf=None, prof_db=None) -> list:
    """One configuration of step 4 under the reference's argument list (search_algo/task2_bsa.py:
    38-147); rank 0 writes, the others return at once. Communicator, control group and buffer are
    accepted and unused."""
    assert prof_db is not None, "profile_all_inter_BSA needs the plan database"
    if dist.is_initialized() and dist.get_rank() != 0:
        return []
    return _profile_inter_one(exp_config.fob, da_config.bsa_config, da_config.shape_config, prof_db)


profile_all_inter_full = profile_all_inter_BSA      # FULL attention takes the same route (best grid per ablation)


def step5_profile_baselines(space, prof_db, device, world: int, iters: int = 2) -> list:
    """Measure the ring-family baselines of every configuration that fits the ranks running now and
    store them beside the plans' profiles under the suffixes the figure tables read (``_ring``,
    ``_zigzag``, ``_stripe``; reference: plot/common.py:48-53, whose baseline rows come from a
    separate repository). Dense causal gets all three, dense full the ring; block-sparse patterns
    get the ring that skips the block pairs the pattern leaves out. Returns the keys written."""
    import torch
    from ..parallel import ring as R
    from ..utils.bsa_helpers import bsa_is_causal, bsa_is_full
    from ..utils.misc import calc_flops
    from .benchmark import benchmark_ops
    written = []
    rank = dist.get_rank() if dist.is_initialized() else 0
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    for fob in space.fobs:
        for cfg in space.inter_bsa_configs:
            if cfg.CP[0] * cfg.CP[1] != world:
                continue
            kinds = ["ring", "zigzag", "stripe"] if bsa_is_causal(cfg) else ["ring"]
            dense = bsa_is_causal(cfg) or bsa_is_full(cfg)
            types = None
            if not dense:
                import math
                n = cfg.bsa_repr.table.shape[0]
                types = cfg.bsa_repr.refined(n * world // math.gcd(n, world))
            for shape in space.shape_configs(world):
                prefix = plan_key_prefix(fob, cfg.CP, shape, cfg)
                S_loc = shape["S"][0] // world
                if types is not None and S_loc % (types.shape[0] // world):
                    continue
                g = torch.Generator().manual_seed(rank)
                mk = lambda h: torch.randn(shape["bs"], S_loc, h, shape["D"], generator=g).to(dtype).to(device)
                q, k, v, d_o = mk(shape["Nh"][0]), mk(shape["Nh"][1]), mk(shape["Nh"][1]), mk(shape["Nh"][0])
                for kind in kinds:
                    key = prefix + "_" + kind
                    if prof_db.get_profile(key, 0) is not None:
                        continue
                    causal = bsa_is_causal(cfg)
                    o, lse = R.ring_forward(q, k, v, None, kind, causal, block_types=types)
                    if fob == 0:
                        fn = lambda: R.ring_forward(q, k, v, None, kind, causal, block_types=types)
                    else:
                        fn = lambda: R.ring_backward(d_o, q, k, v, o, lse, None, kind, causal, block_types=types)
                    t = benchmark_ops(fn, 2, iters, 2, device)
                    _, hw = calc_flops(shape["bs"], shape["S"], shape["Nh"][0], shape["D"], False, fob,
                                       cfg.total_sparsity)
                    from ..planner.cost import ring_step_time
                    model = ring_step_time(cfg.bsa_repr, world, shape["S"][0], shape["Nh"][0], shape["D"],
                                           prof_db.m_config, shape["Nh"][1], shape["bs"],
                                           "ring" if kind == "ring" else "zigzag")
                    if rank == 0:
                        prof_db.put_profile(key, hw / t / world / 1e12, t, model["fwd_s" if fob == 0 else "bwd_s"], 0)
                    written.append(key)
                    if dist.is_initialized():
                        dist.barrier()
    return written


def main(argv=None) -> None:
    args = parse_args(argv)
    info = initialize_distribution()
    prof_db = Prof_DB(os.environ.get("CLUSTER_NAME"), os.environ.get("PLATFORM"))
    space = step0_top_down_decompose(args.exp_class or "bsa_train", max_intra=info["tasks_per_node"],
                                     max_nodes=info["node_num"], quick=bool(args.extra.get("quick")))
    step4_profile_inter_bsa_exe_plans(space, prof_db, info["world_size"])
    import torch
    device = torch.device("cuda", info["local_rank"]) if torch.cuda.is_available() else torch.device("cpu")
    if info["world_size"] > 1:
        step5_profile_baselines(space, prof_db, device, info["world_size"])
    print_rank_0("task2 done")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
