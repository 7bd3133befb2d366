"""Campaign steps 0-3: decompose -> intra-node plans -> profile them -> inter-node plans.

Reference pipeline: search_algo/task1_bsa.py:901-949 (``main``), :581 (step 1), :699 (step 2),
:781 (step 3). Everything is keyed in the plan database, so an interrupted campaign resumes where
it stopped ("Bypassed" entries are skipped).

    torchrun --nproc-per-node 8 search_algo/task1_bsa.py --exp-class bsa_train [--quick]
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..parallel.comm import initialize_distribution
from ..plandb import ABLATION_SUFFIXES, Prof_DB, allocation_key, full_profile_suffix, plan_key_prefix
from ..planner.allocate import naive_allocate_strategy, solve_sparse_from_bsa
from ..planner.cost import Dist_Attn_Config, get_cc_optimal_schedule_from_table
from ..planner.fuse import Graph_Transformation_Engine
from ..planner.graph import Dependent_Graph
from ..planner.schedule import Execution_Plan
from ..utils.misc import print_rank_0
from .arguments import parse_args
from .benchmark import benchmark_orchestrate_bsa
from .exp_configs import step0_top_down_decompose


def get_general_bsa_cc_optimal_schedule(fob, da_config, prof_db, gpu_tile_type=None, time_limit=60.0):
    """Allocation (ILP #1 or the row-owner ablation) with database caching. ``fob``: the pass, or
    (the reference's form, search_algo/task1_bsa.py:86-143) an ``Evaluation_Configs`` that carries it."""
    fob = int(getattr(fob, "fob", fob))
    hier = da_config.hierarchy
    key = allocation_key(fob, da_config.bsa_config, gpu_tile_type)
    hit = prof_db.get_allocation(key, hier)
    if hit is not None:
        print_rank_0(f"allocation {key}: bypassed")
        cp = da_config.bsa_config.CP[0 if hier else 1]
        par_d = hit["Par_D"]
        import numpy as np
        hit["cmap"] = np.arange(par_d) // max(1, par_d // cp)
        res = hit
    else:
        fn = naive_allocate_strategy if gpu_tile_type == "naive" else solve_sparse_from_bsa
        kw = {} if gpu_tile_type == "naive" else {"time_limit": time_limit}
        res = fn(da_config.bsa_config, fob=fob, hierarchy=hier, **kw)
        prof_db.put_allocation(key, res["table"], hier)
    return get_cc_optimal_schedule_from_table(da_config, prof_db.m_config, res)


def generate_bsa_execution_plans(fob, bsa_config, shape_config, prof_db, hierarchy=1, time_limit=20.0) -> list:
    """The five ablation plans of one (pattern, shape, pass); returns the keys written."""
    da = Dist_Attn_Config.from_bsa_config(bsa_config, shape_config, hierarchy)
    prefix = plan_key_prefix(fob, bsa_config.CP, shape_config, bsa_config)
    keys = [prefix + s for s in ABLATION_SUFFIXES]
    if all(prof_db.has_plan(k, hierarchy) for k in keys):
        print_rank_0(f"plans {prefix}: bypassed")
        return keys
    naive = get_general_bsa_cc_optimal_schedule(fob, da, prof_db, "naive")
    tiled = get_general_bsa_cc_optimal_schedule(fob, da, prof_db, None, time_limit)
    g_naive = Dependent_Graph(naive, fob)
    g_tiled = Dependent_Graph(tiled, fob)
    eng = Graph_Transformation_Engine(None, da, prof_db.m_config)
    plans = [
        Execution_Plan(g_naive, fob, "Flexflow"),
        Execution_Plan(Dependent_Graph(tiled, fob), fob, "Flexflow"),
        eng.transform(g_tiled, "greedy", "Flexflow", time_limit=time_limit),
        Execution_Plan(Dependent_Graph(tiled, fob), fob, "ILP", time_limit=time_limit),
        eng.transform(g_tiled, "greedy", "ILP", time_limit=time_limit),
    ]
    for k, p in zip(keys, plans):
        problems = p.verify()
        assert not problems, (k, problems)
        prof_db.put_plan(k, p, hierarchy)
    return keys


def step1_generate_intra_bsa_exe_plans(space, prof_db, time_limit=20.0) -> list:
    work = []
    for fob in space.fobs:
        for cfg in space.intra_bsa_configs:
            for shape in space.shape_configs(cfg.CP[0]):
                work.append((fob, cfg, shape))
    if not dist.is_initialized() or dist.get_rank() == 0:
        for fob, cfg, shape in work:
            generate_bsa_execution_plans(fob, cfg, shape, prof_db, 1, time_limit)
    if dist.is_initialized():
        dist.barrier()
    return work


def _profile_intra_bsa_one(fob, cfg, shape, prof_db, device) -> list:
    """Measure the stored intra plans (every ablation) of one (pass, pattern, shape) that have no
    profile yet; every rank of the job calls this. Returns the keys measured now."""
    done = []
    prefix = plan_key_prefix(fob, cfg.CP, shape, cfg)
    for suf in ABLATION_SUFFIXES:
        key = prefix + suf
        if prof_db.get_profile(key, 1) is not None:
            continue
        plan = prof_db.get_plan(key, 1)
        other = prof_db.get_plan(plan_key_prefix(0, cfg.CP, shape, cfg) + suf, 1) if fob == 1 else plan
        res = benchmark_orchestrate_bsa(other, plan if fob == 1 else None, fob, device)
        if not dist.is_initialized() or dist.get_rank() == 0:
            prof_db.put_profile(key, res["hfu"], res["time"], res["sim_time"], 1)
        if dist.is_initialized():
            dist.barrier()
        done.append(key)
    return done


def step2_profile_intra_bsa_exe_plans(work, prof_db, device, world: int) -> None:
    """Measure every stored intra plan whose CP equals the number of ranks running now."""
    for fob, cfg, shape in work:
        if cfg.CP[0] == world:
            _profile_intra_bsa_one(fob, cfg, shape, prof_db, device)


def profile_all_intra_BSA(args, exp_config, da_config, ncclcomm_global=None, gloo_global_group=None,
                          tensor_buf=None, prof_db=None) -> list:
    """One configuration of step 2 under the reference's argument list (search_algo/task1_bsa.py:
    244-359). The communicator, the control group and the preallocated buffer are accepted and
    unused: the executor here uses the default process group and allocates per plan. Ranks beyond
    the configuration's CP return at once, as there."""
    assert prof_db is not None, "profile_all_intra_BSA needs the plan database"
    world = dist.get_world_size() if dist.is_initialized() else 1
    cp = da_config.bsa_config.CP[0]
    if cp != world:
        print_rank_0(f"[WARN]: this configuration needs {cp} ranks, the job has {world}: skipped")
        return []
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return _profile_intra_bsa_one(exp_config.fob, da_config.bsa_config, da_config.shape_config, prof_db, device)


def _full_configs(space) -> list:
    from ..utils.bsa_helpers import bsa_is_full
    return [c for c in space.intra_bsa_configs if bsa_is_full(c)]


def step1_generate_intra_full_exe_plans(space, prof_db) -> list:
    """FULL attention gets one shape-free manual plan per grid (Y, X) with Y * X = CP (reference:
    search_algo/task1_bsa.py:672-697); returns the plan keys."""
    from .intra_attn_gen import generate
    keys = []
    if not dist.is_initialized() or dist.get_rank() == 0:
        for cp in sorted({c.CP[0] for c in _full_configs(space)}):
            keys += generate(prof_db, cp, space.fobs)
    if dist.is_initialized():
        dist.barrier()
    return keys


def _profile_intra_full_one(fob, cfg, shape, prof_db, device, world: int) -> list:
    """Measure every grid (Y, X) of FULL attention for one (pass, shape), without kernel tile (the
    manual launch plan: one launch and one message per tile) and with it (gathers, one launch,
    merge / reduce-scatter); every rank calls this. Returns the keys measured now."""
    from ..planner.cost import Dist_Attn_Config as _DA
    from ..planner.dense import create_ablation_configs_for_full, create_plan_for_full
    from ..planner.schedule import Fused_Execution_Plan
    from ..runtime.grid import GridExecutor
    from ..utils.misc import calc_flops
    from .benchmark import benchmark_ops
    done = []
    prefix = plan_key_prefix(fob, cfg.CP, shape, cfg)
    for Y, X in create_ablation_configs_for_full(world):
        for kernel_tile in (False, True):
            key = prefix + full_profile_suffix(kernel_tile, Y, X)
            if prof_db.get_profile(key, 1) is not None:
                continue
            if not kernel_tile:
                pf = create_plan_for_full(world, X, 0, prof_db.m_config, shape_config=shape)
                pb = create_plan_for_full(world, X, 1, prof_db.m_config, shape_config=shape) if fob else None
                res = benchmark_orchestrate_bsa(pf, pb, fob, device)
            else:
                dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
                gx = GridExecutor(Y, X, device=device)
                g = torch.Generator().manual_seed(dist.get_rank() if dist.is_initialized() else 0)
                S_loc = shape["S"][0] // world
                mk = lambda h: torch.randn(shape["bs"], S_loc, h, shape["D"], generator=g).to(dtype).to(device)
                q, k, v, d_o = mk(shape["Nh"][0]), mk(shape["Nh"][1]), mk(shape["Nh"][1]), mk(shape["Nh"][0])
                o, lse = gx.forward(q, k, v)
                fn = (lambda: gx.forward(q, k, v)) if fob == 0 else (lambda: gx.backward(d_o, q, k, v, o, lse))
                t = benchmark_ops(fn, 2, 2, 2, device)
                _, hw = calc_flops(shape["bs"], shape["S"], shape["Nh"][0], shape["D"], False, fob, 1.0)
                sim_t = Fused_Execution_Plan(Y, X, None, fob, prof_db.m_config).materialize(
                    _DA.from_bsa_config(cfg, shape, 1))
                res = {"time": t, "hfu": hw / t / world / 1e12, "sim_time": float(sim_t)}
            if not dist.is_initialized() or dist.get_rank() == 0:
                prof_db.put_profile(key, res["hfu"], res["time"], res["sim_time"], 1)
            if dist.is_initialized():
                dist.barrier()
            done.append(key)
    return done


def step2_profile_intra_full_exe_plans(space, prof_db, device, world: int) -> None:
    """Measure every grid (Y, X) of FULL attention on the ranks running now, under the keys the
    inter-level planner looks up (``..._ablation=({w/o_kernel_tile|w_kernel_tile},Y=..,X=..,dim=0)``;
    reference: search_algo/task1_bsa.py:404-470)."""
    for cfg in _full_configs(space):
        if cfg.CP[0] != world:
            continue
        for shape in space.shape_configs(world):
            for fob in space.fobs:
                _profile_intra_full_one(fob, cfg, shape, prof_db, device, world)


def profile_all_intra_full(args, exp_config, da_config, ncclcomm_global=None, gloo_global_group=None,
                           tensor_buf=None, prof_db=None) -> list:
    """One FULL-attention configuration of step 2 under the reference's argument list
    (search_algo/task1_bsa.py:362-498); see :func:`profile_all_intra_BSA` for the unused arguments."""
    assert prof_db is not None, "profile_all_intra_full needs the plan database"
    world = dist.get_world_size() if dist.is_initialized() else 1
    cfg = da_config.bsa_config
    if cfg.CP[0] != world:
        print_rank_0(f"[WARN]: this configuration needs {cfg.CP[0]} ranks, the job has {world}: skipped")
        return []
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return _profile_intra_full_one(exp_config.fob, cfg, da_config.shape_config, prof_db, device, world)


def step3_generate_inter_bsa_exe_plans(space, prof_db, time_limit=20.0) -> list:
    prof_db.m_config_update_inter_bsa_profile()
    work = []
    for fob in space.fobs:
        for cfg in space.inter_bsa_configs:
            if cfg.CP[1] == 1:
                continue            # single node: the intra plan is the whole plan
            for shape in space.shape_configs(cfg.CP[0] * cfg.CP[1]):
                work.append((fob, cfg, shape))
    if not dist.is_initialized() or dist.get_rank() == 0:
        for fob, cfg, shape in work:
            _generate_inter_plans(fob, cfg, shape, prof_db, time_limit)
    if dist.is_initialized():
        dist.barrier()
    return work


def step3_generate_inter_dense_exe_plans(space, prof_db, time_limit=20.0) -> tuple:
    """Inter-node plans of the dense patterns (search_algo/task1_bsa.py:826-899): FULL attention
    gets the shape-free manual plans of every node grid, like step 1 does inside a node; causal
    attention is planned per shape like any block-sparse pattern. Returns (full keys, causal keys)."""
    from ..utils.bsa_helpers import bsa_is_causal, bsa_is_full
    from .intra_attn_gen import generate
    prof_db.m_config_update_inter_bsa_profile()
    multi = [c for c in space.inter_bsa_configs if c.CP[1] > 1]
    full_keys, causal_keys = [], []
    if not dist.is_initialized() or dist.get_rank() == 0:
        for nodes in sorted({c.CP[1] for c in multi if bsa_is_full(c)}):
            full_keys += generate(prof_db, nodes, space.fobs, hierarchy=0)
        for fob in space.fobs:
            for cfg in (c for c in multi if bsa_is_causal(c)):
                for shape in space.shape_configs(cfg.CP[0] * cfg.CP[1]):
                    causal_keys += _generate_inter_plans(fob, cfg, shape, prof_db, time_limit)
    if dist.is_initialized():
        dist.barrier()
    return full_keys, causal_keys


def _generate_inter_plans(fob, cfg, shape, prof_db, time_limit=20.0) -> list:
    """Inter-node plans of one (pattern, shape, pass): one per ablation of the intra level, whose
    measured times price the compute kernels of the inter graph."""
    da = Dist_Attn_Config.from_bsa_config(cfg, shape, 0)
    prefix = plan_key_prefix(fob, cfg.CP, shape, cfg)
    keys = [prefix + suf for suf in ABLATION_SUFFIXES]
    if all(prof_db.has_plan(k, 0) for k in keys):
        print_rank_0(f"plans {prefix}: bypassed")
        return keys
    tiled = get_general_bsa_cc_optimal_schedule(fob, da, prof_db, None, time_limit)
    for key, suf in zip(keys, ABLATION_SUFFIXES):
        g = Dependent_Graph(tiled, fob, bsa_comp_key_suffixes=[suf])
        prof_db.put_plan(key, Execution_Plan(g, fob, "ILP" if "ILP" in suf else "Flexflow", time_limit=time_limit), 0)
    return keys


# ---- the same generators under the reference's argument lists ------------------------------------
def _check_bypass(keys, prof_db, hierarchy, is_bypass_mode) -> None:
    if is_bypass_mode:
        absent = [k for k in keys if not prof_db.has_plan(k, hierarchy)]
        assert not absent, f"bypass mode: these plans are not in the database: {absent[:2]}"


def generate_intra_bsa_execution_plans(exp_config, da_config, prof_db, is_bypass_mode: bool = False,
                                       time_limit: float = 20.0) -> list:
    """``(exp_config, da_config, prof_db, is_bypass_mode)``: search_algo/task1_bsa.py:153-241. In
    bypass mode (ranks of a GPU job, which must not solve) every plan has to be stored already."""
    exp_config.hierarchy = da_config.hierarchy = 1
    cfg, shape = da_config.bsa_config, da_config.shape_config
    _check_bypass([plan_key_prefix(exp_config.fob, cfg.CP, shape, cfg) + s for s in ABLATION_SUFFIXES], prof_db, 1,
                  is_bypass_mode)
    return generate_bsa_execution_plans(exp_config.fob, cfg, shape, prof_db, 1, time_limit)


def generate_inter_bsa_execution_plans(exp_config, da_config, prof_db, is_bypass_mode: bool = False,
                                       time_limit: float = 20.0) -> list:
    """``(exp_config, da_config, prof_db, is_bypass_mode)``: search_algo/task1_bsa.py:501-578."""
    exp_config.hierarchy = da_config.hierarchy = 0
    cfg, shape = da_config.bsa_config, da_config.shape_config
    _check_bypass([plan_key_prefix(exp_config.fob, cfg.CP, shape, cfg) + s for s in ABLATION_SUFFIXES], prof_db, 0,
                  is_bypass_mode)
    return _generate_inter_plans(exp_config.fob, cfg, shape, prof_db, time_limit)


def generate_general_full_execution_plans(exp_config, da_config, hierarchy, prof_db,
                                          is_bypass_mode: bool = False) -> list:
    """Shape-free manual plans of FULL attention on every grid of ``da_config``'s rank count at one
    level (search_algo/task1_bsa.py:615-669); returns the keys."""
    from .intra_attn_gen import full_plan_keys, generate
    exp_config.hierarchy = da_config.hierarchy = hierarchy
    cp = da_config.bsa_config.CP[0 if hierarchy else 1]
    _check_bypass(full_plan_keys(cp, [exp_config.fob], hierarchy), prof_db, hierarchy, is_bypass_mode)
    return generate(prof_db, cp, [exp_config.fob], hierarchy)


def main(argv=None) -> None:
    args = parse_args(argv)
    info = initialize_distribution()
    quick = bool(args.extra.get("quick"))
    prof_db = Prof_DB(os.environ.get("CLUSTER_NAME"), os.environ.get("PLATFORM"))
    space = step0_top_down_decompose(args.exp_class or "bsa_train", max_intra=info["tasks_per_node"],
                                     max_nodes=info["node_num"], quick=quick)
    work = step1_generate_intra_bsa_exe_plans(space, prof_db)
    device = torch.device("cuda", info["local_rank"]) if torch.cuda.is_available() else torch.device("cpu")
    step2_profile_intra_bsa_exe_plans(work, prof_db, device, info["world_size"])
    if _full_configs(space):                        # dense_train: the (Y, X) grids of FULL attention
        step1_generate_intra_full_exe_plans(space, prof_db)
        step2_profile_intra_full_exe_plans(space, prof_db, device, info["world_size"])
    step3_generate_inter_bsa_exe_plans(space, prof_db)
    if space.exp_class == "dense_train" and info["node_num"] > 1:
        step3_generate_inter_dense_exe_plans(space, prof_db)     # + the manual node grids of FULL attention
    print_rank_0("task1 done")
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
