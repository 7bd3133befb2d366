"""The planning / profiling campaign end to end on CPU ranks (tiny shapes), and inter-node planning."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, root, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.drivers import task1
        from ultraattn_b200.drivers.exp_configs import ExpSpace
        from ultraattn_b200.patterns.blocks import BSA_Config
        from ultraattn_b200.plandb import ABLATION_SUFFIXES, Prof_DB, plan_key_prefix
        cfg = BSA_Config(None, None, {"bsa_repr": P.star(4, 1), "CP": (2, 1)})
        space = ExpSpace("bsa_infer", [0], [cfg], [cfg], [256], [2], D=16, S_per_gpu_bounds=(1, 1 << 20))
        db = Prof_DB("unit", "cpu", root=root)
        work = task1.step1_generate_intra_bsa_exe_plans(space, db, time_limit=2.0)
        task1.step2_profile_intra_bsa_exe_plans(work, db, torch.device("cpu"), world)
        dist.barrier()
        shape = {"S": (256, 256), "Nh": (2, 2), "bs": 1, "D": 16}
        prefix = plan_key_prefix(0, (2, 1), shape, cfg)
        prof = [Prof_DB("unit", "cpu", root=root).get_profile(prefix + s) for s in ABLATION_SUFFIXES]
        ret[rank] = all(p is not None and float(p["time"]) > 0 and float(p["sim_time"]) > 0 for p in prof)
        # a second pass is a no-op: everything is keyed in the database
        work2 = task1.step1_generate_intra_bsa_exe_plans(space, db, time_limit=2.0)
        assert len(work2) == len(work)
        # dense_train: every (Y, X) grid of FULL attention, without and with kernel tile
        from ultraattn_b200.plandb import full_plan_key, full_profile_suffix
        full = BSA_Config.create_full((2, 1))
        fspace = ExpSpace("dense_train", [0, 1], [full], [full], [256], [2], D=16, S_per_gpu_bounds=(1, 1 << 20))
        keys = task1.step1_generate_intra_full_exe_plans(fspace, db)
        if rank == 0:
            assert full_plan_key(1, (2, 1), 1, 2) in keys and len(keys) == 4
        task1.step2_profile_intra_full_exe_plans(fspace, db, torch.device("cpu"), world)
        dist.barrier()
        fresh = Prof_DB("unit", "cpu", root=root)
        for fob in (0, 1):
            fprefix = plan_key_prefix(fob, (2, 1), shape, full)
            for Y, X in ((2, 1), (1, 2)):
                for kt in (False, True):
                    p = fresh.get_profile(fprefix + full_profile_suffix(kt, Y, X))
                    assert p is not None and float(p["time"]) > 0 and float(p["sim_time"]) > 0, (fob, Y, X, kt)
        # the per-configuration forms under the reference's argument lists find everything measured
        from search_algo.task1_bsa import profile_all_intra_BSA, profile_all_intra_full
        from search_algo.task2_bsa import profile_all_inter_BSA
        from ultraattn_b200.planner.cost import Dist_Attn_Config, Evaluation_Configs
        exp0 = Evaluation_Configs("ILP", 1, 0)
        assert profile_all_intra_full(None, exp0, Dist_Attn_Config.from_bsa_config(full, shape, 1), None, None, None, db) == []
        da_star = Dist_Attn_Config.from_bsa_config(cfg, shape, 1)
        assert profile_all_intra_BSA(None, exp0, da_star, None, None, None, db) == []
        inter_keys = profile_all_inter_BSA(None, exp0, da_star, None, None, None, db)
        assert len(inter_keys) == (len(ABLATION_SUFFIXES) if rank == 0 else 0)
        dist.barrier()
        # step 4 + baselines: the figure table gets its ring / zigzag / stripe columns
        from ultraattn_b200.drivers import report, task2
        causal = BSA_Config.create_causal((2, 1))
        cspace = ExpSpace("dense_train", [0], [causal], [causal], [256], [2], D=16, S_per_gpu_bounds=(1, 1 << 20))
        task2.step4_profile_inter_bsa_exe_plans(space, db, world)
        keys = task2.step5_profile_baselines(space, db, torch.device("cpu"), world, iters=1)
        keys += task2.step5_profile_baselines(cspace, db, torch.device("cpu"), world, iters=1)
        assert [k.rsplit("_", 1)[1] for k in keys] == ["ring", "ring", "zigzag", "stripe"]
        dist.barrier()
        if rank == 0:
            import json
            prof = json.loads(open(db.INTER_BSA_EXE_PLANS_PROFILE).read())
            rows = {r["key"]: r for r in report.build_rows(prof)}
            star_row = rows[plan_key_prefix(0, (2, 1), shape, cfg)]
            assert star_row["ring"] > 0 and star_row["ultraattn"] > 0 and star_row["speedup_vs_ring"] > 0
            causal_row = rows[plan_key_prefix(0, (2, 1), shape, causal)]
            assert causal_row["zigzag"] > 0 and causal_row["stripe"] > 0
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def test_campaign_steps_1_2_on_gloo(tmp_path):
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, 29790 + os.getpid() % 50, str(tmp_path), ret), nprocs=2, join=True)
    assert ret[0] is True and ret[1] is True, dict(ret)


def test_inter_node_plan_uses_intra_costs():
    """Hierarchy 0: node tiles of a 2-node x 4-GPU causal problem are allocated to nodes and their
    compute kernels are costed by the (measured or estimated) intra-node plans."""
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.patterns.blocks import BSA_Config
    from ultraattn_b200.planner import (Dependent_Graph, Dist_Attn_Config, Execution_Plan, Machine_Config,
                                        get_cc_optimal_schedule_from_table, solve_sparse_from_bsa)
    cfg = BSA_Config(None, None, {"bsa_repr": P.strided(8, 4, 2), "CP": (4, 2)})
    shape = {"S": (65536, 65536), "Nh": (32, 32), "bs": 1, "D": 128}
    da = Dist_Attn_Config.from_bsa_config(cfg, shape, hierarchy=0)
    assert da.SP == (2, 4) and da.hierarchy_sp == 2
    al = solve_sparse_from_bsa(cfg, fob=0, ParD=2, hierarchy=0, time_limit=2.0)
    m = Machine_Config.b200_default()
    sch = get_cc_optimal_schedule_from_table(da, m, al)
    g = Dependent_Graph(sch, 0, bsa_comp_key_suffixes=["_ablation=(w/o_kernel_tile,ILP)"])
    plan = Execution_Plan(g, 0, "ILP", time_limit=2.0)
    assert plan.verify() == []
    comp = [k for k in plan.valid_kernels if k.type == "comp"]
    assert comp and all(isinstance(k.comp_map_key, str) and k.comp_map_key.startswith("fob=0_CP=(4, 1)")
                        for k in comp)
    # a measured intra profile overrides the estimate
    m.update_inter_bsa_profile({comp[0].comp_map_key + "_ablation=(w/o_kernel_tile,ILP)":
                                {"hfu": 1.0, "time": "5.000e-01", "sim_time": "5.000e-01"}})
    g2 = Dependent_Graph(sch, 0, bsa_comp_key_suffixes=["_ablation=(w/o_kernel_tile,ILP)"])
    assert any(abs(k.time[0] - 0.5) < 1e-12 for k in g2.kernel_dict.values() if k.type == "comp")


def test_fusion_table_and_full_plan_generation(tmp_path, capsys):
    """The tile-fusion table (small tiles gain from fusing, big ones do not) and the generator of
    the Y x X plans of FULL attention into the plan database."""
    from ultraattn_b200.drivers import fusion_evaluate, intra_attn_gen
    from ultraattn_b200.plandb import Prof_DB
    from ultraattn_b200.planner.cost import FlashAttn_Profile_Map
    rows = fusion_evaluate.fusion_table(FlashAttn_Profile_Map({}), [1], [256, 16384], degrees=[(2, 2)])
    small = next(r for r in rows if r["S"] == 256 and r["fob"] == 0)
    big = next(r for r in rows if r["S"] == 16384 and r["fob"] == 0)
    assert small["speedup"] > 1.5 and big["speedup"] < small["speedup"]
    measured = FlashAttn_Profile_Map({(256, 1, 1, 128, "1/1", False): [1e-5, 3e-5],
                                      (256, 1, 1, 128, "2/1", False): [1.2e-5, 3.3e-5]})
    r = fusion_evaluate.fusion_table(measured, [1], [256], degrees=[(2, 1)])
    assert abs(r[0]["speedup"] - 2 / 1.2) < 1e-9 and abs(r[1]["speedup"] - 2 * 3 / 3.3) < 1e-9
    assert fusion_evaluate.main(["--nh", "1", "--smin", "256", "--smax", "512"]) == 0
    assert "speed-up" in capsys.readouterr().out
    db = Prof_DB("t", "B200", root=str(tmp_path))
    keys = intra_attn_gen.generate(db, 4, (0, 1))
    assert len(keys) == 6 and "fob=1_CP=(4, 1)_shape_config=full_ablation=(Y=2,X=2,dim=0)" in keys
    plan = db.get_plan(keys[0], 1)
    assert plan.verify() == [] and intra_attn_gen.generate(db, 4, (0, 1)) == keys


_YAML = """
Parallel:
  SP: [1, 2]
Shape: {Sq: 512, Skv: 512, Nhq: 2, Nhkv: 2, BS: 1, D: 16}
Pattern: {pattern_type: stream, n_blocks: 4, global_blocks: 1, local_blocks: 2}
Experiment: {transform_mode: greedy, lowering_mode: ILP}
"""


def _main_worker(rank, world, port, cfg_path, out_dir):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from ultraattn_b200.drivers import main as M
    sys.stdout = open(os.path.join(out_dir, f"rank{rank}.out"), "w")
    rc = M.main(["--config", cfg_path, "--iters", "1", "--time-limit", "3"])
    sys.stdout.flush()
    assert rc == 0


def test_single_configuration_driver(tmp_path, capsys):
    """YAML -> plan -> description (plan only), and the same configuration executed and timed on
    two gloo ranks."""
    import json
    import os
    import torch.multiprocessing as mp
    from ultraattn_b200.drivers import main as M
    cfg = tmp_path / "stream.yaml"
    cfg.write_text(_YAML)
    assert M.main(["--config", str(cfg), "--plan-only", "--time-limit", "3", "--save-plan", str(tmp_path / "plans")]) == 0
    recs = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    assert [r["fob"] for r in recs] == [0, 1] and all(r["problems"] == [] and r["sim_time_ms"] > 0 for r in recs)
    assert all(os.path.exists(r["plan_file"]) for r in recs)
    mp.spawn(_main_worker, args=(2, 29150 + os.getpid() % 40, str(cfg), str(tmp_path)), nprocs=2, join=True)
    lines = [json.loads(line) for line in (tmp_path / "rank0.out").read_text().strip().splitlines()]
    timed = [r for r in lines if "time_ms" in r]
    assert [r["fob"] for r in timed] == [0, 1] and all(r["time_ms"] > 0 and r["n_ranks"] == 2 for r in timed)


def test_step4_full_attention_takes_the_best_grid(tmp_path):
    """Single node, FULL attention: every ablation level of the inter profile is the best (Y, X)
    grid measurement that level may use."""
    from ultraattn_b200.drivers import task2
    from ultraattn_b200.drivers.exp_configs import ExpSpace
    from ultraattn_b200.patterns.blocks import BSA_Config
    from ultraattn_b200.plandb import Prof_DB, full_profile_suffix, plan_key_prefix
    full = BSA_Config.create_full((2, 1))
    space = ExpSpace("dense_train", [0], [full], [full], [256], [2], D=16, S_per_gpu_bounds=(1, 1 << 20))
    db = Prof_DB("unit", "cpu", root=str(tmp_path))
    shape = {"S": (256, 256), "Nh": (2, 2), "bs": 1, "D": 16}
    prefix = plan_key_prefix(0, (2, 1), shape, full)
    times = {(False, 2, 1): 4e-3, (False, 1, 2): 3e-3, (True, 2, 1): 2e-3, (True, 1, 2): 5e-3}
    for (kt, Y, X), t in times.items():
        db.put_profile(prefix + full_profile_suffix(kt, Y, X), 1.0, t, t, 1)
    task2.step4_profile_inter_bsa_exe_plans(space, db, world=2)
    got = {s: float(db.get_profile(prefix + s, 0)["time"]) for s in
           ("_ablation=(w/o_gpu_tile,w/o_kernel_tile,Flexflow)", "_ablation=(w/o_kernel_tile,ILP)",
            "_ablation=(w_kernel_tile,ILP)")}
    assert got["_ablation=(w/o_gpu_tile,w/o_kernel_tile,Flexflow)"] == 4e-3      # Y = CP, X = 1 only
    assert got["_ablation=(w/o_kernel_tile,ILP)"] == 3e-3                         # best grid without kernel tile
    assert got["_ablation=(w_kernel_tile,ILP)"] == 2e-3                           # best of all


def test_plan_generators_under_the_reference_argument_lists(tmp_path, monkeypatch):
    """``generate_{intra,inter}_bsa_execution_plans(exp_config, da_config, prof_db, is_bypass_mode)``
    and ``generate_general_full_execution_plans(exp_config, da_config, hierarchy, prof_db, ...)``:
    first call writes the plans, bypass mode then finds every one, and bypass mode on an empty
    database refuses instead of solving."""
    import pytest
    from search_algo.task1_bsa import (generate_general_full_execution_plans, generate_inter_bsa_execution_plans,
                                       generate_intra_bsa_execution_plans)
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.patterns.blocks import BSA_Config
    from ultraattn_b200.plandb import ABLATION_SUFFIXES, Prof_DB
    from ultraattn_b200.planner.cost import Dist_Attn_Config, Evaluation_Configs
    monkeypatch.setenv("UA_DATABASE_ROOT", str(tmp_path))
    db = Prof_DB("unit", "B200")
    shape = {"S": (4096, 4096), "Nh": (2, 2), "bs": 1, "D": 128}
    exp = Evaluation_Configs("ILP", 1, 0)
    cfg = BSA_Config(None, None, {"bsa_repr": P.strided(4, 2, 1), "CP": (2, 1)})
    da = Dist_Attn_Config.from_bsa_config(cfg, shape, 1)
    with pytest.raises(AssertionError, match="bypass"):
        generate_intra_bsa_execution_plans(exp, da, db, True)
    keys = generate_intra_bsa_execution_plans(exp, da, db, False, time_limit=3.0)
    assert len(keys) == len(ABLATION_SUFFIXES) and all(db.has_plan(k, 1) for k in keys)
    assert generate_intra_bsa_execution_plans(exp, da, db, True) == keys
    assert db.get_plan(keys[0], 1).verify() == []

    full = Dist_Attn_Config.from_bsa_config(BSA_Config.create_full((4, 1)), shape, 1)
    fkeys = generate_general_full_execution_plans(exp, full, 1, db, False)
    assert len(fkeys) == 3 and generate_general_full_execution_plans(exp, full, 1, db, True) == fkeys   # 1x4, 2x2, 4x1
    with pytest.raises(AssertionError, match="bypass"):
        generate_general_full_execution_plans(Evaluation_Configs("ILP", 1, 1), full, 1, db, True)

    cfg2 = BSA_Config(None, None, {"bsa_repr": P.strided(4, 2, 1), "CP": (1, 2)})
    shape2 = {"S": (8192, 8192), "Nh": (2, 2), "bs": 1, "D": 128}
    da2 = Dist_Attn_Config.from_bsa_config(cfg2, shape2, 0)
    ikeys = generate_inter_bsa_execution_plans(exp, da2, db, False, time_limit=3.0)
    assert exp.hierarchy == 0 and da2.hierarchy == 0
    assert all(db.has_plan(k, 0) for k in ikeys) and generate_inter_bsa_execution_plans(exp, da2, db, True) == ikeys
    assert db.get_plan(ikeys[-1], 0).verify() == []


def test_inter_node_plans_of_the_dense_patterns(tmp_path, monkeypatch):
    """Two nodes of two ranks, dense patterns: FULL gets the manual plans of every node grid
    (shape-free, one per pass), causal is planned per shape; a second call finds all of them."""
    from search_algo.task1_bsa import step3_generate_inter_dense_exe_plans
    from ultraattn_b200.drivers.exp_configs import step0_top_down_decompose
    from ultraattn_b200.plandb import Prof_DB
    monkeypatch.setenv("UA_DATABASE_ROOT", str(tmp_path))
    db = Prof_DB("unit", "B200")
    space = step0_top_down_decompose("dense_train", max_intra=2, max_nodes=2, quick=True)
    full_keys, causal_keys = step3_generate_inter_dense_exe_plans(space, db, time_limit=3.0)
    assert full_keys and all("CP=(1, 2)" in k and db.has_plan(k, 0) for k in full_keys)
    assert {k.split("_")[0] for k in full_keys} == {f"fob={f}" for f in space.fobs}
    assert causal_keys and all(db.has_plan(k, 0) and db.get_plan(k, 0).verify() == [] for k in causal_keys)
    again = step3_generate_inter_dense_exe_plans(space, db, time_limit=3.0)
    assert again == (full_keys, causal_keys)
