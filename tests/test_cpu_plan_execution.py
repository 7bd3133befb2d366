"""Plan -> execution -> result on CPU ranks over gloo, checked against the dense oracle.

The headline case: block-sparse global+local attention, S=4096 in 8 blocks of 512 (block 0 global,
causal local window of 2 blocks), 4 heads, D=64, fp32, world size 2; ILP plan, forward and backward.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.planner import make_plan_collective
        from ultraattn_b200.runtime import PlanExecutor
        pattern = case["pattern"]()
        S, H, D = case["S"], case["H"], case["D"]
        kw = dict(pattern=pattern, cp=world, seq_len=S, n_heads=H, head_dim=D, allocation=case.get("allocation", "ilp"),
                  plan_type=case.get("plan_type", "ILP"), time_limit=case.get("time_limit", 5.0),
                  kernel_tile=case.get("kernel_tile", False), cp_inter=case.get("cp_inter", 1))
        if case.get("cp_inter", 1) > 1:
            kw["cp"] = world // case["cp_inter"]
        plan_f = make_plan_collective(fob=0, **kw)     # rank 0 plans, everyone gets the same plan
        plan_b = make_plan_collective(fob=1, **kw)
        assert plan_f.verify() == [] and plan_b.verify() == []
        g = torch.Generator().manual_seed(case.get("seed", 0))
        q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
        ex = PlanExecutor(plan_f, plan_b, group=None, device=torch.device("cpu"), recv_timeout_s=30)
        blk = S // ex.par_d
        idx = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in ex.my_blocks])
        ql, kl, vl, dol = (t[:, idx].contiguous() for t in (q, k, v, d_o))
        o, lse = ex.forward(ql, kl, vl)
        dq, dk, dv = ex.backward(dol, ql, kl, vl, o, lse)
        o_ref, lse_ref, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q, k, v, d_o, pattern)
        errs = {
            "o": (o - o_ref[:, idx]).abs().max().item(),
            "lse": (lse - lse_ref[:, :, idx]).abs().max().item(),
            "dq": (dq - dq_ref[:, idx]).abs().max().item(),
            "dk": (dk - dk_ref[:, idx]).abs().max().item(),
            "dv": (dv - dv_ref[:, idx]).abs().max().item(),
        }
        ret[rank] = errs
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def _run(world, case):
    port = 29500 + (os.getpid() + hash(str(sorted(case.items(), key=str))) % 1000) % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, case, ret), nprocs=world, join=True)
    return dict(ret)


def _pat_global_local():
    from ultraattn_b200 import patterns as P
    return P.global_local(8, 1, 2)


def _pat_causal():
    from ultraattn_b200 import patterns as P
    return P.causal(1)


def _pat_strided():
    from ultraattn_b200 import patterns as P
    return P.strided(8, 4, 2)


def _pat_star():
    from ultraattn_b200 import patterns as P
    return P.star(4, 1)


@pytest.mark.parametrize("plan_type", ["ILP", "Flexflow"])
def test_global_local_s4096_world2(plan_type):
    res = _run(2, {"pattern": _pat_global_local, "S": 4096, "H": 4, "D": 64, "plan_type": plan_type})
    for r in range(2):
        assert "error" not in res[r], res[r].get("error")
        for name, e in res[r].items():
            assert e < 2e-4, (r, name, e)


@pytest.mark.parametrize("case", [
    {"pattern": _pat_causal, "S": 512, "H": 2, "D": 32, "plan_type": "Flexflow"},
    {"pattern": _pat_strided, "S": 1024, "H": 2, "D": 32, "plan_type": "Flexflow"},
    {"pattern": _pat_star, "S": 512, "H": 2, "D": 32, "plan_type": "Flexflow", "allocation": "naive"},
    {"pattern": _pat_causal, "S": 1024, "H": 2, "D": 32, "plan_type": "Flexflow", "kernel_tile": True},
    {"pattern": _pat_strided, "S": 1024, "H": 2, "D": 32, "plan_type": "Flexflow", "cp_inter": 2},
    {"pattern": _pat_causal, "S": 512, "H": 2, "D": 32, "plan_type": "Flexflow", "allocation": "lightseq"},
], ids=["causal", "strided", "star-naive", "causal-kernel-tile", "strided-two-level-2x2", "causal-lightseq"])
def test_patterns_world4(case):
    res = _run(4, case)
    for r in range(4):
        assert "error" not in res[r], res[r].get("error")
        for name, e in res[r].items():
            assert e < 2e-4, (r, name, e)


def _json_worker(rank, world, port, path_f, path_b, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.planner import Execution_Plan
        from ultraattn_b200.runtime import PlanExecutor
        plan_f, plan_b = Execution_Plan.from_json(path_f), Execution_Plan.from_json(path_b)
        assert plan_f.sanity_check_stream_exclusive()
        pattern = plan_f.da_config.bsa_config.bsa_repr
        S, (H, _), D = plan_f.da_config.S[0], plan_f.da_config.Nh, plan_f.da_config.D
        g = torch.Generator().manual_seed(2)
        q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
        ex = PlanExecutor(plan_f, plan_b, group=None, device=torch.device("cpu"), recv_timeout_s=30)
        blk = S // ex.par_d
        idx = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in ex.my_blocks])
        o, lse = ex.forward(*(t[:, idx].contiguous() for t in (q, k, v)))
        dq, dk, dv = ex.backward(d_o[:, idx].contiguous(), *(t[:, idx].contiguous() for t in (q, k, v)), o, lse)
        o_ref, _, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q, k, v, d_o, pattern)
        ret[rank] = max((o - o_ref[:, idx]).abs().max().item(), (dq - dq_ref[:, idx]).abs().max().item(),
                        (dk - dk_ref[:, idx]).abs().max().item(), (dv - dv_ref[:, idx]).abs().max().item())
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def test_plans_execute_from_their_json_form(tmp_path):
    """A plan written as JSON (no pickle) is read back by other processes and executed on two
    ranks: same results as the dense oracle."""
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.planner import make_plan
    kw = dict(pattern=P.global_local(4, 1, 2), cp=2, seq_len=256, n_heads=2, head_dim=16, allocation="ilp",
              plan_type="ILP", time_limit=3.0, kernel_tile=True)
    paths = []
    for fob in (0, 1):
        plan = make_plan(fob=fob, **kw)
        paths.append(str(tmp_path / f"plan{fob}.json"))
        plan.to_json(paths[-1])
    ret = mp.Manager().dict()
    mp.spawn(_json_worker, args=(2, 29480 + os.getpid() % 15, paths[0], paths[1], ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], float), ret[r]
        assert ret[r] < 2e-4, (r, ret[r])


def _random_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import random
        import numpy as np
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.patterns.blocks import BSA_Repr
        from ultraattn_b200.planner import make_plan_collective
        from ultraattn_b200.runtime import PlanExecutor
        worst = 0.0
        for seed in range(4):
            rng = random.Random(seed)           # the same table on every rank
            n = rng.choice([4, 8])
            t = np.zeros((n, n), dtype=np.int8)
            for i in range(n):
                t[i, i] = 2
                for j in range(i):
                    t[i, j] = rng.choice([0, 1])
            pattern = BSA_Repr(t)
            S, H, D = 256, 2, 16
            kw = dict(pattern=pattern, cp=world, seq_len=S, n_heads=H, head_dim=D, allocation="ilp",
                      plan_type=rng.choice(["ILP", "Flexflow"]), time_limit=2.0, kernel_tile=rng.random() < 0.5)
            pf, pb = make_plan_collective(fob=0, **kw), make_plan_collective(fob=1, **kw)
            assert pf.verify() == [] and pb.verify() == []
            g = torch.Generator().manual_seed(seed)
            q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
            ex = PlanExecutor(pf, pb, group=None, device=torch.device("cpu"), recv_timeout_s=30)
            blk = S // ex.par_d
            idx = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in ex.my_blocks])
            o, lse = ex.forward(*(x[:, idx].contiguous() for x in (q, k, v)))
            dq, dk, dv = ex.backward(d_o[:, idx].contiguous(), *(x[:, idx].contiguous() for x in (q, k, v)), o, lse)
            o_ref, _, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q, k, v, d_o, pattern)
            worst = max(worst, (o - o_ref[:, idx]).abs().max().item(), (dq - dq_ref[:, idx]).abs().max().item(),
                        (dk - dk_ref[:, idx]).abs().max().item(), (dv - dv_ref[:, idx]).abs().max().item())
        ret[rank] = worst
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def test_random_patterns_execute_correctly_world4():
    """Four seeded random causal-type patterns, random scheduler and kernel tiling, planned and
    executed on four gloo ranks: results match dense attention."""
    ret = mp.Manager().dict()
    mp.spawn(_random_worker, args=(4, 29460 + os.getpid() % 15, ret), nprocs=4, join=True)
    for r in range(4):
        assert isinstance(ret[r], float), ret[r]
        assert ret[r] < 2e-4, (r, ret[r])


def _ref_harness_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from search_algo.benchmark import benchmark_orchestrate_bsa
        from search_algo.execute_plan import Execution_Plan
        from search_algo.search_engine import Evaluation_Configs
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.planner import make_plan_collective
        out = []
        for fob in (0, 1):
            plan = make_plan_collective(pattern=P.strided(8, 4, 2), cp=world, seq_len=1024, n_heads=2, head_dim=32,
                                        fob=fob, plan_type="Flexflow", time_limit=3.0)
            inter = Execution_Plan.create_one_node_exe_plan(fob)
            exp = Evaluation_Configs(plan_type="Flexflow", MAX_QUEUE_SIZE=100, fob=fob, hierarchy=1, transform_mode="greedy")
            res = benchmark_orchestrate_bsa(None, None, plan.da_config, exp, None, [inter], [{((1, 1), "k"): plan}],
                                            warmup=1, num_iter=1, log=False)
            out.append(res)
        ret[rank] = out
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def test_harness_with_the_reference_argument_list():
    """`search_algo.benchmark.benchmark_orchestrate_bsa(args, raw_f, da_config, exp_config, tensor_buf,
    inter_plans, comp_plan_dicts, ...)`: one result dict per plan on rank 0, None elsewhere."""
    ret = mp.Manager().dict()
    mp.spawn(_ref_harness_worker, args=(2, 29500 + os.getpid() % 90, ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], list), ret[r]
    for res in ret[0]:
        assert len(res) == 1 and set(res[0]) == {"hfu", "time"} and float(res[0]["time"]) > 0
    assert all(res == [None] for res in ret[1])


def _switch_over_worker(rank, world, port, dbroot, ret):
    """A script written against the reference's modules, names and argument lists (the sequence of
    calls its campaign makes for one configuration), run against this distribution."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world), CLUSTER_NAME="testbox", PLATFORM="CPU", UA_DATABASE_ROOT=dbroot)
    try:
        import numpy as np
        from search_algo.initialize import initialize_distribution, initialize_prof_db
        from search_algo.bsa_config import BSA_Config, BSA_Repr
        from search_algo.utils import Block_Type
        from search_algo.search_engine import Dist_Attn_Config, Evaluation_Configs
        from search_algo.dependent_graph import Dependent_Graph
        from search_algo.execute_plan import Execution_Plan
        from search_algo.task1_bsa import get_general_bsa_cc_optimal_schedule
        from search_algo.benchmark import benchmark_orchestrate_bsa
        from search_algo.global_vars import get_global_var
        ncclcomm_global, gloo_group = initialize_distribution()
        assert get_global_var("PROC_INFO")["rank"] == rank and ncclcomm_global.world_size == world
        prof_db = initialize_prof_db(gloo_group)
        table = np.full((8, 8), Block_Type.EMPTY, dtype=object)
        for i in range(8):
            for j in range(i + 1):
                if i == j:
                    table[i, j] = Block_Type.CAUSAL
                elif i - j <= 1 or (i - j) % 4 == 0:
                    table[i, j] = Block_Type.FULL
        bsa_repr = BSA_Repr(block_table=table, cmap=None)
        bsa_config = BSA_Config(None, None, {"bsa_repr": bsa_repr, "CP": (world, 1)})
        shape_config = {"Nh": (2, 2), "S": (1024, 1024), "bs": 1, "D": 32}
        da_config = Dist_Attn_Config.from_bsa_config(bsa_config, shape_config=shape_config, hierarchy=1)
        results = []
        for fob in (0, 1):
            exp_config = Evaluation_Configs(plan_type="Flexflow", MAX_QUEUE_SIZE=100, fob=fob, hierarchy=1,
                                            transform_mode="greedy")
            schedule = get_general_bsa_cc_optimal_schedule(exp_config, da_config, prof_db, gpu_tile_type="naive")
            plan = Execution_Plan(Dependent_Graph(schedule, fob), fob, plan_type="Flexflow")
            inter_plan = Execution_Plan.create_one_node_exe_plan(fob)
            res = benchmark_orchestrate_bsa(None, None, da_config, exp_config, None,
                                            inter_bsa_execution_plans=[inter_plan],
                                            inter_comp_plans_dicts=[{((1, 1), str(bsa_repr)): plan}],
                                            warmup=1, num_iter=1, log=False, global_group=None)
            results.append((plan.verify(), res))
        ret[rank] = results
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\\n{traceback.format_exc()}"
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_a_script_written_against_the_reference_runs_unchanged(tmp_path):
    ret = mp.Manager().dict()
    mp.spawn(_switch_over_worker, args=(2, 29600 + os.getpid() % 90, str(tmp_path), ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], list), ret[r]
        for problems, _ in ret[r]:
            assert problems == []
    for _, res in ret[0]:
        assert float(res[0]["time"]) > 0 and res[0]["hfu"] >= 0
