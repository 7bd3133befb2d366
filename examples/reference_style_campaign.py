"""One configuration planned, executed and timed through the module paths, class names and
argument lists of oliverYoung2001/UltraAttn (the sequence of calls its campaign makes for one
pattern): code written against the reference runs on this distribution as it is.

    torchrun --nproc-per-node 2 examples/reference_style_campaign.py         # GPUs, or CPU ranks over gloo

Every import below is a path of the reference; nothing of ``ultraattn_b200`` is named."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np  # noqa: E402

from search_algo.benchmark import benchmark_orchestrate_bsa  # noqa: E402
from search_algo.bsa_config import BSA_Config, BSA_Repr  # noqa: E402
from search_algo.dependent_graph import Dependent_Graph  # noqa: E402
from search_algo.execute_plan import Execution_Plan  # noqa: E402
from search_algo.global_vars import get_global_var  # noqa: E402
from search_algo.initialize import initialize_distribution, initialize_prof_db  # noqa: E402
from search_algo.search_engine import Dist_Attn_Config, Evaluation_Configs  # noqa: E402
from search_algo.task1_bsa import (generate_intra_bsa_execution_plans, get_general_bsa_cc_optimal_schedule,  # noqa: E402
                                   profile_all_intra_BSA)
from search_algo.utils import Block_Type  # noqa: E402


def strided_table(n: int, stride: int = 4, window: int = 2):
    table = np.full((n, n), Block_Type.EMPTY, dtype=object)
    for i in range(n):
        for j in range(i + 1):
            if i == j:
                table[i, j] = Block_Type.CAUSAL
            elif i - j < window or (i - j) % stride == 0:
                table[i, j] = Block_Type.FULL
    return table


def main() -> None:
    os.environ.setdefault("CLUSTER_NAME", "example")
    os.environ.setdefault("PLATFORM", "B200")
    os.environ.setdefault("UA_DATABASE_ROOT", os.path.join(tempfile.gettempdir(), "ua_example_database"))
    ncclcomm_global, gloo_group = initialize_distribution()
    info = get_global_var("PROC_INFO")
    rank, world = info["rank"], info["world_size"]
    prof_db = initialize_prof_db(gloo_group)

    bsa_repr = BSA_Repr(block_table=strided_table(8), cmap=None)
    bsa_config = BSA_Config(None, None, {"bsa_repr": bsa_repr, "CP": (world, 1)})
    shape_config = {"Nh": (4, 4), "S": (4096, 4096), "bs": 1, "D": 128}
    da_config = Dist_Attn_Config.from_bsa_config(bsa_config, shape_config=shape_config, hierarchy=1)

    for fob in (0, 1):
        exp_config = Evaluation_Configs(plan_type="Flexflow", MAX_QUEUE_SIZE=100, fob=fob, hierarchy=1,
                                        transform_mode="greedy")
        schedule = get_general_bsa_cc_optimal_schedule(exp_config, da_config, prof_db, gpu_tile_type=None)
        plan = Execution_Plan(Dependent_Graph(schedule, fob), fob, plan_type="Flexflow")
        inter_plan = Execution_Plan.create_one_node_exe_plan(fob)
        results = benchmark_orchestrate_bsa(None, None, da_config, exp_config, None,
                                            inter_bsa_execution_plans=[inter_plan],
                                            inter_comp_plans_dicts=[{((1, 1), str(bsa_repr)): plan}],
                                            warmup=2, num_iter=2, log=False)
        if rank == 0:
            print(f"fob={fob}: {len(plan.valid_kernels)} kernels, predicted {plan.end_time:.3e} s, "
                  f"measured {results[0]['time']} s, plan checks: {'ok' if plan.verify() == [] else plan.verify()}",
                  flush=True)

    # the same configuration through the plan database, as the campaign does it: rank 0 writes the
    # five ablation plans (a second call would find them: "bypass"), every rank then measures them
    import torch.distributed as dist
    exp_config = Evaluation_Configs(plan_type="ILP", MAX_QUEUE_SIZE=100, fob=0, hierarchy=1, transform_mode="greedy")
    if rank == 0:
        generate_intra_bsa_execution_plans(exp_config, da_config, prof_db, False)
    dist.barrier(gloo_group)
    generate_intra_bsa_execution_plans(exp_config, da_config, prof_db, True)      # bypass mode: all stored
    measured = profile_all_intra_BSA(None, exp_config, da_config, ncclcomm_global, gloo_group, None, prof_db)
    if rank == 0:
        print(f"database: {len(measured)} ablation plans measured", flush=True)


if __name__ == "__main__":
    main()
