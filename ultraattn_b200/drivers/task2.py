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


def prepare_inter_comp_plans(inter_plan, prof_db) -> None:
    """Attach to every inter-level compute kernel the intra-level plan that implements it."""
    for k in inter_plan.valid_kernels:
        if k.type == "comp" and isinstance(k.comp_map_key, str):
            k.execution_plan = prof_db.get_plan(k.comp_map_key, 1)


def step4_profile_inter_bsa_exe_plans(space, prof_db, world: int) -> None:
    if dist.is_initialized() and dist.get_rank() != 0:
        return
    for fob in space.fobs:
        for cfg in space.inter_bsa_configs:
            if cfg.CP[0] * cfg.CP[1] != world:
                continue
            for shape in space.shape_configs(world):
                prefix = plan_key_prefix(fob, cfg.CP, shape, cfg)
                for suf in ABLATION_SUFFIXES:
                    intra = prof_db.get_profile(prefix + suf, 1)
                    if intra is not None and cfg.CP[1] == 1:
                        prof_db.put_profile(prefix + suf, intra["hfu"], float(intra["time"]),
                                            float(intra["sim_time"]), 0)


def main(argv=None) -> None:
    args = parse_args(argv)
    info = initialize_distribution()
    prof_db = Prof_DB(os.environ.get("CLUSTER_NAME"), os.environ.get("PLATFORM"))
    space = step0_top_down_decompose(args.exp_class or "bsa_train", max_intra=info["tasks_per_node"],
                                     max_nodes=info["node_num"], quick=bool(args.extra.get("quick")))
    step4_profile_inter_bsa_exe_plans(space, prof_db, info["world_size"])
    print_rank_0("task2 done")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
