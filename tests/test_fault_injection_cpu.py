"""Failure detection, exercised on the host only: a dropped message and a rank that raises make
the other rank's step fail with a clear error within its deadline instead of hanging."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, mode, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.planner import make_plan_collective
        from ultraattn_b200.runtime import FaultInjector, PlanExecutor
        plan = make_plan_collective(pattern=P.causal(1), cp=2, seq_len=256, n_heads=2, head_dim=16, fob=0,
                                    allocation="naive", plan_type="Flexflow")
        msg = next(k for k in plan.valid_kernels if k.type == "comm" and k.key[5] == "i")
        fault = None
        if mode == "drop" and rank == msg.key[3]:
            fault = FaultInjector(drop_keys=[msg.key])          # the sender silently loses a message
        if mode == "raise" and rank == msg.key[3]:
            fault = FaultInjector(raise_before=msg.key)         # the sender dies before sending
        ex = PlanExecutor(plan, None, device=torch.device("cpu"), recv_timeout_s=3.0, fault=fault)
        q = torch.randn(1, 128, 2, 16)
        try:
            ex.forward(q, q.clone(), q.clone())
            ret[rank] = "completed"
        except TimeoutError as e:
            ret[rank] = f"timeout: {e}"
        except RuntimeError as e:
            ret[rank] = f"error: {e}"
    finally:
        dist.destroy_process_group()


def _run(mode):
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, 29850 + os.getpid() % 50 + (7 if mode == "raise" else 0), mode, ret),
             nprocs=2, join=True)
    return dict(ret)


def test_dropped_message_is_detected():
    res = _run("drop")
    assert any(v.startswith("timeout") for v in res.values()), res


def test_failing_rank_is_detected():
    res = _run("raise")
    assert any("injected failure" in v for v in res.values()), res
    assert any(v.startswith("timeout") or v.startswith("error") for v in res.values()), res
