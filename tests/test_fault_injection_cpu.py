"""Failure detection, exercised on the host only: a dropped message and a rank that raises make
the other rank's step fail with a clear error within its deadline instead of hanging."""
import os

import pytest
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


def _replan_worker(rank, world, port, ret):
    import os, sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.runtime import ContextParallelAttention
        S, H, D = 512, 2, 16
        pat = P.causal(1)
        g = torch.Generator().manual_seed(5)
        q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
        o_ref, _, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q, k, v, d_o, pat)

        def run(rt, r, w):
            sl = slice(r * S // w, (r + 1) * S // w)
            ql, kl, vl = (t[:, sl].clone().requires_grad_() for t in (q, k, v))
            o = rt(ql, kl, vl)
            o.backward(d_o[:, sl])
            return max((o - o_ref[:, sl]).abs().max().item(), (ql.grad - dq_ref[:, sl]).abs().max().item(),
                       (kl.grad - dk_ref[:, sl]).abs().max().item(), (vl.grad - dv_ref[:, sl]).abs().max().item())

        from ultraattn_b200.runtime.heartbeat import StepHeartbeat
        hb = StepHeartbeat()
        rt = ContextParallelAttention(pat, S, H, D, device=torch.device("cpu"), path="nccl", dtype=torch.float32,
                                      plan_time_limit=3.0)
        hb.beat(0)
        assert hb.missing(0, timeout_s=20.0) == []
        err = run(rt, rank, world)
        # between two steps rank 2 says good-bye and rank 3 just stops announcing; the survivors
        # notice on the host before launching anything, re-plan for two ranks and go on
        if rank == 2:
            hb.leave()
        if rank < 2:
            hb.beat(1)
            assert hb.missing(1, timeout_s=1.5) == [2, 3] and hb.alive == [0, 1]
            sub = dist.new_group(hb.alive, use_local_synchronization=True)
            rt2 = rt.replan(sub)
            assert rt2.world == 2 and rt2.table.shape[0] >= 2
            err = max(err, run(rt2, rank, 2))
        ret[rank] = err
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def test_survivors_replan_after_ranks_leave():
    import os
    port = 29400 + os.getpid() % 90
    ret = mp.Manager().dict()
    mp.spawn(_replan_worker, args=(4, port, ret), nprocs=4, join=True)
    for r in range(4):
        assert isinstance(ret[r], float), ret[r]
        assert ret[r] < 2e-4, (r, ret[r])


def test_heartbeat_survivors_adopt_one_member_list():
    """A rank whose announcement lands between two survivors' scans must not split them: the first
    survivor to finish publishes its member list, the others adopt it, and the late rank learns
    that it is out."""
    from ultraattn_b200.runtime.heartbeat import ExcludedFromGroup, StepHeartbeat
    store = dist.HashStore()
    hbs = [StepHeartbeat(store, rank=r, world=4, prefix="t") for r in range(4)]
    for hb in hbs[:3]:
        hb.beat(7)
    assert hbs[0].missing(7, timeout_s=0.2) == [3] and hbs[0].alive == [0, 1, 2]     # rank 3 is late
    hbs[3].beat(7)                                  # ... and announces just now
    # rank 1's own scan sees all four, but it adopts the list rank 0 published
    assert hbs[1].missing(7, timeout_s=0.2) == [3] and hbs[1].alive == [0, 1, 2]
    assert hbs[2].missing(7, timeout_s=0.2) == [3] and hbs[2].alive == [0, 1, 2]
    with pytest.raises(ExcludedFromGroup):
        hbs[3].missing(7, timeout_s=0.2)
