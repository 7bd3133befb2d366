"""Kernel-tile execution on a Y x X rank grid (gather, one launch, merge / reduce-scatter) on gloo
CPU ranks against dense attention."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, cases, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = {f"{Y}x{X}-{causal}": _one_grid(rank, world, Y, X, causal) for Y, X, causal in cases}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def _one_grid(rank, world, Y, X, causal):
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.planner import Fused_Execution_Plan
    from ultraattn_b200.runtime.grid import GridExecutor
    S, H, Hk, D = 256, 4, 2, 16
    g = torch.Generator().manual_seed(7)
    q, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(2))
    k, v = (torch.randn(1, S, Hk, D, generator=g) for _ in range(2))
    sl = slice(rank * S // world, (rank + 1) * S // world)
    ex = GridExecutor.from_plan(Fused_Execution_Plan(Y, X, None, 0, causal=causal), device=torch.device("cpu"))
    assert ex.row_chunks == list(range(rank // X * X, rank // X * X + X))
    o, lse = ex.forward(q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous())
    dq, dk, dv = ex.backward(d_o[:, sl].contiguous(), q[:, sl].contiguous(), k[:, sl].contiguous(),
                             v[:, sl].contiguous(), o, lse)
    pat = P.causal(1) if causal else P.full(1)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q, k, v, d_o, pat)
    return max((o - o_ref[:, sl]).abs().max().item(), (lse - lse_ref[:, :, sl]).abs().max().item(),
               (dq - dq_ref[:, sl]).abs().max().item(), (dk - dk_ref[:, sl]).abs().max().item(),
               (dv - dv_ref[:, sl]).abs().max().item())


def test_grid_executor_world4():
    """2 x 2 (full and causal), 4 x 1 (keys / values move) and 1 x 4 (queries move, causal)."""
    cases = [(2, 2, False), (2, 2, True), (4, 1, False), (1, 4, True)]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(4, 29300 + os.getpid() % 90, cases, ret), nprocs=4, join=True)
    for r in range(4):
        assert isinstance(ret[r], dict), ret[r]
        for name, err in ret[r].items():
            assert err < 2e-4, (r, name, err)


def _api_worker(rank, world, port, ret):
    """The reference-named entry points: carriers through the kernel-tile functions, and the
    autograd class on a launch plan."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import orchestrated_attn as OA
        from orchestrated_attn.orchestrated_attn_impl import fused_attn_backward, fused_attn_forward
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.planner import Fused_Execution_Plan, make_plan_collective
        S, H, D = 128, 2, 16
        Sl = S // world
        g = torch.Generator().manual_seed(8)
        q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
        sl = slice(rank * Sl, (rank + 1) * Sl)
        o_ref, lse_ref, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q, k, v, d_o, P.full(1))
        plan = Fused_Execution_Plan(1, 2, None, 0)
        f32 = torch.float32
        ir = OA.Input_Row_Fwd.from_shapes(1, Sl, Sl, H, H, D, f32, device="cpu")
        ic = OA.Input_Col_Fwd.from_shapes(1, Sl, Sl, H, H, D, f32, device="cpu")
        ir.Q.copy_(q[:, sl]); ic.K.copy_(k[:, sl]); ic.V.copy_(v[:, sl])
        out = fused_attn_forward(plan, ir, ic)
        err = [(out.O - o_ref[:, sl]).abs().max().item()]
        irb = OA.Input_Row_Bwd.from_shapes(1, Sl, Sl, H, H, D, f32, device="cpu")
        irb.Q.copy_(q[:, sl]); irb.dO.copy_(d_o[:, sl]); irb.lse.copy_(out.lse)
        r, c = fused_attn_backward(plan, irb, ic, out)
        err += [(r.dQ - dq_ref[:, sl]).abs().max().item(), (c.dK - dk_ref[:, sl]).abs().max().item(),
                (c.dV - dv_ref[:, sl]).abs().max().item()]
        # autograd class on a launch plan (causal, row-owner allocation)
        kw = dict(pattern=P.causal(1), cp=world, seq_len=S, n_heads=H, head_dim=D, allocation="naive",
                  plan_type="Flexflow")
        plans = {"fwd": make_plan_collective(fob=0, **kw), "bwd": make_plan_collective(fob=1, **kw)}
        ql, kl, vl = (t[:, sl].clone().requires_grad_() for t in (q, k, v))
        o = OA.OrchestratedAttnFunc.apply(ql, kl, vl, None, plans)
        o.backward(d_o[:, sl])
        o_c, _, dq_c, dk_c, dv_c = P.dense_attention_with_grads(q, k, v, d_o, P.causal(1))
        err += [(o - o_c[:, sl]).abs().max().item(), (ql.grad - dq_c[:, sl]).abs().max().item(),
                (kl.grad - dk_c[:, sl]).abs().max().item(), (vl.grad - dv_c[:, sl]).abs().max().item()]
        # context-parallel runtime with the ownership chosen by the remap stage
        from ultraattn_b200.runtime import ContextParallelAttention
        pat = P.strided(8, 4, 2)
        rt = ContextParallelAttention(pat, S, H, D, device=torch.device("cpu"), path="nccl", dtype=torch.float32,
                                      plan_time_limit=3.0, cmap="search")
        blk = S // rt.table.shape[0]
        idx = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in range(rt.table.shape[0]) if rt.cmap[b] == rank])
        ql, kl, vl = (t[:, idx].clone().requires_grad_() for t in (q, k, v))
        o = rt(ql, kl, vl)
        o.backward(d_o[:, idx])
        o_s, _, dq_s, dk_s, dv_s = P.dense_attention_with_grads(q, k, v, d_o, pat)
        err += [(o - o_s[:, idx]).abs().max().item(), (ql.grad - dq_s[:, idx]).abs().max().item(),
                (kl.grad - dk_s[:, idx]).abs().max().item(), (vl.grad - dv_s[:, idx]).abs().max().item()]
        ret[rank] = max(err)
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def test_reference_named_entry_points_world2():
    port = 29200 + os.getpid() % 90
    ret = mp.Manager().dict()
    mp.spawn(_api_worker, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], float), ret[r]
        assert ret[r] < 2e-4, (r, ret[r])
