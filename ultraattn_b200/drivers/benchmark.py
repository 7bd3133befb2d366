"""Measurement harness of the campaign (reference: search_algo/benchmark.py:85-229, 336-619).

``benchmark_ops`` times a callable: warm-up, then ``num_iter`` calls bracketed by CUDA events on the
launching stream (wall clock on CPU ranks), repeated ``repeats`` times, last value kept, MAX over
ranks. The reference lines the ranks up with an 8 GiB NCCL all-reduce before each timing
(benchmark.py:593-594) so that the CPU can queue the kernels ahead of the GPU; a barrier plus
device synchronisation lines the ranks up here, and ``start_gate=True`` adds the run-ahead: the
stream is held at a bounded device-side wait (:class:`ultraattn_b200.ops.gate.StartGate`) while
the calls are queued, then released, so launch latency stays out of the measurement of short
kernels.
Optional torch.profiler -> TensorBoard traces follow the reference's schedule (wait 4, warm-up 4,
active 12).
"""
from __future__ import annotations

import time
from typing import Callable, Optional

import torch
import torch.distributed as dist

from ..utils.misc import calc_flops


def benchmark_ops(fn: Callable[[], object], warmup: int = 3, num_iter: int = 4, repeats: int = 3,
                  device: Optional[torch.device] = None, group=None, tb_dir: Optional[str] = None,
                  trace_name: str = "trace", start_gate: bool = False) -> float:
    """Seconds per call, max over the ranks of ``group``."""
    cuda = device is not None and device.type == "cuda"
    gate = None
    if start_gate and cuda:
        from ..ops.gate import StartGate
        gate = StartGate(device)

    def sync():
        if dist.is_initialized():
            dist.barrier(group)
        if cuda:
            torch.cuda.synchronize(device)

    for _ in range(warmup):
        fn()
    if tb_dir:
        from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if cuda else [])
        with profile(activities=acts, schedule=schedule(wait=4, warmup=4, active=12, repeat=1),
                     on_trace_ready=tensorboard_trace_handler(tb_dir, worker_name=trace_name),
                     record_shapes=True, profile_memory=True, with_stack=True) as prof:
            for i in range(20):
                fn()
                if i % 4 == 3:
                    sync()
                prof.step()
    td = 0.0
    for _ in range(repeats):
        sync()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if gate is not None:
                gate.close()
            e0.record()
            for _ in range(num_iter):
                fn()
            e1.record()
            if gate is not None:
                gate.open()
            sync()
            if gate is not None:
                gate.check()
            td = e0.elapsed_time(e1) / 1e3 / num_iter
        else:
            t0 = time.perf_counter()
            for _ in range(num_iter):
                fn()
            sync()
            td = (time.perf_counter() - t0) / num_iter
    if dist.is_initialized():
        t = torch.tensor([td], dtype=torch.float64, device=device if cuda else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        td = float(t.item())
    return td


def benchmark_orchestrate_bsa(plan_fwd, plan_bwd, fob: int, device: torch.device, group=None,
                              dtype=None, warmup: int = 2, num_iter: int = 2, repeats: int = 2,
                              p2p_groups=None, tb_dir=None) -> dict:
    """Execute a plan on the ranks of ``group`` with random inputs and time the pass ``fob``.
    Returns {'time': s, 'hfu': TFLOP/s per rank, 'sim_time': the plan's predicted makespan}."""
    from ..runtime.executor import PlanExecutor
    da = plan_fwd.da_config
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    ex = PlanExecutor(plan_fwd, plan_bwd, group=group, device=device, p2p_groups=p2p_groups)
    S_loc = da.S[0] // ex.cp
    g = torch.Generator(device="cpu").manual_seed(ex.rank)
    mk = lambda h: torch.randn(da.bs, S_loc, h, da.D, generator=g).to(dtype).to(device)
    q, k, v, d_o = mk(da.Nh[0]), mk(da.Nh[1]), mk(da.Nh[1]), mk(da.Nh[0])
    o, lse = ex.forward(q, k, v)
    if fob == 0:
        fn = lambda: ex.forward(q, k, v)
    else:
        fn = lambda: ex.backward(d_o, q, k, v, o, lse)
    t = benchmark_ops(fn, warmup, num_iter, repeats, device, group, tb_dir)
    _, hw = calc_flops(da.bs, da.S, da.Nh[0], da.D, False, fob, da.bsa_config.total_sparsity)
    plan = plan_fwd if fob == 0 else plan_bwd
    return {"time": t, "hfu": hw / t / ex.cp / 1e12, "sim_time": float(plan.end_time)}


def benchmark_orchestrate_bsa_reference_form(args, raw_f, da_config, exp_config, tensor_buf, inter_bsa_execution_plans,
                                             inter_comp_plans_dicts, warmup: int = 11, num_iter: int = 20,
                                             log: bool = True, global_group=None, ncclcomm_global=None,
                                             use_cudagraph: bool = False, mode: str = "test") -> list:
    """The harness with the reference's argument list (search_algo/benchmark.py:336-619): a list
    of inter-level plans, each with the dict of intra-level plans its compute kernels stand for,
    measured for the pass ``exp_config.fob``; returns one ``{'hfu': TFLOP/s per rank, 'time': '%.3e'}``
    per plan on rank 0 and ``None`` elsewhere. ``raw_f`` and ``tensor_buf`` (the reference's attention
    callable and its one big buffer that every tile aliases) are accepted and not used: the plans
    run on :class:`ultraattn_b200.runtime.PlanExecutor` with tensors of their own. One node per
    inter-level plan (its single compute kernel = the intra-level plan); for more nodes use
    ``make_plan(..., cp_inter=n)`` and the short form."""
    from ..planner.graph import Dependent_Graph
    from ..planner.schedule import Execution_Plan
    assert len(inter_bsa_execution_plans) == len(inter_comp_plans_dicts), \
        "inter_bsa_execution_plans and inter_comp_plans_dicts must correspond one to one"
    fob = int(exp_config.fob)
    cuda = torch.cuda.is_available() and dist.is_initialized() and dist.get_backend(global_group) == "nccl"
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    rank = dist.get_rank() if dist.is_initialized() else 0
    out = []
    for inter_plan, comp_plans in zip(inter_bsa_execution_plans, inter_comp_plans_dicts):
        assert len(inter_plan.gpu_kernel_lists) == 1 and len(comp_plans) == 1, \
            "this form covers one node per inter-level plan"
        plan = next(iter(comp_plans.values()))
        if fob == 0:
            plan_f, plan_b = plan, None
        else:
            # the backward needs a forward result: plan the forward on the same allocation
            plan_f = Execution_Plan(Dependent_Graph(plan.d_graph.schedule, 0), 0, "Flexflow")
            plan_b = plan
        res = benchmark_orchestrate_bsa(plan_f, plan_b, fob, device, global_group,
                                        warmup=min(int(warmup), 3), num_iter=max(1, min(int(num_iter), 4)), repeats=1)
        if rank == 0:
            if log:
                print(f"hfu: {res['hfu']:.3f} Tflops/s, {1.0 / res['time']:.3f} iter/s, {res['time']:.3e} s/iter", flush=True)
            out.append({"hfu": round(res["hfu"], 3), "time": f"{res['time']:.3e}"})
        else:
            out.append(None)
    return out
