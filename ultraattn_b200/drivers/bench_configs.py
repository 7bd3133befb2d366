"""Measure the named attention configurations on the GPUs of this job and print one JSON line each.

    torchrun --nproc-per-node N -m ultraattn_b200.drivers.bench_configs [--configs causal128k,strided512k,...]
             [--paths fused,nccl,zigzag,ring] [--iters 3]

Configurations: ``causal128k`` (dense causal, S = 128k, forward + backward), ``strided512k``
(32 blocks of 16k, stride 4, window 2, forward + backward), ``gl512k`` (global+local, block 0
global, causal window 2, forward + backward), ``star512k`` and ``streaming512k`` (prefill, forward
only); all with 32 heads of 128, batch 1, bf16. Paths: ``fused`` (peer-memory kernels), ``nccl``
(plan executed with NCCL messages, launch order by list scheduling; ``nccl-ilp``: by the
kernel-schedule integer program), ``ring`` (K/V ring; under a block-sparse pattern it skips the excluded block pairs) / ``zigzag`` (dense causal),
``grid<Y>x<X>`` (kernel-tile form: gathers, one launch, merge / reduce-scatter; dense patterns only).

Every line carries the device time (max over ranks), the model TFLOP/s per GPU and the achieved
fraction of the roofline = max(FLOPs / measured bf16 peak, bytes that must cross NVLink per GPU /
770 GB/s) / measured time. The peak comes from ``MEASURED_PEAKS.json`` when present.
"""
from __future__ import annotations

import argparse
import json
import math
import os
from pathlib import Path

import torch
import torch.distributed as dist

from .. import patterns as P
from ..ops import attention as A
from ..parallel import ring as R
from ..runtime import ContextParallelAttention

H, D = 32, 128
CONFIGS = {
    "causal128k": (lambda: P.causal(1), 131072, True),
    "strided512k": (lambda: P.strided(32, 4, 2), 524288, True),
    "gl512k": (lambda: P.global_local(32, 1, 2), 524288, True),
    "star512k": (lambda: P.star(32, 1), 524288, False),
    "streaming512k": (lambda: P.streaming(32, 1, 2), 524288, False),
}
NVLINK_GBS = 770.0


def _peak_tflops() -> float:
    for base in (Path.cwd(), Path(__file__).resolve().parents[2]):
        f = base / "MEASURED_PEAKS.json"
        if f.exists():
            return float(json.loads(f.read_text()).get("bf16_tflops", 1590.0))
    return 1590.0


def _timed(fn, iters, dev, world):
    for _ in range(2):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="causal128k,strided512k,star512k,streaming512k")
    ap.add_argument("--paths", default="fused,nccl")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--scale", type=int, default=1, help="divide every sequence length (smoke runs)")
    ap.add_argument("--trace", action="store_true",
                    help="fused path: also print the device time of every phase of a step (slowest rank per phase)")
    ap.add_argument("--metrics-jsonl", default=None, help="append one JSON object per measured call to this file")
    a = ap.parse_args()
    from ..utils.metrics import MetricsLogger
    metrics = MetricsLogger(a.metrics_jsonl) if a.metrics_jsonl else None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    peak = _peak_tflops()
    for name in a.configs.split(","):
        mk, S, train = CONFIGS[name]
        S //= a.scale
        pat = mk()
        S_loc = S // world
        g = torch.Generator(device=dev).manual_seed(rank)
        q, k, v, d_o = (torch.randn(1, S_loc, H, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
                        for _ in range(4))
        n = pat.table.shape[0]
        flops_f = pat.volume * (S / n) ** 2 * 4 * D * H
        flops = flops_f * (3.5 if train else 1.0)
        for path in a.paths.split(","):
            if world == 1 and path != "fused":
                continue
            dense = pat.check_causal() and n == 1 or pat.check_full()
            if (path == "zigzag" or path.startswith("grid")) and not dense:
                continue
            if path.startswith("grid") and math.prod(int(t) for t in path[4:].split("x")) != world:
                continue
            try:
                nvl_bytes = 0.0
                if world == 1:
                    from .. import api
                    fplan, bplan = api.local_plans(pat, S, dev)
                    o = torch.empty_like(q)
                    lse = torch.empty(1, H, S, dtype=torch.float32, device=dev)

                    def step():
                        A.attn_fwd([q], [k], [v], [(o, lse)], fplan)
                        if train:
                            api.local_backward(q, k, v, o, lse, d_o, bplan)
                elif path in ("fused", "nccl", "nccl-ilp"):
                    rt = ContextParallelAttention(pat, S, H, D, device=dev, path=path.split("-")[0], plan_time_limit=15.0,
                                                  plan_type="ILP" if path.endswith("-ilp") else "Flexflow")
                    if path == "fused":
                        im = rt.impl
                        blk_q = im.blk * H * D * 2
                        # bytes this rank pulls over NVLink per step (staging) + pushes (partials)
                        nvl_bytes = len(im.remote_rows) * blk_q * (1 + (3 if train else 0)) \
                            + len(im.remote_cols) * 2 * blk_q * (1 + (2 if train else 0))

                    def step():
                        o_, l_ = rt.forward(q, k, v)
                        if train:
                            rt.backward(d_o, q, k, v, o_, l_)
                elif path.startswith("grid"):
                    # kernel-tile form with NCCL collectives, e.g. grid1x2 = Y 1, X 2 (dense patterns)
                    from ..runtime.grid import GridExecutor
                    Y, X = (int(t) for t in path[4:].split("x"))
                    gx = GridExecutor(Y, X, device=dev, causal=pat.check_causal())

                    def step():
                        o_, l_ = gx.forward(q, k, v)
                        if train:
                            gx.backward(d_o, q, k, v, o_, l_)
                else:
                    kind = path
                    qs, ks, vs = (t.clone().requires_grad_() for t in (q, k, v))
                    # block-sparse patterns: the ring that skips the block pairs the pattern excludes
                    types = None if dense else pat.refined(n * world // math.gcd(n, world))

                    def step():
                        o_, l_ = R.ring_forward(qs.detach(), ks.detach(), vs.detach(), None, kind, pat.check_causal(),
                                                block_types=types)
                        if train:
                            R.ring_backward(d_o, qs.detach(), ks.detach(), vs.detach(), o_, l_, None, kind,
                                            pat.check_causal(), block_types=types)
                ms = _timed(step, a.iters, dev, world)
                A.check_status(dev)
                phases = None
                if a.trace and world > 1 and path == "fused":
                    rt.impl.enable_trace(kernels=True)
                    step()
                    met = rt.impl.metrics()
                    ph = met["phases_ms"]
                    kernels_rank0 = met.get("kernels")
                    rt.impl.enable_trace(False)
                    names = sorted(ph)
                    t = torch.tensor([ph[n] for n in names], device=dev)
                    tmax, tmin = t.clone(), t.clone()
                    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
                    dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
                    phases = {n: [round(lo, 3), round(hi, 3)] for n, lo, hi in zip(names, tmin.tolist(), tmax.tolist())}
                t_comp = flops / world / (peak * 1e12)
                t_link = nvl_bytes / (NVLINK_GBS * 1e9)
                if rank == 0:
                    print(json.dumps({"config": name, "S": S, "path": path if world > 1 else "local", "n_gpus": world,
                                      "ms": round(ms, 3), "model_tflops_per_gpu": round(flops / world / ms / 1e9, 1),
                                      "roofline_ms": round(max(t_comp, t_link) * 1e3, 3),
                                      "roofline_bound": "compute" if t_comp >= t_link else "nvlink",
                                      "fraction_of_roofline": round(max(t_comp, t_link) * 1e3 / ms, 3),
                                      "peak_tflops_of_measured": peak,
                                      **({"phases_ms_min_max_over_ranks": phases,
                                          "kernel_trace_rank0": kernels_rank0} if phases else {})}), flush=True)
                    if metrics is not None:
                        metrics.log(name, ms * 1e-3, flops_per_gpu=flops / world, pull_bytes=int(nvl_bytes),
                                    path=path if world > 1 else "local", n_gpus=world, S=S)
            except Exception as e:  # noqa: BLE001
                if rank == 0:
                    print(json.dumps({"config": name, "path": path, "n_gpus": world, "error": f"{type(e).__name__}: {e}"}),
                          flush=True)
            finally:
                rt = None
                torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
