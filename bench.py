"""Headline benchmark: context-parallel block-sparse attention forward + backward.

Config (fixed): strided block-sparse training attention, S = 512k tokens in 32 blocks of 16k
(query block i attends key block j iff j <= i and (i - j <= 1 or (i - j) % 4 == 0)), 32 heads,
head dim 128, batch 1, bf16, Q/K/V/dO ~ N(0,1) seed 1, context-parallel over N GPUs of one node
(strong scaling: the problem is fixed, N = 1 runs it on one GPU).

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torchrun)
    python bench.py --impl reference ...                      (the reference arm)
    python bench.py --gpus N --e2e-model [--seq-algo ulysses]  (Llama-2-7B training step, tokens/s)

Prints one JSON line on rank 0. ``value`` = milliseconds per forward+backward, device-timed with
CUDA events around exactly K steps, max over ranks. ``e2e`` = the same step through the public
API (``ultraattn_b200.attention``) including, every step, the host-to-device copy of this rank's
Q/K/V/dO shards from pinned memory and the device-to-host read of the step's scalar result.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "cp_attn_fwd_bwd_ms_S512k_strided"
S_TOTAL, N_BLOCKS, N_HEADS, HEAD_DIM = 512 * 1024, 32, 32, 128


def reference_arm(args) -> None:
    """Hands this process over to ``baseline/run_reference.py``: the unmodified reference under
    ``baseline/_ref`` on the same config, N, steps and warm-up, in an interpreter state that cannot
    import this repository's package. That script prints the JSON line (or an ``unavailable`` line
    carrying the exception of the step that failed) and exits 0."""
    runner = os.path.join(ROOT, "baseline", "run_reference.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "search_algo")):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "baseline/_ref is missing: run `python baseline/install_reference.py <reference checkout>`"}))
        return
    cmd = [sys.executable, runner, "--gpus", str(args.gpus), "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--seq", str(args.seq)]
    if args.no_e2e:
        cmd.append("--no-e2e")
    sys.stdout.flush()
    os.execv(sys.executable, cmd)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU execution path: fused peer-memory kernels or the NCCL baseline")
    ap.add_argument("--seq", type=int, default=S_TOTAL, help="(debug) total sequence length")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-model", action="store_true",
                    help="run the other half of the headline metric instead: one Llama-2-7B training step "
                         "(32 layers, global+local mask, S = --seq) over the N GPUs, tokens per second")
    ap.add_argument("--seq-algo", default="cp", choices=["cp", "ulysses"], help="(--e2e-model) sequence parallelism")
    ap.add_argument("--layers", type=int, default=32, help="(--e2e-model) decoder layers")
    ap.add_argument("--check", action="store_true",
                    help="before timing, compare sampled rows of O / lse / dQ / dK / dV at the benchmark shape with an fp32 oracle")
    ap.add_argument("--check-rows", type=int, default=64, help="query rows sampled by --check (whole job)")
    ap.add_argument("--e2e-head-chunks", type=int, default=4,
                    help="end-to-end arm: head groups whose host-to-device copies overlap the compute")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.e2e_model:
        # config 5 of the baseline: end-to-end training step, tokens per second over the whole job
        from ultraattn_b200.drivers import train_llama
        sys.argv = [sys.argv[0], "--seq", str(args.seq), "--steps", str(max(1, args.steps)),
                    "--warmup", str(max(1, min(args.warmup, 2))), "--path", args.path, "--seq-algo", args.seq_algo,
                    "--layers", str(args.layers), "--breakdown"]
        train_llama.main()
        return

    import torch
    import torch.distributed as dist
    import ultraattn_b200 as ua
    from ultraattn_b200 import _lib
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.ops import attention as A

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))

    S = args.seq
    pattern = P.strided(N_BLOCKS, 4, 2)
    S_loc = S // world
    blk = S // N_BLOCKS
    assert N_BLOCKS % world == 0
    owned = list(range(rank * N_BLOCKS // world, (rank + 1) * N_BLOCKS // world))   # contiguous chunks
    KINDS = {"q": 0, "k": 1, "v": 2, "do": 3}

    def gen_block(kind: str, b: int) -> torch.Tensor:
        """Block ``b`` (16k tokens) of one input tensor, N(0,1) in bf16. Every block has its own
        random stream derived from seed 1, so the global tensors are the same for every N and
        any rank can regenerate any block (the sampled check below needs other ranks' keys)."""
        gen = torch.Generator(device=dev).manual_seed(1 + 7919 * KINDS[kind] + 104729 * b)
        out = torch.empty(blk, N_HEADS, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        flat = out.view(-1)
        chunk = 1 << 25
        for off in range(0, flat.numel(), chunk):        # bounded temporary fp32 memory
            n = min(chunk, flat.numel() - off)
            flat[off:off + n] = torch.randn(n, generator=gen, dtype=torch.float32, device=dev).to(torch.bfloat16)
        return out

    # ---- inputs: generated once on the device, kept as pinned host copies (for the end-to-end
    # arm) and as device copies (kernel arm) ----------------------------------------------------
    def make_pair(kind):
        d = torch.empty(1, S_loc, N_HEADS, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        for i, b in enumerate(owned):
            d[0, i * blk:(i + 1) * blk] = gen_block(kind, b)
        h = torch.empty(d.shape, dtype=torch.bfloat16, pin_memory=True)
        h.copy_(d)
        return h, d
    (h_q, q), (h_k, k), (h_v, v), (h_do, d_o) = (make_pair(kd) for kd in ("q", "k", "v", "do"))
    torch.cuda.synchronize()

    if world == 1:
        runtime = None
        fplan, bplan = ua.api.local_plans(pattern, S, dev)
        o = torch.empty_like(q)
        lse = torch.empty(1, N_HEADS, S, dtype=torch.float32, device=dev)

        def step_kernels():
            A.attn_fwd([q], [k], [v], [(o, lse)], fplan)
            return ua.api.local_backward(q, k, v, o, lse, d_o, bplan)
        parallelism = "cp1"
    else:
        from ultraattn_b200.runtime import ContextParallelAttention
        runtime = ContextParallelAttention(pattern, S, N_HEADS, HEAD_DIM, group=dist.group.WORLD,
                                           device=dev, path=args.path)

        def step_kernels():
            o_, lse_ = runtime.forward(q, k, v)
            return runtime.backward(d_o, q, k, v, o_, lse_)
        parallelism = f"cp{world}-{args.path}"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = _lib.LAUNCHES[0]
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms, _lib.LAUNCHES[0] - n0

    # ---- correctness at the benchmark shape: sampled rows against an fp32 oracle --------------
    check = None
    if args.check:
        from ultraattn_b200.utils.sampled_check import SampledCheck, pick_rows
        if world == 1:
            A.attn_fwd([q], [k], [v], [(o, lse)], fplan)
            o_c, lse_c = o, lse
            dq_c, dk_c, dv_c = ua.api.local_backward(q, k, v, o, lse, d_o, bplan)
        else:
            o_c, lse_c = runtime.forward(q, k, v)
            dq_c, dk_c, dv_c = runtime.backward(d_o, q, k, v, o_c, lse_c)
        A.check_status(dev)
        from ultraattn_b200.ops import elementwise as E
        dvec_c = torch.empty(1, N_HEADS, S_loc, dtype=torch.float32, device=dev)         # D = rowsum(dO * O)
        E.rowdot(o_c[0], d_o[0], dvec_c[0])
        if world > 1:       # lse / D of the other ranks' rows (needed by the key-row oracle)
            lse_all = [torch.empty_like(lse_c) for _ in range(world)]
            dvec_all = [torch.empty_like(dvec_c) for _ in range(world)]
            dist.all_gather(lse_all, lse_c.contiguous())
            dist.all_gather(dvec_all, dvec_c)
        else:
            lse_all, dvec_all = [lse_c], [dvec_c]
        local = {"q": q, "k": k, "v": v, "do": d_o}
        per_rank = N_BLOCKS // world

        def get_block(kind, b):
            if b in owned:
                i = owned.index(b)
                return local[kind][0, i * blk:(i + 1) * blk]
            return gen_block(kind, b)

        def stat_block(parts):
            return lambda b: parts[b // per_rank][0, :, (b % per_rank) * blk:(b % per_rank + 1) * blk]

        loc = lambda t: (t // blk - owned[0]) * blk + t % blk            # global token -> index in the shard
        chk = SampledCheck(pattern, S, get_block, head_dim=HEAD_DIM)
        rows = pick_rows(pattern, S, owned, max(8, args.check_rows // world), seed=rank)
        res = chk.check_query_rows(rows, lambda t: (o_c[0, loc(t)], lse_c[0, :, loc(t)], dq_c[0, loc(t)]))
        res.update(chk.check_key_rows(rows[::4], lambda u: (dk_c[0, loc(u)], dv_c[0, loc(u)]),
                                      stat_block(lse_all), stat_block(dvec_all)))
        flat = torch.tensor([res[kk][m] for kk in sorted(res) for m in ("max_abs_over_max_ref", "max_row_relative")],
                            device=dev, dtype=torch.float64)
        cks = torch.stack([o_c.sum(dtype=torch.float64), dq_c.sum(dtype=torch.float64)])
        if world > 1:
            dist.all_reduce(flat, op=dist.ReduceOp.MAX)
            dist.all_reduce(cks)
        it = iter(flat.tolist())
        check = {kk: {"max_abs_over_max_ref": next(it), "max_row_relative": next(it)} for kk in sorted(res)}
        check["rows_per_rank"] = len(rows)
        check["includes_last_token"] = (S - 1) in rows if rank == world - 1 else None
        check["sum_o"], check["sum_dq"] = cks.tolist()          # same data for every N: comparable across N
        worst = max(vv["max_row_relative"] for vv in check.values() if isinstance(vv, dict) and "max_row_relative" in vv)
        check["ok"] = bool(worst < 0.05)
        del o_c, lse_c, dq_c, dk_c, dv_c, dvec_c, lse_all, dvec_all
        torch.cuda.empty_cache()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, launches = timed(step_kernels, args.steps, max(args.warmup, 3))
    A.check_status(dev)
    clocks = sampler.stop() if rank == 0 else None
    # NVLink bytes rank 0 moves per step on the fused path (from the tables its kernels execute)
    traffic = dict(runtime.impl.traffic) if (runtime is not None and args.path == "fused") else None

    # ---- end-to-end arm: public API, H2D of the inputs and D2H of the result every step ---------
    # The heads are independent, so the step runs as `--e2e-head-chunks` calls of the public
    # attention function on head groups; a second stream copies the next group's Q/K/V/dO from
    # pinned memory while the current group computes. Inside the timed region the first group of
    # the NEXT step is fetched while the last group of this step computes (what a training loop's
    # input prefetch does), so only the first timed step's first copy is exposed; nothing is
    # fetched across the warm-up / timed boundary, so every timed step's bytes cross inside the
    # timed region.
    e2e = None
    if not args.no_e2e:
        chunks = max(1, min(args.e2e_head_chunks, N_HEADS))
        assert N_HEADS % chunks == 0
        hc = N_HEADS // chunks
        del q, k, v, d_o
        plan = (runtime.table, runtime.cmap) if runtime is not None else None
        runtime = None
        step_kernels = None
        torch.cuda.empty_cache()
        if world > 1:
            from ultraattn_b200.runtime import ContextParallelAttention
            runtime = ContextParallelAttention(pattern, S, hc, HEAD_DIM, group=dist.group.WORLD,
                                               device=dev, path=args.path, plan=plan)
        # per-group pinned host tensors (a framework user would hold its inputs like this)
        def split(h):
            parts = []
            for c in range(chunks):
                t = torch.empty(1, S_loc, hc, HEAD_DIM, dtype=torch.bfloat16, pin_memory=True)
                t.copy_(h[:, :, c * hc:(c + 1) * hc])
                parts.append(t)
            return parts
        hq, hk, hv, hdo = split(h_q), split(h_k), split(h_v), split(h_do)
        del h_q, h_k, h_v, h_do
        bytes_in = 4 * chunks * hq[0].numel() * 2
        result = {}
        copy_stream = torch.cuda.Stream(device=dev)

        def fetch(c):
            """Start the copies of head group c on the copy stream; returns tensors + event."""
            with torch.cuda.stream(copy_stream):
                t = [h[c].to(dev, non_blocking=True) for h in (hq, hk, hv, hdo)]
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            return t, ev

        e2e_steps, e2e_warmup = max(1, min(args.steps, 3)), 3
        calls = {"n": 0, "ahead": None}

        def step_e2e():
            main = torch.cuda.current_stream(dev)
            calls["n"] += 1
            nxt, calls["ahead"] = calls["ahead"], None
            if nxt is None:
                copy_stream.wait_stream(main)      # the previous step's tensors are released
                nxt = fetch(0)
            # the next step's first group is fetched ahead only from one timed step to the next
            ahead_ok = e2e_warmup < calls["n"] < e2e_warmup + e2e_steps
            for c in range(chunks):
                (qd, kd, vd, wd), ev = nxt
                if c + 1 < chunks:
                    nxt = fetch(c + 1)
                elif ahead_ok:
                    calls["ahead"] = fetch(0)
                main.wait_event(ev)
                for t in (qd, kd, vd, wd):
                    t.record_stream(main)
                qd.requires_grad_(); kd.requires_grad_(); vd.requires_grad_()
                out = ua.attention(qd, kd, vd, pattern, runtime=runtime)
                out.backward(wd)
                if c == 0:
                    chk = qd.grad[0, :64].float().sum()
            # the step's scalar result: a checksum over a slice of dQ, read back to the host
            result["v"] = float(chk.cpu())
        e2e_ms, _ = timed(step_e2e, e2e_steps, e2e_warmup)
        A.check_status(dev)
        e2e = {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": 4,
               "checksum": result.get("v"), "head_chunks": chunks,
               "prefetch": "next head group during compute; next step's first group during the last group (timed steps only)"}

    if rank == 0:
        vol = pattern.volume * (S / N_BLOCKS) ** 2 * 4 * HEAD_DIM * N_HEADS      # forward model FLOPs
        # the backward runs five GEMMs for the forward's two (2.5x, recomputing S) but the model
        # needs only 2x: hardware FLOPs (what the tensor cores did) vs model FLOPs
        hw_tflops = vol * 3.5 / (ms * 1e-3) / 1e12 / world
        model_tflops = vol * 3.0 / (ms * 1e-3) / 1e12 / world
        roof = None
        try:        # achieved fraction of max(FLOPs at the measured GEMM peak, NVLink bytes at link bandwidth)
            from ultraattn_b200.utils.metrics import load_peaks, roofline
            tr = traffic if isinstance(traffic, dict) else {}
            pull = sum(tr.get(k, 0) or 0 for k in ("fwd_pull_bytes", "fwd_multicast_in_bytes", "bwd_pull_bytes"))
            push = sum(tr.get(k, 0) or 0 for k in ("fwd_push_bytes", "fwd_multicast_out_bytes", "bwd_push_bytes"))
            peaks = load_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
            r = roofline(vol * 3.5 / world, max(pull, push), ms * 1e-3, peaks, sustained=True)
            roof = {"bound": r["bound"], "target_ms": r["target_s"] * 1e3, "fraction": r["fraction"],
                    "of": f"{peaks.get('source', 'measured')} sustained bf16 peak {peaks['bf16_tflops_sustained']} TFLOP/s, "
                          "770 GB/s per NVLink direction"}
        except Exception as e:  # noqa: BLE001  (never let the report break the benchmark line)
            roof = {"error": f"{type(e).__name__}: {e}"}
        print(json.dumps({
            "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic N(0,1), seed 1 (one stream per 16k block: the same tensors for every N)",
            "config": {"model": "attention-only (Llama2-7B attention shape: 32 heads x 128)",
                       "pattern": "strided: 32 blocks of 16k, j<=i and (i-j<=1 or (i-j)%4==0)",
                       "global_batch": 1, "seq_len": S, "parallelism": parallelism,
                       "l2": "inputs (4 GiB per tensor in total) far exceed the 126 MB L2; no flush needed"},
            "hw_tflops_per_gpu": hw_tflops, "model_tflops_per_gpu": model_tflops, "check": check, "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "nvlink_bytes_rank0": traffic, "roofline": roof,
            "tokens_per_s": S / (ms * 1e-3) if ms else None,
            "e2e_tokens_per_s": (S / (e2e["value"] * 1e-3)) if isinstance(e2e, dict) and e2e.get("value") else None,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
