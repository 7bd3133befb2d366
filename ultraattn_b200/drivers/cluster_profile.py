"""Machine micro-profiles for the cost model: kernel grid and link bandwidth.

Equivalent of the reference's ``make cluster_profile`` (scripts/Makefile:90-96), which runs two
external tools that are not part of its tree (``kernel_profiler`` -> ``time_*.json`` and
``comm_test`` -> ``cb_8_*.log`` / ``cb_16_*.log``). Both outputs keep the reference's formats
(parsers: search_algo/utils.py:229-272), so they drop into ``database/<cluster>/<platform>/m_configs``.

    python -m ultraattn_b200.drivers.cluster_profile --kernels --out logs/m_configs [--quick]
    torchrun --nproc-per-node 2 -m ultraattn_b200.drivers.cluster_profile --comm --out logs/m_configs

``--one fwd|bwd --S .. --Nh ..`` runs a single shape a few times (the workload used for ncu
captures of the attention kernels).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def _time(fn, iters=5, warmup=2) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters / 1e3


def _setup(sq, skv, nh, causal, dev):
    from ..ops import attention as A
    from ..ops import elementwise as E
    g = torch.Generator(device=dev).manual_seed(0)
    mk = lambda s: torch.randn(1, s, nh, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, d_o = mk(sq), mk(skv), mk(skv), mk(sq)
    rows = [A.Row(0, 0, sq, (A.Seg(0, 0, skv, causal, 0),), 0, 0, False)]
    cols = [A.Col(0, 0, skv, (A.Seg(0, 0, sq, causal, 0),), 0, 0)]
    fp, bp = A.FwdPlan(rows, dev), A.BwdPlan(cols, dev)
    o = torch.empty_like(q)
    lse = torch.empty(1, nh, sq, device=dev, dtype=torch.float32)
    A.attn_fwd([q], [k], [v], [(o, lse)], fp)
    dvec = E.rowdot(o[0], d_o[0]).unsqueeze(0)
    dq = torch.zeros(1, sq, nh, 128, device=dev, dtype=torch.float32)
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    fwd = lambda: A.attn_fwd([q], [k], [v], [(o, lse)], fp)
    bwd = lambda: A.attn_bwd([A.BwdQSide(q, d_o, lse, dvec, dq)], [k], [v], [A.BwdKvOut(dk, dv)], bp)
    return fwd, bwd


def profile_kernels(out_dir: Path, quick: bool, max_seconds: float = 0.0) -> Path:
    """Tile grid: Smin in 256..64k, Sq/Skv ratios p/q with max(p, q) <= 8, full and causal,
    Nh in {1, 32}. Writes ``time_b200_flash_all.json`` (rewritten after every few shapes, so an
    interrupted run keeps what it measured; ``max_seconds`` > 0 stops the sweep cleanly). Shapes
    run smallest first within each head count, and 32 heads before 1 (the planner's configs)."""
    import time
    dev = torch.device("cuda")
    sizes = [256, 1024, 4096, 16384] if quick else [256 << i for i in range(9)]
    ratios = ["1/1", "2/1", "1/2"] if quick else ["1/1", "2/1", "1/2", "4/1", "1/4", "8/1", "1/8", "3/1", "1/3"]
    rows = []
    out_dir.mkdir(parents=True, exist_ok=True)
    path = out_dir / "time_b200_flash_all.json"
    t_start = time.time()

    def flush():
        path.write_text(json.dumps({"flash_attn": rows}, indent=1))

    for nh in ([32] if quick else [32, 1]):
        for smin in sizes:
            for ratio in ratios:
                p, q_ = (int(x) for x in ratio.split("/"))
                sq, skv = (smin * p // q_, smin) if p >= q_ else (smin, smin * q_ // p)
                if max(sq, skv) > 131072 or sq * skv * nh > (1 << 38):
                    continue
                for causal in ([False, True] if ratio == "1/1" else [False]):
                    if max_seconds and time.time() - t_start > max_seconds:
                        flush()
                        return path
                    fwd, bwd = _setup(sq, skv, nh, causal, dev)
                    big = sq * skv * nh >= (1 << 34)
                    tf, tb = _time(fwd, 3 if big else 5, 1 if big else 2), _time(bwd, 3 if big else 5, 1 if big else 2)
                    fl = 4.0 * sq * skv * 128 * nh * (0.5 if causal else 1.0)
                    rows.append([[smin, 1, nh, 128, ratio, causal],
                                 [tf * 1e6, tb * 1e6, fl / tf / 1e12, 2.5 * fl / tb / 1e12]])
                    print(rows[-1], flush=True)
                    if len(rows) % 8 == 0:
                        flush()
    flush()
    return path


def profile_comm(out_dir: Path, quick: bool) -> None:
    """Pairwise bidirectional peer bandwidth vs message size through symmetric memory (peer loads,
    the transport of the fused path) — pattern [[0,1],[1,0]] of the reference's conflict bench."""
    import torch.distributed as dist
    from ..parallel.comm import initialize_distribution
    from ..runtime.fused import SymmMemSpace
    info = initialize_distribution()
    dev = torch.device("cuda", info["local_rank"])
    space = SymmMemSpace(dist.group.WORLD, dev)
    max_bytes = 1 << (26 if quick else 29)
    space.alloc("buf", (max_bytes,), torch.uint8)
    space.finalize()
    peer = space.peer("buf", (space.rank + 1) % space.world)
    local = torch.empty(max_bytes, dtype=torch.uint8, device=dev)
    lines = ["[[0, 1], [1, 0]]"]
    size = 8192
    while size <= max_bytes:
        fn = lambda: local[:size].copy_(peer[:size])
        dist.barrier()
        t = _time(fn, 10, 3)
        tt = torch.tensor([t], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t = tt.item()
        gbs = size / t / 1e9
        lines.append(f"SIZE {size // 2}, REAL_BD {2 * gbs:.3f} GB/s, BD/PAIR {gbs:.3f} GB/s, "
                     f"time {t:.3e} s, comm_vol {size / 1e6:.3f} MB")
        size *= 2
    if space.rank == 0:
        out_dir.mkdir(parents=True, exist_ok=True)
        (out_dir / "cb_8_b200_all.log").write_text("\n".join(lines) + "\n")
        (out_dir / "cb_16_b200_all.log").write_text("\n".join(lines) + "\n")
        print("\n".join(lines))
    dist.destroy_process_group()


def profile_comm_fused(out_dir: Path, quick: bool) -> None:
    """The transports of the fused path, every rank active at once (rank r talks to r + 1), device
    time as the max over ranks: (i) staging pulls by peer loads against the number of CTAs that
    copy, (ii) peer ``red.global.add.v4.f32`` pushes, (iii) ``multimem.st`` broadcast and
    ``multimem.ld_reduce`` all-to-one sums through the switch when the allocation has a multicast
    address. One JSON line per point; the table goes to ``fused_comm_b200.json`` beside the link
    logs, where ``planner.cost`` looks for it. Counterpart of the reference's conflict bench
    (third_party/comm_test, outputs prof_data/*/cb_*.log), for transports it does not have."""
    import torch.distributed as dist
    from .. import _lib
    from ..ops import elementwise as E
    from ..parallel.comm import initialize_distribution
    from ..runtime.fused import SymmMemSpace
    info = initialize_distribution()
    dev = torch.device("cuda", info["local_rank"])
    space = SymmMemSpace(dist.group.WORLD, dev)
    nbytes = 1 << (26 if quick else 28)
    space.alloc("buf", (nbytes,), torch.uint8)
    space.alloc("acc", (nbytes // 4,), torch.float32)
    space.finalize()
    nxt = (space.rank + 1) % space.world
    peer_buf, peer_acc = space.peer("buf", nxt), space.peer("acc", nxt)
    local = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    part = torch.ones(nbytes // 4, dtype=torch.float32, device=dev)
    lib = _lib.load()
    stream = lambda: torch.cuda.current_stream(dev).cuda_stream
    rows = []

    def measure(kind, fn, bytes_moved, **extra):
        dist.barrier()
        t = torch.tensor([_time(fn, 5, 2)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rec = {"transport": kind, "ranks": space.world, "bytes": bytes_moved, "ms": round(t.item() * 1e3, 4),
               "gbs_per_rank": round(bytes_moved / t.item() / 1e9, 1), **extra}
        rows.append(rec)
        if space.rank == 0:
            print(json.dumps(rec), flush=True)

    for ctas in (8, 16, 32, 64, 148):
        measure("peer_pull", lambda: _lib.check(lib.ua_peer_pull(local.data_ptr(), peer_buf.data_ptr(), nbytes, ctas,
                                                                 stream()), "ua_peer_pull"), nbytes, copy_ctas=ctas)
    for size in (1 << 22, 1 << 25, nbytes):
        n = size // 4
        measure("peer_red_add_f32", lambda: E.peer_add_(peer_acc[:n], part[:n]), size)
    if space.has_multicast():
        mc = space.multicast_ptr("buf")
        for size in (1 << 22, 1 << 25, nbytes):
            measure("multimem_st_broadcast", lambda: E.multimem_bcast_(mc, local[:size]), size)
        mca = space.multicast_ptr("acc")
        out = torch.empty(nbytes // 4, dtype=torch.float32, device=dev)
        for size in (1 << 22, 1 << 25, nbytes):
            # every rank sums all replicas of its own size-byte window (an all-to-one reduction per rank)
            measure("multimem_ld_reduce_f32", lambda: E.multimem_reduce(mca, out[:size // 4], size, torch.float32, dev), size)
    if space.rank == 0:
        out_dir.mkdir(parents=True, exist_ok=True)
        (out_dir / "fused_comm_b200.json").write_text(json.dumps(rows, indent=0))
    dist.destroy_process_group()


def _profile_memory_bound_ops(rows: int, iters: int) -> None:
    """Time the memory-bound kernels of the model on tensors larger than L2 (``rows`` x 4096 bf16 and
    relatives) and print achieved GB/s (algorithmic bytes / device time) next to the measured copy
    bandwidth from ``MEASURED_PEAKS.json`` when present."""
    from ..ops import elementwise as E
    dev = torch.device("cuda")
    peak = None
    for base in (Path.cwd(), Path(__file__).resolve().parents[2]):
        f = base / "MEASURED_PEAKS.json"
        if f.exists():
            peak = float(json.loads(f.read_text()).get("hbm_gbs", 0.0)) or None
            break
    Hd, F, H = 4096, 11008, 32
    bf = torch.bfloat16
    x = torch.randn(rows, Hd, device=dev, dtype=bf)
    w = torch.ones(Hd, device=dev, dtype=bf)
    g = torch.randn(rows, Hd, device=dev, dtype=bf)
    y, rstd = E.rmsnorm_fwd(x, w, 1e-5)
    gu = torch.randn(rows, 2 * F, device=dev, dtype=bf)
    dy = torch.randn(rows, F, device=dev, dtype=bf)
    q = torch.randn(rows, H, 128, device=dev, dtype=bf)
    cos, sin = E.rope_tables(rows, 128, device=dev)
    pos = torch.arange(rows, device=dev, dtype=torch.int32)
    o1, o2 = torch.randn(2, rows, H, 128, device=dev, dtype=bf)
    l1, l2 = torch.randn(2, H, rows, device=dev, dtype=torch.float32)
    oo, lo = torch.empty_like(o1), torch.empty_like(l1)
    acc = torch.randn(rows, Hd, device=dev, dtype=torch.float32)
    n = rows * Hd
    master, m, v = (torch.zeros(n, device=dev, dtype=torch.float32) for _ in range(3))
    grad, par = torch.randn(n, device=dev, dtype=bf), torch.zeros(n, device=dev, dtype=bf)
    b2, b4 = 2, 4
    ops = [
        ("rmsnorm_fwd", lambda: E.rmsnorm_fwd(x, w, 1e-5), 2 * n * b2),
        ("rmsnorm_bwd", lambda: E.rmsnorm_bwd(x, w, g, rstd), 3 * n * b2 + n * b2),
        ("rope", lambda: E.rope(q, cos, sin, pos), 2 * q.numel() * b2),
        ("swiglu_fwd", lambda: E.swiglu_fwd(gu), 3 * rows * F * b2),
        ("swiglu_bwd", lambda: E.swiglu_bwd(gu, dy), 5 * rows * F * b2),
        ("lse_merge_2way", lambda: E.lse_merge([(o1, l1), (o2, l2)], (oo, lo)), 3 * o1.numel() * b2),
        ("rowdot", lambda: E.rowdot(o1, o2), 2 * o1.numel() * b2),
        ("cast_scale", lambda: E.cast_scale(acc, g), n * (b4 + b2)),
        ("adam", lambda: E.adam_step(master, m, v, grad, par, 1e-4, 0.9, 0.95, 1e-8, 0.0, 1), n * (6 * b4 + 2 * b2)),
    ]
    for name, fn, nbytes in ops:
        t = _time(fn, iters, 2)
        rec = {"op": name, "rows": rows, "ms": t * 1e3, "gbs": nbytes / t / 1e9}
        if peak:
            rec["of_measured_copy_bandwidth"] = rec["gbs"] / peak
        print(json.dumps(rec))


def _profile_gemm_shapes(iters: int = 20) -> None:
    """The GEMM kernel on the projection / FFN shapes of Llama-2-7B at 64k tokens per GPU (and
    8192^3), single-CTA tiles and CTA pairs, next to the library GEMM PyTorch calls (cuBLAS) on
    the same tensors; one JSON line per shape. The variants take turns (five launches each per
    round, ``iters`` launches in total), because under the power cap the clock sags within a few
    hundred milliseconds of load: timed one after the other, whichever variant runs first would
    look fastest."""
    import os
    from ..ops import gemm as G
    dev = torch.device("cuda")
    saved = os.environ.get("UA_GEMM_PAIR")

    def force(value):
        if value is None:
            os.environ.pop("UA_GEMM_PAIR", None)
        else:
            os.environ["UA_GEMM_PAIR"] = value

    for (M, N, K) in [(8192, 8192, 8192), (65536, 4096, 4096), (65536, 12288, 4096), (65536, 22016, 4096),
                      (65536, 4096, 11008)]:
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        force(None)
        G._pair_choice.clear()
        G.gemm(a, b, out=out)                       # the wrapper picks its form for this shape here
        form = "cta_pair" if G._pair_choice.get((M, N, K, False, False)) else "single_cta"
        variants = {
            "single_cta_tflops": ("0", lambda: G.gemm(a, b, out=out)),
            "cta_pair_tflops": ("1", lambda: G.gemm(a, b, out=out)),
            "library_tflops": (None, lambda: torch.matmul(a, b.t(), out=out)),
        }
        spent = {k: 0.0 for k in variants}
        per_round = 5
        rounds = max(1, iters // per_round)
        for rnd in range(rounds + 1):               # round 0 warms up and is not counted
            for name, (env, fn) in variants.items():
                force(env)
                t = _time(fn, per_round, 1 if rnd == 0 else 0)
                if rnd:
                    spent[name] += t
        force(saved)
        rec = {"op": "gemm", "M": M, "N": N, "K": K}
        rec.update({k: round(fl / (v / rounds) / 1e12, 1) for k, v in spent.items()})
        rec["default_form"] = form
        print(json.dumps(rec), flush=True)


def _profile_mma_rate(iters: int = 200) -> None:
    """Clocks per ``tcgen05.mma`` (M = 128, K = 16, bf16) for N = 64 / 128 / 256, operands from
    shared memory (SS) or A from tensor memory (TS), four ways of issuing; one JSON line each."""
    from .. import _lib
    from ..ops import attention as A
    dev = torch.device("cuda")
    out = torch.zeros(2, dtype=torch.int64, device=dev)
    st = A.status_buffer(dev)
    for n in (64, 128, 256):
        for mode in (0, 1):
            for variant in range(4):
                rc = _lib.load().ua_mma_rate(variant, mode, n, iters, out.data_ptr(), st.data_ptr(),
                                             torch.cuda.current_stream(dev).cuda_stream)
                _lib.check(rc, "ua_mma_rate")
                torch.cuda.synchronize()
                A.check_status(dev)
                issue, complete = (x / (8.0 * iters) for x in out.tolist())
                print(json.dumps({"op": "tcgen05.mma", "operands": "TS" if mode else "SS", "N": n, "variant": variant,
                                  "clk_per_mma_issue": round(issue, 1), "clk_per_mma_complete": round(complete, 1)}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernels", action="store_true")
    ap.add_argument("--comm", action="store_true")
    ap.add_argument("--comm-fused", action="store_true",
                    help="peer-load staging vs copy CTAs, peer red.add, multimem broadcast / reduce (all ranks at once)")
    ap.add_argument("--out", default="logs/m_configs")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--max-seconds", type=float, default=0.0, help="(--kernels) stop the sweep after this long")
    ap.add_argument("--one", choices=["fwd", "bwd", "gemm", "gemm_shapes", "ops", "gate", "mma_rate"], default=None)
    ap.add_argument("--S", type=int, default=16384)
    ap.add_argument("--Nh", type=int, default=32)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    if a.one == "ops":
        _profile_memory_bound_ops(a.S, a.iters)
        return
    if a.one == "mma_rate":
        _profile_mma_rate()
        return
    if a.one == "gemm_shapes":
        _profile_gemm_shapes(a.iters)
        return
    if a.one == "gate":
        # small tiles with and without the start gate: what the host launch path adds to a timing
        from .benchmark import benchmark_ops
        dev = torch.device("cuda")
        for S in (256, 512, 1024, 2048, 4096):
            fwd, bwd = _setup(S, S, a.Nh, a.causal, dev)
            for name, fn in (("fwd", fwd), ("bwd", bwd)):
                plain = benchmark_ops(fn, warmup=3, num_iter=50, repeats=2, device=dev)
                gated = benchmark_ops(fn, warmup=3, num_iter=50, repeats=2, device=dev, start_gate=True)
                print(json.dumps({"op": name, "S": S, "Nh": a.Nh, "us_per_launch": round(plain * 1e6, 2),
                                  "us_per_launch_behind_gate": round(gated * 1e6, 2)}), flush=True)
        return
    if a.one:
        dev = torch.device("cuda")
        if a.one == "gemm":
            from ..ops import gemm as G
            x = torch.randn(a.S, 4096, device=dev, dtype=torch.bfloat16)
            w = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
            fn = lambda: G.gemm(x, w)
            fl = 2.0 * a.S * 4096 * 4096
        else:
            fwd, bwd = _setup(a.S, a.S, a.Nh, a.causal, dev)
            fn = fwd if a.one == "fwd" else bwd
            fl = 4.0 * a.S * a.S * 128 * a.Nh * (0.5 if a.causal else 1.0) * (1.0 if a.one == "fwd" else 2.5)
        t = _time(fn, a.iters, 1)
        print(json.dumps({"op": a.one, "S": a.S, "Nh": a.Nh, "causal": a.causal, "ms": t * 1e3,
                          "tflops": fl / t / 1e12}))
        return
    if a.kernels:
        print(profile_kernels(Path(a.out), a.quick, a.max_seconds))
    if a.comm:
        profile_comm(Path(a.out), a.quick)
    if a.comm_fused:
        profile_comm_fused(Path(a.out), a.quick)


if __name__ == "__main__":
    main()
