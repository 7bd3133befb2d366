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
import os
import time
from pathlib import Path

import numpy as np
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


def profile_kernels(out_dir: Path, quick: bool) -> Path:
    """Tile grid: Smin in 256..64k, Sq/Skv ratios p/q with max(p, q) <= 8, full and causal,
    Nh in {1, 32}. Writes ``time_b200_flash_all.json``."""
    dev = torch.device("cuda")
    sizes = [256, 1024, 4096, 16384] if quick else [256 << i for i in range(9)]
    ratios = ["1/1", "2/1", "1/2"] if quick else ["1/1", "2/1", "1/2", "4/1", "1/4", "8/1", "1/8", "3/1", "1/3"]
    rows = []
    for nh in ([32] if quick else [1, 32]):
        for smin in sizes:
            for ratio in ratios:
                p, q_ = (int(x) for x in ratio.split("/"))
                sq, skv = (smin * p // q_, smin) if p >= q_ else (smin, smin * q_ // p)
                if max(sq, skv) > 131072 or sq * skv * nh > (1 << 38):
                    continue
                for causal in ([False, True] if ratio == "1/1" else [False]):
                    fwd, bwd = _setup(sq, skv, nh, causal, dev)
                    tf, tb = _time(fwd), _time(bwd)
                    fl = 4.0 * sq * skv * 128 * nh * (0.5 if causal else 1.0)
                    rows.append([[smin, 1, nh, 128, ratio, causal],
                                 [tf * 1e6, tb * 1e6, fl / tf / 1e12, 2.5 * fl / tb / 1e12]])
                    print(rows[-1], flush=True)
    out_dir.mkdir(parents=True, exist_ok=True)
    path = out_dir / "time_b200_flash_all.json"
    path.write_text(json.dumps({"flash_attn": rows}, indent=1))
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernels", action="store_true")
    ap.add_argument("--comm", action="store_true")
    ap.add_argument("--out", default="logs/m_configs")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--one", choices=["fwd", "bwd", "gemm"], default=None)
    ap.add_argument("--S", type=int, default=16384)
    ap.add_argument("--Nh", type=int, default=32)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
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
        print(profile_kernels(Path(a.out), a.quick))
    if a.comm:
        profile_comm(Path(a.out), a.quick)


if __name__ == "__main__":
    main()
