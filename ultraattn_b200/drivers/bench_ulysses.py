"""Time the head-parallel (Ulysses) attention block with the all-to-alls fused into the projection
GEMMs against the same block with plain GEMMs and ``all_to_all`` collectives.

    torchrun --nproc-per-node N -m ultraattn_b200.drivers.bench_ulysses [--seq 131072] [--iters 3]

Llama-2-7B attention block (hidden 4096, 32 heads of 128, RoPE, dense causal mask by default),
forward + backward per step, bf16. Prints one JSON line per variant with the device time (max over
ranks) and, for the fused variant, the bytes its GEMM epilogues / prologues move over NVLink per
rank and step. The unfused variant is the structure of the reference's Ulysses baseline
(head_parallel_attn/deepspeed_ulysses_attn.py:10-198 with comm_lib/comm_utils.py:32-45).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import patterns as P
from ..ops import attention as A
from ..ops import elementwise as E
from ..parallel.ulysses_fused import FusedUlyssesAttention, unfused_reference


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=131072)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--pattern", default="causal", choices=["causal", "full", "global_local"])
    ap.add_argument("--with-peer-gather", action="store_true",
                    help="also time the fused block whose gather GEMMs read the owners' buffers directly")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    import datetime
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    group = dist.group.WORLD
    S, Hd, H = a.seq, a.hidden, a.heads
    S_loc = S // world
    pattern = {"causal": lambda: P.causal(1), "full": lambda: P.full(1),
               "global_local": lambda: P.global_local(32, 1, 2)}[a.pattern]()
    gen = torch.Generator(device=dev).manual_seed(5 + rank)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=gen, device=dev) * s).to(torch.bfloat16)
    x, dy = rnd(S_loc, Hd, s=0.5), rnd(S_loc, Hd, s=0.5)
    wqkv, wo = rnd(3 * H * 128, Hd, s=0.02), rnd(Hd, H * 128, s=0.02)
    cos, sin = E.rope_tables(S, 128, 10000.0, dev)
    blocks = {"fused": FusedUlyssesAttention(group, dev, S, Hd, H, pattern=pattern)}
    if a.with_peer_gather:
        blocks["fused, gathers read peer memory directly"] = FusedUlyssesAttention(
            group, dev, S, Hd, H, pattern=pattern, gather="peer")

    def step(variant: str):
        xl = x.detach().requires_grad_()
        w1 = wqkv.detach().requires_grad_()
        w2 = wo.detach().requires_grad_()
        y = blocks[variant](xl, w1, w2, cos, sin) if variant in blocks else \
            unfused_reference(xl, w1, w2, group, H, H, 128, pattern, cos, sin)
        y.backward(dy)

    n = pattern.table.shape[0]
    attn_flops = pattern.volume * (S / n) ** 2 * 4 * 128 * H * 3.5 / world
    gemm_flops = 2.0 * S_loc * Hd * (3 * H * 128 + H * 128) * 3
    for name in ["unfused"] + list(blocks):
        fused = name in blocks
        for _ in range(2):
            step(name)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            step(name)
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        A.check_status(dev)
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            rec = {"block": "ulysses attention fwd+bwd", "variant": name, "n_gpus": world, "S": S, "hidden": Hd,
                   "heads": H, "pattern": a.pattern, "ms": round(t.item(), 3),
                   "hw_tflops_per_gpu": round((attn_flops + gemm_flops) / t.item() / 1e9, 1)}
            if fused:
                rec["nvlink_bytes_per_rank"] = blocks[name].traffic
            print(json.dumps(rec), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
