"""End-to-end training step of the Llama-2 style model with context-parallel block-sparse attention.

    torchrun --nproc-per-node 8 -m ultraattn_b200.drivers.train_llama --seq 524288 --steps 2

Default: Llama2-7B shape (32 layers, hidden 4096, 32 heads x 128, FFN 11008, vocab 32000), random
init N(0, 0.02), bf16 with fp32 Adam sharded over the ranks, attention-aware activation
checkpointing, one sequence of ``--seq`` token ids (uniform over the vocabulary, seed 3) sharded
over the ranks, global+local block-sparse mask (32 blocks, block 0 global, causal window 2).
Prints one JSON line with tokens/s (whole job), device-timed, max over ranks. The reference has no
trainer; its end-to-end figures add a constant to attention time (plot/e2e_pick.py:13-31).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import patterns as P
from ..models.llama import LlamaConfig, LlamaModel
from ..ops import attention as A
from ..runtime import ContextParallelAttention


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=524288)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--blocks", type=int, default=32)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--path", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--offload-checkpoints", action="store_true",
                    help="keep the per-layer activation checkpoints in pinned host memory")
    ap.add_argument("--estimate-memory", type=int, default=0, metavar="CP",
                    help="print the per-GPU memory plan for CP ranks and exit (needs no GPU)")
    a = ap.parse_args()
    if a.estimate_memory:
        from ..models.llama import estimate_memory
        plan = estimate_memory(LlamaConfig(n_layers=a.layers, hidden=a.hidden, n_heads=a.heads, head_dim=128,
                                           ffn=a.ffn, vocab=a.vocab), a.seq, a.estimate_memory, a.offload_checkpoints)
        print(json.dumps({k: round(v, 2) if isinstance(v, float) else v for k, v in plan.items()}))
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
        group = dist.group.WORLD
    cfg = LlamaConfig(n_layers=a.layers, hidden=a.hidden, n_heads=a.heads, head_dim=128, ffn=a.ffn, vocab=a.vocab)
    pattern = P.global_local(a.blocks, 1, 2)
    runtime = None
    if world > 1:
        runtime = ContextParallelAttention(pattern, a.seq, a.heads, 128, group=group, device=dev, path=a.path)
        cmap = runtime.cmap
        par_d = runtime.table.shape[0]
        blk = a.seq // par_d
        mine = [b for b in range(par_d) if cmap[b] == rank]
        pos = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in mine])
    else:
        pos = torch.arange(a.seq)
    model = LlamaModel(cfg, device=dev, pattern=pattern, runtime=runtime, group=group, seed=0,
                       offload_checkpoints=a.offload_checkpoints)
    g = torch.Generator().manual_seed(3)
    ids_all = torch.randint(0, a.vocab, (a.seq + 1,), generator=g)
    ids = ids_all[pos].to(dev)
    targets = ids_all[pos + 1].to(dev)
    pos_dev = pos.to(dev)

    def step():
        return model.train_step(ids, targets, pos_dev, n_total_tokens=a.seq)

    loss = None
    for _ in range(a.warmup):
        loss = step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    A.check_status(dev)
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        n_params = model.flat.numel()
        print(json.dumps({"metric": "e2e_tokens_per_s", "value": a.seq / (ms.item() / 1e3), "ms_per_step": ms.item(),
                          "n_gpus": world, "seq_len": a.seq, "layers": a.layers, "params": n_params, "loss": loss,
                          "path": a.path if world > 1 else "local", "dtype": "bf16",
                          "max_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
