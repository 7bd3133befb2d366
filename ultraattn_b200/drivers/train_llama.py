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


def _breakdown(model, step, dev) -> dict:
    """One instrumented step: device time inside the attention calls (context-parallel runtime or
    head-parallel block, forward and backward), inside the GEMM kernel, and the rest."""
    from ..ops import gemm as G
    spans = {"attention": [], "gemm": []}

    def timed(kind, fn):
        def wrapper(*args, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*args, **kw)
            e1.record()
            spans[kind].append((e0, e1))
            return out
        return wrapper

    saved = (model._attn_fwd, model._attn_bwd, G.gemm, G.gemm_scatter, G.gemm_gather)
    model._attn_fwd, model._attn_bwd = timed("attention", saved[0]), timed("attention", saved[1])
    G.gemm, G.gemm_scatter, G.gemm_gather = (timed("gemm", f) for f in saved[2:])
    if model.ulysses is not None:       # head-parallel: the attention kernels are called inside the block
        from ..ops import attention as Aops
        saved_a = (Aops.attn_fwd, Aops.attn_bwd)
        Aops.attn_fwd, Aops.attn_bwd = timed("attention", saved_a[0]), timed("attention", saved_a[1])
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    step()
    t1.record()
    torch.cuda.synchronize(dev)
    model._attn_fwd, model._attn_bwd, G.gemm, G.gemm_scatter, G.gemm_gather = saved
    if model.ulysses is not None:
        Aops.attn_fwd, Aops.attn_bwd = saved_a
    total = t0.elapsed_time(t1)
    out = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in spans.items()}
    out["other"] = total - out["attention"] - out["gemm"]
    out["step"] = total
    return out


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
    ap.add_argument("--seq-algo", default="cp", choices=["cp", "ulysses", "halo"],
                    help="cp: context-parallel attention; ulysses: head-parallel attention with the all-to-alls "
                         "fused into the projection GEMMs; halo: contiguous shards, --sliding-window keys fetched "
                         "from the preceding ranks")
    ap.add_argument("--breakdown", action="store_true",
                    help="after the timed steps, run one more step with CUDA events around the attention calls "
                         "and the GEMMs and report the attention / GEMM / other split")
    ap.add_argument("--offload-checkpoints", action="store_true",
                    help="keep the per-layer activation checkpoints in pinned host memory")
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--kv-heads", type=int, default=None, help="grouped-query attention: key/value heads")
    ap.add_argument("--sliding-window", type=int, default=None,
                    help="Mistral-style token-exact sliding window (one rank; replaces the block pattern)")
    ap.add_argument("--sink-tokens", type=int, default=0, help="with --sliding-window: leading tokens that stay visible")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: fp32 ranks over gloo running the PyTorch restatements of the kernels (small shapes; "
                         "checks the token sharding, the plan execution and the sharded optimizer without a GPU)")
    ap.add_argument("--estimate-memory", type=int, default=0, metavar="CP",
                    help="print the per-GPU memory plan for CP ranks and exit (needs no GPU)")
    a = ap.parse_args()
    if a.estimate_memory:
        from ..models.llama import estimate_memory
        plan = estimate_memory(LlamaConfig(n_layers=a.layers, hidden=a.hidden, n_heads=a.heads, head_dim=a.head_dim,
                                           ffn=a.ffn, vocab=a.vocab), a.seq, a.estimate_memory, a.offload_checkpoints)
        print(json.dumps({k: round(v, 2) if isinstance(v, float) else v for k, v in plan.items()}))
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    on_gpu = a.device == "cuda"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(dev)
    else:
        assert a.path == "nccl" or world == 1, "--device cpu runs the plan executor (--path nccl)"
        assert a.seq_algo in ("cp", "halo") and not a.breakdown, "--device cpu: context-parallel or halo path, no breakdown"
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        if on_gpu:
            dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
        else:
            dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=300))
        group = dist.group.WORLD
    cfg = LlamaConfig(n_layers=a.layers, hidden=a.hidden, n_heads=a.heads, head_dim=a.head_dim, ffn=a.ffn,
                      vocab=a.vocab, n_kv_heads=a.kv_heads, sliding_window=a.sliding_window, sink_tokens=a.sink_tokens)
    assert a.sliding_window is None or world == 1 or a.seq_algo == "halo", \
        "--sliding-window runs on one rank or with --seq-algo halo"
    pattern = P.global_local(a.blocks, 1, 2)
    runtime = None
    if world > 1 and a.seq_algo in ("ulysses", "halo"):
        s_loc = a.seq // world
        pos = torch.arange(rank * s_loc, (rank + 1) * s_loc)
    elif world > 1:
        runtime = ContextParallelAttention(pattern, a.seq, a.heads, a.head_dim, group=group, device=dev, path=a.path)
        cmap = runtime.cmap
        par_d = runtime.table.shape[0]
        blk = a.seq // par_d
        mine = [b for b in range(par_d) if cmap[b] == rank]
        pos = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in mine])
    else:
        pos = torch.arange(a.seq)
    model = LlamaModel(cfg, device=dev, pattern=pattern, runtime=runtime, group=group, seed=0,
                       offload_checkpoints=a.offload_checkpoints, seq_algo=a.seq_algo, seq_len=a.seq)
    g = torch.Generator().manual_seed(3)
    ids_all = torch.randint(0, a.vocab, (a.seq + 1,), generator=g)
    ids = ids_all[pos].to(dev)
    targets = ids_all[pos + 1].to(dev)
    pos_dev = pos.to(dev)

    def step():
        return model.train_step(ids, targets, pos_dev, n_total_tokens=a.seq)

    loss = None
    losses = []
    for _ in range(a.warmup):
        loss = step()
        losses.append(loss)
    if world > 1:
        dist.barrier()
    if on_gpu:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    else:
        import time
        t_start = time.perf_counter()
    for _ in range(a.steps):
        loss = step()
        losses.append(loss)
    if on_gpu:
        e1.record()
    if world > 1:
        dist.barrier()
    if on_gpu:
        torch.cuda.synchronize()
        A.check_status(dev)
        ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    else:
        ms = torch.tensor([(time.perf_counter() - t_start) * 1e3 / a.steps])
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    split = None
    if a.breakdown:
        split = _breakdown(model, step, dev)
        if world > 1:
            t = torch.tensor([split[k] for k in sorted(split)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            split = dict(zip(sorted(split), [round(x, 2) for x in t.tolist()]))
    if rank == 0:
        n_params = model.flat.numel()
        print(json.dumps({"metric": "e2e_tokens_per_s", "value": a.seq / (ms.item() / 1e3), "ms_per_step": ms.item(),
                          "n_gpus": world, "seq_len": a.seq, "layers": a.layers, "params": n_params, "loss": loss,
                          "losses": losses,
                          "path": "local" if world == 1 else
                                  {"cp": a.path, "ulysses": "ulysses-fused", "halo": "halo"}[a.seq_algo],
                          "dtype": "bf16" if on_gpu else "fp32", "device": a.device,
                          "max_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30 if on_gpu else None,
                          **({"split_ms_max_over_ranks": split} if split else {})}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
