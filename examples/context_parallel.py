"""Context-parallel block-sparse attention in a dozen lines.

    # two CPU ranks (gloo, fp32 reference executor): runs anywhere
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/context_parallel.py
    # eight B200s (fused peer-memory kernels, bf16)
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/context_parallel.py --seq 524288

Every rank holds a contiguous shard of the sequence; the call returns the matching shard of the
output and autograd gives the shards of dQ, dK, dV. The result is checked against dense attention
on rank 0 when the sequence is short enough to do that.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ultraattn_b200 import patterns as P  # noqa: E402
from ultraattn_b200.runtime import ContextParallelAttention  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--pattern", default="strided", choices=["strided", "global_local", "star", "streaming", "causal", "full"])
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    pattern = {"strided": lambda: P.strided(8, 4, 2), "global_local": lambda: P.global_local(8, 1, 2),
               "star": lambda: P.star(8, 1), "streaming": lambda: P.streaming(8, 1, 2),
               "causal": lambda: P.causal(1), "full": lambda: P.full(1)}[a.pattern]()
    dtype, head_dim = (torch.bfloat16, 128) if cuda else (torch.float32, 32)
    attn = ContextParallelAttention(pattern, a.seq, a.heads, head_dim, device=dev, dtype=dtype,
                                    path="fused" if cuda else "nccl", plan_time_limit=5.0)
    g = torch.Generator().manual_seed(0)                      # the same full tensors on every rank
    q, k, v, d_o = (torch.randn(1, a.seq, a.heads, head_dim, generator=g) for _ in range(4))
    blk = a.seq // attn.table.shape[0]                        # this rank's blocks under the plan's ownership map
    idx = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in range(attn.table.shape[0]) if attn.cmap[b] == rank])
    ql, kl, vl = (t[:, idx].to(dtype).to(dev).requires_grad_() for t in (q, k, v))
    out = attn(ql, kl, vl)
    out.backward(d_o[:, idx].to(dtype).to(dev))
    if a.seq <= 8192:
        o_ref, _, dq_ref, _, _ = P.dense_attention_with_grads(q, k, v, d_o, pattern)
        err = max((out.float().cpu() - o_ref[:, idx]).abs().max().item(),
                  (ql.grad.float().cpu() - dq_ref[:, idx]).abs().max().item())
        print(f"rank {rank}/{world}: output shard {tuple(out.shape)}, max error against dense attention {err:.2e}")
    else:
        print(f"rank {rank}/{world}: output shard {tuple(out.shape)}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
