"""Block-sparse attention on one device with autograd, and the plan a cluster would run.

    python examples/single_gpu.py            # CUDA (sm_100a kernels, bf16) if present, else the CPU restatement

Shows the three things a user touches: a named pattern, the differentiable operator, and the
planner (allocation of tiles to ranks + launch schedule) for the same pattern on eight ranks.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ultraattn_b200 as ua  # noqa: E402
from ultraattn_b200 import patterns as P  # noqa: E402
from ultraattn_b200.planner import make_plan  # noqa: E402


def main() -> None:
    cuda = torch.cuda.is_available()
    dev, dtype, head_dim = (("cuda", torch.bfloat16, 128) if cuda else ("cpu", torch.float32, 32))
    pattern = P.strided(n_blocks=8, stride=4, window=2)
    print("pattern:", pattern)
    S, H = 2048, 4
    q, k, v = (torch.randn(1, S, H, head_dim, device=dev, dtype=dtype, requires_grad=True) for _ in range(3))
    out = ua.attention(q, k, v, pattern)
    out.backward(torch.randn_like(out))
    o_ref, *_ = P.dense_attention(q.detach().float().cpu(), k.detach().float().cpu(), v.detach().float().cpu(),
                                  pattern.token_mask(S, S))
    print(f"output {tuple(out.shape)} on {dev}; max error against dense attention "
          f"{(out.detach().float().cpu() - o_ref).abs().max().item():.2e}; dQ norm {q.grad.float().norm().item():.3f}")
    plan = make_plan(pattern=pattern, cp=8, seq_len=524288, n_heads=32, head_dim=128, fob=0, time_limit=5.0)
    comp = sum(kk.type == "comp" for kk in plan.valid_kernels)
    print(f"plan for 8 ranks, S = 512k: {comp} compute kernels, {len(plan.valid_kernels) - comp} messages, "
          f"predicted forward {plan.end_time * 1e3:.1f} ms, checks: {plan.verify() or 'ok'}")
    print("tile -> rank:\n", plan.allocation.table)


if __name__ == "__main__":
    main()
