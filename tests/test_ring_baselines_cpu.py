"""Ring / zigzag / stripe / Ulysses baselines on CPU ranks over gloo against dense attention."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, kind, causal, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ultraattn_b200 import parallel as PL, patterns as P
        S, H, D = 256, 4, 16
        g = torch.Generator().manual_seed(0)
        q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
        sh = lambda t: PL.shard_sequence(t, rank, world, kind)
        ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
        fn = {"ring": PL.ring_flash_attn_func, "zigzag": PL.zigzag_ring_flash_attn_func,
              "stripe": PL.stripe_flash_attn_func, "ulysses": PL.deepspeed_ulysses_attn_func}[kind]
        o = fn(ql, kl, vl, causal=causal)
        o.backward(sh(d_o))
        pat = P.causal(1) if causal else P.full(1)
        o_ref, _, dq, dk, dv = P.dense_attention_with_grads(q, k, v, d_o, pat)
        ret[rank] = max((o - sh(o_ref)).abs().max().item(), (ql.grad - sh(dq)).abs().max().item(),
                        (kl.grad - sh(dk)).abs().max().item(), (vl.grad - sh(dv)).abs().max().item())
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind,causal", [("ring", True), ("ring", False), ("zigzag", True),
                                         ("stripe", True), ("ulysses", True)])
def test_baselines_world4(kind, causal):
    port = 29900 + (os.getpid() + hash(kind)) % 90
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(4, port, kind, causal, ret), nprocs=4, join=True)
    for r in range(4):
        assert isinstance(ret[r], float), ret[r]
        assert ret[r] < 2e-4, (r, ret[r])
