"""The Llama-style model on CPU against a plain PyTorch restatement: loss, gradients, and that the
fused Adam step moves the weights the same way."""
import math

import torch
import torch.nn.functional as F

from ultraattn_b200 import patterns as P
from ultraattn_b200.models.llama import LlamaConfig, LlamaModel


def _ref_loss(model: LlamaModel, params: dict, ids, targets, pattern, mask=None):
    c = model.cfg
    T = ids.shape[0]
    x = F.embedding(ids, params["embed"])
    half = c.head_dim // 2
    inv = 1.0 / (c.rope_base ** (torch.arange(0, c.head_dim, 2, dtype=torch.float32) / c.head_dim))
    ang = torch.arange(T, dtype=torch.float32)[:, None] * inv[None]
    cos, sin = torch.cos(ang)[:, None], torch.sin(ang)[:, None]

    def rms(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + c.eps) * w

    def rope(t):
        lo, hi = t[..., :half], t[..., half:]
        return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], -1)

    mask = pattern.token_mask(T, T) if mask is None else mask
    nkv = c.kv_heads * c.head_dim
    g = c.n_heads // c.kv_heads
    for i in range(c.n_layers):
        h = rms(x, params[f"l{i}.norm1"])
        qkv = h @ params[f"l{i}.wqkv"].t()
        nq = c.n_heads * c.head_dim
        q = rope(qkv[:, :nq].view(T, c.n_heads, c.head_dim))
        k = rope(qkv[:, nq:nq + nkv].view(T, c.kv_heads, c.head_dim)).repeat_interleave(g, 1)
        v = qkv[:, nq + nkv:].view(T, c.kv_heads, c.head_dim).repeat_interleave(g, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(c.head_dim)
        s = s.masked_fill(~mask[None], float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, nq)
        x = x + o @ params[f"l{i}.wo"].t()
        h = rms(x, params[f"l{i}.norm2"])
        gu = h @ params[f"l{i}.wgu"].t()
        x = x + (F.silu(gu[:, :c.ffn]) * gu[:, c.ffn:]) @ params[f"l{i}.wdown"].t()
    x = rms(x, params["norm_f"])
    return F.cross_entropy(x @ params["lm_head"].t(), targets)


def test_llama_matches_plain_pytorch():
    torch.manual_seed(0)
    cfg = LlamaConfig(n_layers=2, hidden=64, n_heads=2, head_dim=32, ffn=96, vocab=50)
    pat = P.global_local(4, 1, 2, global_rows_see_all=False)
    model = LlamaModel(cfg, pattern=pat, lr=1e-2)
    T = 64
    ids = torch.randint(0, cfg.vocab, (T,))
    tg = torch.randint(0, cfg.vocab, (T,))
    ref_params = {k: v.detach().clone().requires_grad_() for k, v in model.p.items()}
    ref = _ref_loss(model, ref_params, ids, tg, pat)
    ref.backward()
    loss = model.loss(ids, tg, chunk=16)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 1e-4
    for name, p in model.p.items():
        err = (p.grad - ref_params[name].grad).abs().max().item()
        assert err < 2e-4, (name, err)
    before = model.flat.detach().clone()
    opt = torch.optim.AdamW([ref_params[k] for k in model.p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    opt.step()
    model.optimizer_step()
    assert (model.flat - before).abs().max().item() > 0
    for name, p in model.p.items():
        assert (p.detach() - ref_params[name].detach()).abs().max().item() < 1e-4, name
    assert model.flat_grad.abs().max().item() == 0


def test_memory_plan_of_the_headline_training_config():
    """Llama-2-7B, S = 512k, CP = 8: parameter count, and the per-GPU plan fits a 180 GB GPU with
    the checkpoints on the device; offloading moves exactly the checkpoints to the host."""
    from ultraattn_b200.models.llama import LlamaConfig, estimate_memory
    cfg = LlamaConfig.llama2_7b()
    m = estimate_memory(cfg, 524288, 8)
    assert m["n_params"] == 6738415616
    assert abs(m["parameters"] - 12.55) < 0.01 and abs(m["optimizer_shard"] - 3 * 4 * m["n_params"] / 8 / 2**30) < 1e-9
    assert 80 < m["device_total"] < 140
    off = estimate_memory(cfg, 524288, 8, offload_checkpoints=True)
    assert off["checkpoints_device"] == 0 and abs(off["checkpoints_host"] - m["checkpoints_device"]) < 1e-9
    assert abs((m["device_total"] - off["device_total"]) - m["checkpoints_device"]) < 1e-9
    small = estimate_memory(LlamaConfig(n_layers=4), 65536, 2)
    assert 15 < small["device_total"] < 30                     # a run of this size peaked at 18.4 GiB per GPU


def test_token_cross_entropy_wrappers_match_pytorch():
    """The loss head's two fused passes (CPU restatement of the CUDA kernels): loss and in-place
    gradient against torch.nn.functional.cross_entropy, with an ignored target."""
    import torch
    import torch.nn.functional as F
    from ultraattn_b200.ops import elementwise as E
    torch.manual_seed(0)
    T, V = 16, 40
    logits = torch.randn(T, V)
    tg = torch.randint(0, V, (T,))
    tg[2] = -1
    keep = tg >= 0
    lse, loss = E.xent_fwd(logits, tg)
    ref = F.cross_entropy(logits, tg.clamp(min=0), reduction="none") * keep
    assert torch.allclose(loss, ref, atol=1e-5) and torch.allclose(lse, torch.logsumexp(logits, -1), atol=1e-6)
    x = logits.clone().requires_grad_()
    ((F.cross_entropy(x, tg.clamp(min=0), reduction="none") * keep).sum() * 0.5).backward()
    work = logits.clone()
    got = E.xent_bwd_(work, tg, lse, torch.tensor(0.5))
    assert got is work and torch.allclose(got, x.grad, atol=1e-6) and got[2].abs().max() == 0


def test_trainer_on_two_cpu_ranks_follows_the_single_rank_losses():
    """The end-to-end trainer as fp32 CPU ranks: two context-parallel ranks (tokens sharded by the
    plan's block ownership, attention through the plan executor over gloo, Adam sharded over the
    ranks) must walk the same loss curve as one rank holding the whole sequence."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = ["--device", "cpu", "--path", "nccl", "--seq", "1024", "--layers", "2", "--hidden", "128", "--heads", "4",
            "--head-dim", "32", "--ffn", "256", "--vocab", "512", "--blocks", "8", "--steps", "2", "--warmup", "1"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True, cwd=root, env=env, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        return json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])

    one = run([sys.executable, "-m", "ultraattn_b200.drivers.train_llama"] + args)
    two = run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", str(29930 + os.getpid() % 40), "-m",
               "ultraattn_b200.drivers.train_llama"] + args)
    assert one["n_gpus"] == 1 and two["n_gpus"] == 2 and two["path"] == "nccl" and one["device"] == "cpu"
    assert len(one["losses"]) == 3 and one["losses"][0] > one["losses"][-1], one["losses"]   # it learns
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 2e-5 * abs(a), (one["losses"], two["losses"])


def test_mistral_style_model_with_sliding_window_and_grouped_query_heads():
    """``LlamaConfig(sliding_window=..., n_kv_heads=...)`` (``LlamaConfig.mistral_7b()`` is that at
    full size): loss and every weight gradient against plain PyTorch with the band mask; with
    sink tokens the mask keeps the first tokens visible."""
    for sinks in (0, 3):
        torch.manual_seed(1)
        cfg = LlamaConfig(n_layers=2, hidden=64, n_heads=4, head_dim=16, ffn=96, vocab=50, n_kv_heads=2,
                          sliding_window=24, sink_tokens=sinks)
        model = LlamaModel(cfg, lr=1e-2)
        T = 96
        ids = torch.randint(0, cfg.vocab, (T,))
        tg = torch.randint(0, cfg.vocab, (T,))
        r, c = torch.arange(T)[:, None], torch.arange(T)[None, :]
        mask = ((c <= r) & (c >= r - 23)) | ((c < sinks) & (c <= r))
        ref_params = {k: v.detach().clone().requires_grad_() for k, v in model.p.items()}
        ref = _ref_loss(model, ref_params, ids, tg, None, mask)
        ref.backward()
        loss = model.loss(ids, tg, chunk=32)
        loss.backward()
        assert abs(loss.item() - ref.item()) < 1e-4
        for name, p in model.p.items():
            err = (p.grad - ref_params[name].grad).abs().max().item()
            assert err < 2e-4, (sinks, name, err)
    big = LlamaConfig.mistral_7b()
    assert (big.kv_heads, big.ffn, big.sliding_window, big.n_layers) == (8, 14336, 4096, 32)
    import pytest
    with pytest.raises(NotImplementedError, match="sliding window"):
        LlamaModel(cfg, runtime=object())


def test_mistral_style_trainer_with_halo_exchange_follows_the_single_rank_losses():
    """Sliding-window model (grouped-query heads, window of 300 tokens): four ranks with contiguous
    shards of 256 tokens fetch the window's keys from up to two preceding ranks and walk the same
    loss curve as one rank with the whole sequence."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = ["--device", "cpu", "--path", "nccl", "--seq", "1024", "--layers", "2", "--hidden", "128", "--heads", "4",
            "--kv-heads", "2", "--head-dim", "32", "--ffn", "256", "--vocab", "512", "--steps", "2", "--warmup", "1",
            "--sliding-window", "300"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True, cwd=root, env=env, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        return json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])

    one = run([sys.executable, "-m", "ultraattn_b200.drivers.train_llama"] + args)
    four = run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
                "127.0.0.1", "--master-port", str(29960 + os.getpid() % 30), "-m",
                "ultraattn_b200.drivers.train_llama"] + args + ["--seq-algo", "halo"])
    assert four["n_gpus"] == 4 and four["path"] == "halo" and one["losses"][0] > one["losses"][-1]
    for a, b in zip(one["losses"], four["losses"]):
        assert abs(a - b) < 2e-5 * abs(a), (one["losses"], four["losses"])
