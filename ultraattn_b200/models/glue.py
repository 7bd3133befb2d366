"""Model integration helpers (reference: easy_context/__init__.py:8-42,
easy_context/zigzag_ring_attn/prepare_inputs.py:4-40, easy_context/*/monkey_patch.py).

``prepare_seq_parallel_inputs`` shards token / position / target ids the way each strategy expects.
``apply_seq_parallel_monkey_patch`` routes a HuggingFace model's attention through one of this
framework's context-parallel functions; it uses the attention-function registry of current
``transformers`` instead of overwriting private methods of ``LlamaFlashAttention2``.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel import ring as R

_KIND = {"zigzag_ring_attn": "zigzag", "zigzag": "zigzag", "ring_attn": "ring", "ring": "ring",
         "stripe_attn": "stripe", "stripe": "stripe", "ulysses_attn": "ulysses", "ulysses": "ulysses",
         "dist_flash_attn": "lightseq", "lightseq": "lightseq", "data_parallel": None, "ultra_attn": "ring", "ultraattn": "ring"}


def prepare_seq_parallel_inputs(seq_algo: str, input_ids, position_ids, target_ids, rank: int, world_size: int,
                                device=None) -> dict:
    kind = _KIND.get(seq_algo, seq_algo)
    if kind is None:
        sh = lambda t: t
    elif kind == "lightseq":        # contiguous chunks, like the plain ring
        sh = lambda t: None if t is None else R.shard_sequence(t, rank, world_size, "ring", dim=1)
    else:
        sh = lambda t: None if t is None else R.shard_sequence(t, rank, world_size, kind, dim=1)
    out = {"local_input_ids": sh(input_ids), "local_position_ids": sh(position_ids),
           "local_target_ids": sh(target_ids)}
    if device is not None:
        out = {k: (v.to(device) if v is not None else None) for k, v in out.items()}
    return out


def make_attention_interface(seq_algo: str, group=None, runtime=None):
    """An attention function with the calling convention of transformers' attention registry:
    ``(module, query[B,H,T,D], key, value, attention_mask, dropout, scaling, **kw) -> (out[B,T,H,D], None)``."""
    kind = _KIND.get(seq_algo, seq_algo)
    lightseq_runtimes = {}

    def lightseq_fn(q, k, v, softmax_scale=None, causal=True, group=None):
        """LightSeq's balanced causal schedule (worker / helper ranks) run by the context-parallel
        runtime; one runtime per shape, built on first use."""
        import torch.distributed as dist
        from .. import patterns as P
        from ..runtime import ContextParallelAttention
        assert causal, "the LightSeq schedule is causal"
        world = dist.get_world_size(group)
        key = (q.shape[1], q.shape[2], q.shape[3], k.shape[2])
        if key not in lightseq_runtimes:
            lightseq_runtimes[key] = ContextParallelAttention(
                P.causal(1), q.shape[1] * world, q.shape[2], q.shape[3], group=group, device=q.device,
                n_kv_heads=k.shape[2], batch=q.shape[0], allocation="lightseq",
                path="fused" if q.is_cuda else "nccl", dtype=q.dtype)
        return lightseq_runtimes[key](q, k, v, softmax_scale)

    fn = {"ring": R.ring_flash_attn_func, "zigzag": R.zigzag_ring_flash_attn_func,
          "stripe": R.stripe_flash_attn_func, "ulysses": R.deepspeed_ulysses_attn_func,
          "lightseq": lightseq_fn}[kind]

    def attention_forward(module, query, key, value, attention_mask=None, dropout: float = 0.0,
                          scaling: Optional[float] = None, **kwargs):
        q = query.transpose(1, 2).contiguous()
        k = key.transpose(1, 2).contiguous()
        v = value.transpose(1, 2).contiguous()
        if runtime is not None:
            out = runtime(q, k, v, scaling)
        else:
            out = fn(q, k, v, softmax_scale=scaling, causal=True, group=group)
        return out, None
    return attention_forward


def apply_seq_parallel_monkey_patch(seq_algo: str, model, group=None, runtime=None):
    """Make ``model`` (a HuggingFace causal LM) use context-parallel attention. Returns the name
    under which the attention function was registered."""
    if _KIND.get(seq_algo, seq_algo) is None:
        return None
    from transformers import AttentionInterface
    name = f"ultraattn_{seq_algo}"
    AttentionInterface.register(name, make_attention_interface(seq_algo, group, runtime))
    cfg = model if not hasattr(model, "config") else model.config
    cfg._attn_implementation = name
    return name
