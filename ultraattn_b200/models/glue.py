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
         "dist_flash_attn": "lightseq", "lightseq": "lightseq", "halo_attn": "halo", "halo": "halo", "data_parallel": None, "ultra_attn": "ring", "ultraattn": "ring"}


def shard_by_ownership(x: torch.Tensor, cmap, rank: int, dim: int = 1) -> torch.Tensor:
    """The blocks of ``x`` (along ``dim``) that ``cmap`` (block -> rank) gives to ``rank``, in
    increasing block order: the shard a context-parallel runtime expects under a remapped
    ownership (``ContextParallelAttention(cmap=...)``, ``plan_allocation(cmap="search")``)."""
    n = len(cmap)
    blk = x.shape[dim] // n
    assert blk * n == x.shape[dim], "the token count is not a multiple of the number of blocks"
    idx = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in range(n) if int(cmap[b]) == rank])
    return x.index_select(dim, idx.to(x.device)).contiguous()


def prepare_seq_parallel_inputs(seq_algo: str, input_ids, position_ids, target_ids, rank: int, world_size: int,
                                device=None, cmap=None) -> dict:
    """Shard token / position / target ids the way ``seq_algo`` expects. ``cmap`` (block -> rank,
    e.g. a runtime's ``.cmap``) overrides the layout for the planner-driven runtime."""
    kind = _KIND.get(seq_algo, seq_algo)
    if cmap is not None:
        sh = lambda t: None if t is None else shard_by_ownership(t, cmap, rank, dim=1)
    elif kind is None:
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


_mask_warned = [False]


def _warn_if_not_causal(mask) -> None:
    """The strategies apply a causal mask over the global positions themselves and do not read
    ``attention_mask``. A mask that says more than "causal" (padding, packed documents) would be
    dropped silently, so it is reported once; masks too large to compare cheaply are not checked."""
    if mask is None or _mask_warned[0] or mask.dim() < 2 or mask.numel() > (1 << 24):
        return
    allowed = mask if mask.dtype == torch.bool else mask == 0
    tq, tk = allowed.shape[-2], allowed.shape[-1]
    causal = torch.ones(tq, tk, dtype=torch.bool, device=mask.device).tril(tk - tq)
    if not torch.equal(allowed.reshape(-1, tq, tk), causal.expand(allowed.numel() // (tq * tk), tq, tk)):
        import warnings
        _mask_warned[0] = True
        warnings.warn("the context-parallel attention function ignores attention_mask, and this mask is not a plain "
                      "causal one (padding or packed sequences?): use the varlen strategies for packed batches",
                      RuntimeWarning, stacklevel=3)


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

    def halo_fn(q, k, v, softmax_scale=None, causal=True, group=None, window_size=None):
        """Contiguous shards, the window's keys fetched from the preceding ranks (parallel/halo.py)."""
        from ..parallel.halo import halo_window_attn_func
        if window_size is None:
            raise NotImplementedError("seq_algo='halo' is the strategy for layers with a sliding window; this layer has none")
        return halo_window_attn_func(q, k, v, window_size, softmax_scale, causal, group)

    fn = {"ring": R.ring_flash_attn_func, "zigzag": R.zigzag_ring_flash_attn_func,
          "stripe": R.stripe_flash_attn_func, "ulysses": R.deepspeed_ulysses_attn_func,
          "lightseq": lightseq_fn, "halo": halo_fn}[kind]

    def attention_forward(module, query, key, value, attention_mask=None, dropout: float = 0.0,
                          scaling: Optional[float] = None, **kwargs):
        q = query.transpose(1, 2).contiguous()
        k = key.transpose(1, 2).contiguous()
        v = value.transpose(1, 2).contiguous()
        if dropout:
            raise NotImplementedError("attention dropout is not implemented by these kernels (set attention_dropout=0)")
        _warn_if_not_causal(attention_mask)
        window = kwargs.get("sliding_window")
        if window is not None:
            # transformers hands a layer's sliding window (Mistral and others) to the attention
            # function. The head-parallel strategy holds whole sequences and the halo strategy
            # fetches the window's keys, so both apply a token-exact band. Anything else must
            # refuse rather than attend too far back.
            if runtime is not None or kind not in ("ulysses", "halo"):
                raise NotImplementedError(
                    f"sliding_window={window} needs seq_algo='halo' or 'ulysses' (token-exact windows are not part of "
                    f"the {seq_algo!r} strategy; a block-level window is a pattern of the context-parallel runtime)")
            out = fn(q, k, v, softmax_scale=scaling, causal=True, group=group, window_size=(int(window) - 1, 0))
            return out, None
        if runtime is not None:
            out = runtime(q, k, v, scaling)
        else:
            out = fn(q, k, v, softmax_scale=scaling, causal=True, group=group)
        return out, None
    return attention_forward


def apply_seq_parallel_monkey_patch(seq_algo: str, model, group=None, runtime=None):
    """Make ``model`` use context-parallel attention. ``model`` is a HuggingFace causal LM (or
    its config), which is switched to the new attention function, or, as in the reference, the
    family name ``"llama"`` / ``"mistral"``: the function is then only registered and models are
    built with ``attn_implementation=<returned name>``. Returns the registered name."""
    if _KIND.get(seq_algo, seq_algo) is None:
        return None
    from transformers import AttentionInterface
    name = f"ultraattn_{seq_algo}"
    AttentionInterface.register(name, make_attention_interface(seq_algo, group, runtime))
    if isinstance(model, str):
        assert model in ("llama", "mistral"), f"Invalid model: {model}"
        return name
    cfg = model if not hasattr(model, "config") else model.config
    cfg._attn_implementation = name
    return name


# -------------------------------------------------------------------------------------------------
# the reference's per-strategy names (easy_context/__init__.py:1-6)
# -------------------------------------------------------------------------------------------------
def prepare_zigzag_ring_attn_inputs(input_ids, position_ids, target_ids, rank, world_size, device=None):
    """Reference: easy_context/zigzag_ring_attn/prepare_inputs.py:4-40 (rank r holds chunks r and
    2W-1-r of the 2W chunks of the sequence)."""
    return prepare_seq_parallel_inputs("zigzag_ring_attn", input_ids, position_ids, target_ids, rank,
                                       world_size, device)


def prepare_dist_flash_attn_inputs(input_ids, position_ids, target_ids, rank, world_size, device=None):
    """Reference: easy_context/dist_flash_attn/prepare_input.py (contiguous chunks)."""
    return prepare_seq_parallel_inputs("dist_flash_attn", input_ids, position_ids, target_ids, rank,
                                       world_size, device)


def prepare_dataloader(seq_algo: str, dataloader, accelerator=None):
    """Reference: easy_context/__init__.py:44-48. Under data parallelism every rank reads its own
    samples (``accelerator.prepare`` shards the loader); under sequence parallelism all ranks of
    the group read the same sample and shard it with :func:`prepare_seq_parallel_inputs`."""
    if _KIND.get(seq_algo, seq_algo) is None and accelerator is not None:
        return accelerator.prepare(dataloader)
    return dataloader


def apply_zigzag_ring_attn_monkey_patch_llama(group=None):
    return apply_seq_parallel_monkey_patch("zigzag_ring_attn", "llama", group)


def apply_zigzag_ring_attn_monkey_patch_mistral(group=None):
    return apply_seq_parallel_monkey_patch("zigzag_ring_attn", "mistral", group)


def apply_dist_flash_attn_monkey_patch_llama(group=None):
    return apply_seq_parallel_monkey_patch("dist_flash_attn", "llama", group)


class OffloadedCheckpoint(torch.autograd.Function):
    """Activation checkpoint whose saved input lives in pinned host memory (reference:
    easy_context/unsloth_offloaded_gradient_checkpoint/monkey_patch.py:20-60). The copy out runs
    on a side stream so the layer's forward does not wait for it; the backward brings the
    input back, re-runs the layer with gradients enabled and back-propagates through it."""

    @staticmethod
    def forward(ctx, forward_function, hidden_states, *args):
        if hidden_states.is_cuda:
            host = torch.empty(hidden_states.shape, dtype=hidden_states.dtype, device="cpu", pin_memory=True)
            side = _offload_stream(hidden_states.device)
            side.wait_stream(torch.cuda.current_stream(hidden_states.device))
            with torch.cuda.stream(side):
                host.copy_(hidden_states, non_blocking=True)
            hidden_states.record_stream(side)
            ctx.copied = torch.cuda.Event()
            ctx.copied.record(side)
        else:
            host, ctx.copied = hidden_states.detach().clone(), None
        with torch.no_grad():
            output = forward_function(hidden_states, *args)
        ctx.host, ctx.device = host, hidden_states.device
        ctx.forward_function, ctx.args = forward_function, args
        return output

    @staticmethod
    def backward(ctx, *d_out):
        if ctx.copied is not None:
            ctx.copied.synchronize()
        x = ctx.host.to(ctx.device, non_blocking=True).detach().requires_grad_(True)
        with torch.enable_grad():
            out = ctx.forward_function(x, *ctx.args)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, d_out) if isinstance(o, torch.Tensor) and o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, x.grad) + (None,) * len(ctx.args)


_offload_streams: dict = {}


def _offload_stream(device):
    if device not in _offload_streams:
        _offload_streams[device] = torch.cuda.Stream(device)
    return _offload_streams[device]


def apply_unsloth_offloaded_gradient_checkpoint_monkey_patch(model=None):
    """Make gradient checkpointing of HuggingFace models keep the checkpoints in host memory
    (reference: easy_context/unsloth_offloaded_gradient_checkpoint/monkey_patch.py:63-94). With a
    model, only that model is switched; without, every ``PreTrainedModel`` that enables gradient
    checkpointing afterwards."""
    def checkpoint(function, *args, **kwargs):
        hidden, rest = args[0], args[1:]
        fn = (lambda h, *a: function(h, *a, **kwargs)) if kwargs else function
        return OffloadedCheckpoint.apply(fn, hidden, *rest)

    if model is not None:
        model.gradient_checkpointing_enable()
        for m in model.modules():
            if hasattr(m, "_gradient_checkpointing_func"):
                m._gradient_checkpointing_func = checkpoint
        return checkpoint
    import transformers

    def enable(self, gradient_checkpointing_kwargs=None):
        if not self.supports_gradient_checkpointing:
            raise ValueError(f"{type(self).__name__} does not support gradient checkpointing")
        self._set_gradient_checkpointing(enable=True, gradient_checkpointing_func=checkpoint)
        if getattr(self, "_hf_peft_config_loaded", False):
            self.enable_input_require_grads()
    transformers.modeling_utils.PreTrainedModel.gradient_checkpointing_enable = enable
    return checkpoint
