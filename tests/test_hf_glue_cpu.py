"""A HuggingFace Llama routed through this framework's context-parallel attention on gloo ranks:
sharded inputs, registered attention function, logits and weight gradients against the unsharded
model."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, seq_algo, ret, family="llama"):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import easy_context
        if family == "mistral":             # every layer attends a sliding window of 24 tokens
            from transformers import MistralConfig, MistralForCausalLM
            cfg = MistralConfig(vocab_size=97, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                sliding_window=24, attn_implementation="eager")
            torch.manual_seed(0)
            model = MistralForCausalLM(cfg).train()
        else:
            from transformers import LlamaConfig, LlamaForCausalLM
            cfg = LlamaConfig(vocab_size=97, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                              num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                              attn_implementation="eager")
            torch.manual_seed(0)
            model = LlamaForCausalLM(cfg).train()
        T = 64
        g = torch.Generator().manual_seed(1)
        ids = torch.randint(0, 97, (1, T), generator=g)
        pos = torch.arange(T)[None]
        # the unsharded model: logits, and gradients of the summed token losses
        logits = model(input_ids=ids, position_ids=pos).logits
        loss = torch.nn.functional.cross_entropy(logits[0, :-1], ids[0, 1:], reduction="sum")
        loss.backward()
        ref_grad = {n: p.grad.clone() for n, p in model.named_parameters()}
        model.zero_grad()
        # context-parallel: shard ids / positions / targets, route attention through the ring
        name = easy_context.apply_seq_parallel_monkey_patch(seq_algo, model)
        assert model.config._attn_implementation == name
        targets = torch.cat([ids[:, 1:], torch.full((1, 1), -100)], dim=1)
        sh = easy_context.prepare_seq_parallel_inputs(seq_algo, ids, pos, targets, rank, world, "cpu")
        out = model(input_ids=sh["local_input_ids"], position_ids=sh["local_position_ids"]).logits
        want = easy_context.prepare_seq_parallel_inputs(seq_algo, logits.detach(), None, None, rank, world)["local_input_ids"]
        err = (out - want).abs().max().item()
        local = torch.nn.functional.cross_entropy(out[0], sh["local_target_ids"][0], reduction="sum", ignore_index=-100)
        local.backward()
        gerr = 0.0
        for n, p in model.named_parameters():
            gr = p.grad.clone()
            dist.all_reduce(gr)                      # weights are replicated: gradients add over ranks
            gerr = max(gerr, (gr - ref_grad[n]).abs().max().item() / (ref_grad[n].abs().max().item() + 1e-6))
        ret[rank] = (err, gerr)
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq_algo", ["zigzag_ring_attn", "dist_flash_attn"])
def test_hf_llama_context_parallel_world2(seq_algo):
    port = 29000 + (os.getpid() + len(seq_algo)) % 90
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, seq_algo, ret), nprocs=2, join=True)
    for r in range(2):
        assert isinstance(ret[r], tuple), ret[r]
        assert ret[r][0] < 1e-4 and ret[r][1] < 1e-4, (r, ret[r])


def test_hf_mistral_sliding_window_world2():
    """A Mistral whose layers use a sliding window: the registered head-parallel and halo-exchange
    attention functions apply the token-exact window (logits and weight gradients match the
    unsharded eager model), and a strategy that cannot apply it refuses instead of attending too
    far back."""
    for i, seq_algo in enumerate(("ulysses_attn", "halo_attn")):
        ret = mp.Manager().dict()
        mp.spawn(_worker, args=(2, 29100 + (os.getpid() + 7 * i) % 90, seq_algo, ret, "mistral"), nprocs=2, join=True)
        for r in range(2):
            assert isinstance(ret[r], tuple), (seq_algo, ret[r])
            assert ret[r][0] < 1e-4 and ret[r][1] < 1e-4, (seq_algo, r, ret[r])
    sys.path.insert(0, ROOT)
    from ultraattn_b200.models.glue import make_attention_interface
    fn = make_attention_interface("zigzag_ring_attn")
    q = torch.randn(1, 2, 8, 4)
    with pytest.raises(NotImplementedError, match="sliding_window"):
        fn(None, q, q, q, None, 0.0, None, sliding_window=4)
    with pytest.raises(NotImplementedError, match="dropout"):
        fn(None, q, q, q, None, 0.1, None)
    # a mask that is more than causal is reported (once), a causal one is not
    import warnings
    from ultraattn_b200.models import glue
    glue._mask_warned[0] = False
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        glue._warn_if_not_causal(torch.ones(8, 8, dtype=torch.bool).tril()[None, None])
        glue._warn_if_not_causal(torch.zeros(8, 8).masked_fill(~torch.ones(8, 8, dtype=torch.bool).tril(), float("-inf"))[None, None])
    padded = torch.ones(8, 8, dtype=torch.bool).tril()
    padded[:, :2] = False
    with pytest.warns(RuntimeWarning, match="ignores attention_mask"):
        glue._warn_if_not_causal(padded[None, None])
