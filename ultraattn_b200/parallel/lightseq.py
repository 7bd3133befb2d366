"""LightSeq's DistAttn surface: sequence-parallel group helpers, the worker / helper time-step
schedule, and ``attention(q, k, v, causal, sm_scale)`` on ``[batch, heads, tokens, head_dim]``.

Reference: easy_context/dist_flash_attn/async_communication.py:42-257 (group set-up and the
schedule predicates), lightseq_async_attn.py:244-464 (forward / backward driver and the autograd
function), prepare_input.py. The reference drives Triton kernels with hand-rolled double-buffered
sends; here the balanced causal schedule is an allocation table
(``planner.dense.get_lightseq_schedule_table``) executed by the context-parallel runtime, so the
same schedule runs on the fused path, the NCCL executor and the gloo CPU executor. The predicates
below restate the time-step view of that table and are checked against it in the tests.

Schedule, for W ranks and causal attention over contiguous shards: there are ``W // 2 + 1`` time
steps. At step t rank r computes its own queries against the keys of rank ``r - t`` while
``t <= r`` ("local" work). Ranks in the first half run out of local work early (rank r after step
r) and then *help*: at step t > r they take the queries of rank ``r - t + W`` (which are far
behind in the causal order) against their own keys, and send the partial result back, where it is
merged ("sync from remote").
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .comm import print_and_reset_comm_stats  # noqa: F401  (part of the reference's surface)

_SP = {"group": None, "rank": None, "size": None}


# -------------------------------------------------------------------------------------------------
# sequence-parallel group
# -------------------------------------------------------------------------------------------------
def initialize_distributed(backend: Optional[str] = None) -> None:
    """Initialise ``torch.distributed`` from the torchrun variables if needed, select the GPU and
    create the sequence-parallel group over all ranks."""
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        dist.init_process_group(backend=backend)
        if torch.cuda.is_available():
            local_world = int(os.environ.get("LOCAL_WORLD_SIZE", dist.get_world_size()))
            torch.cuda.set_device(dist.get_rank() % local_world)
    if _SP["group"] is None:
        _initialize_sequence_parallel()


def _initialize_sequence_parallel(sequence_parallel_size: Optional[int] = None) -> None:
    """Consecutive ranks form groups of ``sequence_parallel_size`` (default: one group over the
    world). Several groups are allowed here (the reference asserts a single one): each is an
    independent context-parallel domain and the groups are data-parallel to each other."""
    assert dist.is_initialized()
    world = dist.get_world_size()
    size = sequence_parallel_size or world
    assert world % size == 0
    assert _SP["group"] is None, "sequence parallel group is already initialized"
    rank = dist.get_rank()
    for i in range(world // size):
        ranks = list(range(i * size, (i + 1) * size))
        group = dist.new_group(ranks)
        if rank in ranks:
            _SP.update(group=group, rank=ranks.index(rank), size=size)


def get_sequence_parallel_group():
    return _SP["group"]


def get_sequence_parallel_rank() -> int:
    return _SP["rank"] if _SP["rank"] is not None else dist.get_rank()


def get_sequence_parallel_size() -> int:
    return _SP["size"] if _SP["size"] is not None else dist.get_world_size()


def destroy_sequence_parallel() -> None:
    _SP.update(group=None, rank=None, size=None)
    _runtimes.clear()


# -------------------------------------------------------------------------------------------------
# time-step schedule (pure functions; rank / world default to the sequence-parallel group)
# -------------------------------------------------------------------------------------------------
def _rw(rank, world):
    return (get_sequence_parallel_rank() if rank is None else rank,
            get_sequence_parallel_size() if world is None else world)


def num_time_steps(world: Optional[int] = None) -> int:
    return _rw(0, world)[1] // 2 + 1


def is_last_time(time_step: int, rank=None, world=None) -> bool:
    """Whether this is the last step at which rank's own queries are computed on this rank:
    step ``rank`` for the first half (nobody helps them), step ``W // 2`` for the others."""
    r, w = _rw(rank, world)
    return time_step == min(r, w // 2)


def is_compute_for_local_query(time_step: int, rank=None, world=None) -> bool:
    r, w = _rw(rank, world)
    return r >= min(w // 2, time_step)


def is_idle(time_step: int, rank=None, world=None) -> bool:
    """First-half ranks have nothing to do at the last step (even W): every query block that
    needed help has been served by then."""
    return time_step_work(time_step, rank, world)[0] == "idle"


def is_sync_from_remote(time_step: int, rank=None, world=None) -> bool:
    """Whether a helper's partial result for this rank's queries arrives at this step."""
    r, w = _rw(rank, world)
    return r > max(w // 2, w - time_step)


def time_step_work(time_step: int, rank=None, world=None):
    """What rank does at a step: ``("local", key_owner)``, ``("help", query_owner)`` or
    ``("idle", None)``."""
    r, w = _rw(rank, world)
    if time_step <= r and time_step <= w // 2:
        return "local", r - time_step
    helped = r - time_step + w
    if time_step <= w // 2 and helped < w and helped - r > w // 2:
        return "help", helped
    return "idle", None


# -------------------------------------------------------------------------------------------------
# the operator
# -------------------------------------------------------------------------------------------------
_runtimes: dict = {}


def _runtime(q, k, group):
    from .. import patterns as P
    from ..runtime import ContextParallelAttention
    world = dist.get_world_size(group)
    key = (tuple(q.shape), k.shape[2], q.dtype, str(q.device), id(group))
    if key not in _runtimes:
        _runtimes[key] = ContextParallelAttention(
            P.causal(1), q.shape[1] * world, q.shape[2], q.shape[3], group=group, device=q.device,
            n_kv_heads=k.shape[2], batch=q.shape[0], allocation="lightseq",
            path="fused" if q.is_cuda else "nccl", dtype=q.dtype)
    return _runtimes[key]


def attention(q, k, v, causal: bool = True, sm_scale: Optional[float] = None, group=None):
    """DistAttn: ``q`` ``[batch, heads, tokens / W, head_dim]``, ``k`` / ``v`` with the same or
    fewer heads (grouped-query), this rank's contiguous shard; returns the matching shard of the
    output in the same layout. Differentiable."""
    assert causal, "the LightSeq schedule is defined for causal attention"
    group = group if group is not None else (get_sequence_parallel_group() or dist.group.WORLD)
    qt, kt, vt = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    return _runtime(qt, kt, group)(qt, kt, vt, sm_scale).transpose(1, 2)


def extract_local(value, rank: int, world_size: int, device=None, dim: int = 1):
    """This rank's contiguous chunk of ``value`` along ``dim``."""
    out = value.chunk(world_size, dim=dim)[rank]
    return out.to(device) if device is not None else out


# ---- grouped-query helpers under the reference's names (lightseq_async_attn.py:221-247) ----------
# The kernels here take fewer key/value heads directly (``kv_group``), so nothing in this package
# calls these; they serve code written against the reference.
def maybe_repeat_kv_fwd(nqh: int, kv: torch.Tensor) -> torch.Tensor:
    """``[batch, kv_heads, tokens, dim]`` -> ``[batch, nqh, tokens, dim]`` (every head repeated in place)."""
    rep = nqh // kv.shape[1]
    return kv if rep == 1 else kv.repeat_interleave(rep, dim=1)


def maybe_repeat_kv_bwd(nqh: int, kv: torch.Tensor) -> torch.Tensor:
    """``[batch, tokens, kv_heads, dim]`` -> ``[batch, tokens, nqh, dim]``."""
    rep = nqh // kv.shape[2]
    return kv if rep == 1 else kv.repeat_interleave(rep, dim=2)


def maybe_reduce_dkv(nkvh: int, dkv: torch.Tensor) -> torch.Tensor:
    """Gradient of the repeat: ``[batch, tokens, nqh, dim]`` summed over each group of repeated heads."""
    b, s, nqh, d = dkv.shape
    rep = nqh // nkvh
    return dkv if rep == 1 else dkv.reshape(b, s, nkvh, rep, d).sum(dim=3)
