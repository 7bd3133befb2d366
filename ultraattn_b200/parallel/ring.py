"""Ring-family context-parallel baselines on this framework's kernels: ring, zigzag ring, striped
ring (K/V travel around a ring of ranks, every rank keeps its queries) and Ulysses head-parallel
attention (all-to-all between sequence and head sharding).

Reference: ring_flash_attn/ring_flash_attn.py:7-135, zigzag_ring_flash_attn.py:78-283,
stripe_flash_attn.py:7-185, head_parallel_attn/deepspeed_ulysses_attn.py:10-198. The reference
merges partial outputs with a chain of PyTorch element-wise ops (and its zigzag merge is
short-circuited); here every step's kernel merges into the running (O, lse) in its epilogue, so
the results are numerically correct and there is no merge kernel. The striped variant needs no
slicing of Q / K: the kernels take the diagonal offset of the causal mask as a parameter.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import attention as A
from ..ops import elementwise as E
from .comm import A2AComm, RingComm, set_comm_phase


# A rule maps (ring position of the rank whose K/V block is held, own ring position, shard length)
# to this step's work: a list of (q_start, q_len, [(k_start, k_len, causal, diag), ...]), or None
# when the block is invisible. Rules depend on positions only, never on the step number, so the
# same rules serve the flat ring and the two-level ring (which visits the blocks in another order).
def _ring_rule(src, rank, S, causal):
    if not causal:
        return [(0, S, [(0, S, False, 0)])]
    if src == rank:
        return [(0, S, [(0, S, True, 0)])]
    if src < rank:
        return [(0, S, [(0, S, False, 0)])]
    return None


def _zigzag_rule(src, rank, S, causal):
    assert causal, "zigzag sharding is defined for causal attention"
    c = S // 2
    if src == rank:
        return [(0, c, [(0, c, True, 0)]), (c, c, [(0, c, False, 0), (c, c, True, 0)])]
    if src < rank:
        return [(0, S, [(0, c, False, 0)])]
    return [(c, c, [(0, S, False, 0)])]


def _stripe_rule(src, rank, S, causal):
    assert causal, "striped sharding is defined for causal attention"
    # token t of a shard is global token t * world + position: a key of rank src is visible to
    # the query with the same index iff src <= rank, otherwise only to later queries
    return [(0, S, [(0, S, True, 0 if src <= rank else -1)])]


_RULES = {"ring": _ring_rule, "zigzag": _zigzag_rule, "stripe": _stripe_rule}
_NAMES = {"ring": "ring_flash_attn", "zigzag": "zigzag_ring_flash_attn", "stripe": "stripe_flash_attn"}


def _table_work(types, world, src, rank, S):
    """Work of one ring step under a block table: ``types`` is the pattern refined to a multiple of
    the ring size (0 empty, 1 full, 2 causal) and every rank owns ``len(types) / world``
    consecutive blocks of ``S / that`` tokens. Query block i of ``rank`` meets key block j of
    ``src`` iff the table says so; empty pairs are skipped, which is all the block sparsity a ring
    can exploit (the blocks still travel)."""
    per = types.shape[0] // world
    blk = S // per
    out = []
    for i in range(per):
        segs = [(j * blk, blk, int(types[rank * per + i, src * per + j]) == 2, 0)
                for j in range(per) if int(types[rank * per + i, src * per + j])]
        if segs:
            out.append((i * blk, blk, segs))
    return out


def _work(kind, src, rank, bounds, causal, types=None, world=None):
    """The rule applied to every packed sequence ((start, end) pairs of this rank's shard)."""
    if types is not None:
        return _table_work(types, world, src, rank, bounds[0][1] - bounds[0][0])
    out = []
    for a, b in bounds:
        w = _RULES[kind](src, rank, b - a, causal) if b > a else None
        for qs, ql, segs in w or []:
            segs = [(a + ks, kl, c, d) for ks, kl, c, d in segs if kl > 0]
            if ql > 0 and segs:
                out.append((a + qs, ql, segs))
    return out


def _fwd_rows(work, started):
    return [A.Row(0, qs, ql, tuple(A.Seg(0, ks, kl, c, d) for ks, kl, c, d in segs), 0, qs, started)
            for qs, ql, segs in work]


def _bwd_cols(work):
    """Transpose a step's work into key-major form."""
    by_kv = {}
    for qs, ql, segs in work:
        for ks, kl, c, d in segs:
            by_kv.setdefault((ks, kl), []).append(A.Seg(0, qs, ql, c, d))
    return [A.Col(0, ks, kl, tuple(segs), 0, ks) for (ks, kl), segs in sorted(by_kv.items())]


class _Route:
    """The order in which the K/V blocks of all ranks visit this rank.

    One level: a ring over ``group``. Two levels (``intra``, ``inter``): the block makes a full
    tour of the intra-node ring, then one hop on the inter-node ring (to the same local rank of
    the next node), and so on; only every ``len(intra)``-th hop crosses nodes. The ring position
    ``inter_rank * len(intra) + intra_rank`` orders the sequence shards.
    """

    def __init__(self, group=None, intra=None, inter=None, offset: int = 0):
        """``offset`` is added to every ring position (a ring that is one node of a larger job
        reports job-wide positions to the mask rules)."""
        self.levels = [group] if intra is None else [intra, inter]
        self.sizes = [dist.get_world_size(g) for g in self.levels]
        self.pos = [dist.get_rank(g) for g in self.levels]
        self.world = math.prod(self.sizes)
        self.offset = offset
        self.rank = self._flat(self.pos)
        self.shift = [0] * len(self.levels)

    def _flat(self, pos):
        r, mul = self.offset, 1
        for p, n in zip(pos, self.sizes):
            r, mul = r + p * mul, mul * n
        return r

    def comms(self):
        return [RingComm(g) for g in self.levels]

    @property
    def src(self) -> int:
        """Ring position of the rank whose block is held now."""
        return self._flat([(p - s) % n for p, s, n in zip(self.pos, self.shift, self.sizes)])

    def level_after(self, step: int) -> int:
        """The ring that the block takes after compute step ``step``."""
        lvl, n = 0, step + 1
        while lvl + 1 < len(self.sizes) and n % self.sizes[lvl] == 0:
            n //= self.sizes[lvl]
            lvl += 1
        return lvl

    def advance(self, lvl: int) -> None:
        self.shift[lvl] = (self.shift[lvl] + 1) % self.sizes[lvl]

    def send_home(self, tensors):
        """Return travelling buffers to the ranks whose blocks they belong to: one exchange per
        level, to the position ``shift`` places back."""
        for lvl, g in enumerate(self.levels):
            s, n, p = self.shift[lvl], self.sizes[lvl], self.pos[lvl]
            if s == 0:
                continue
            glob = (lambda r: dist.get_global_rank(g, r)) if g is not None else (lambda r: r)
            recv = [torch.empty_like(t) for t in tensors]
            ops = []
            for t, r in zip(tensors, recv):
                ops.append(dist.P2POp(dist.isend, t, glob((p - s) % n), group=g))
                ops.append(dist.P2POp(dist.irecv, r, glob((p + s) % n), group=g))
            for req in dist.batch_isend_irecv(ops):
                req.wait()
            tensors = recv
        return tensors


def _route(group):
    if isinstance(group, _Route):
        group.shift = [0] * len(group.levels)
        return group
    if isinstance(group, dict):
        return _Route(intra=group["intra"], inter=group["inter"])
    return _Route(group)


def ring_forward(q, k, v, group, kind: str, causal: bool, softmax_scale=None, bounds=None, q_rank=None,
                 block_types=None):
    """``group``: a process group (flat ring) or ``{'intra': pg, 'inter': pg}`` (two-level ring).
    ``bounds``: (start, end) of every packed sequence in this rank's shard; default one sequence.
    ``q_rank``: ring position of the rank that owns the queries, when they are a visitor's.
    ``block_types``: a block table (pattern refined to a multiple of the ring size) that replaces
    the dense rule of ``kind``: the ring baseline for block-sparse patterns.

    Accuracy: the running output is held in the input dtype and every ring step's kernel epilogue
    merges into it (log-sum-exp weights in fp32, one rounding to the input dtype per step), so a
    bf16 result carries up to ``world`` roundings of 2^-9 relative each instead of one; the
    reference keeps out / lse in fp32 across steps and casts once
    (ring_flash_attn/utils.py:38-52). lse itself is fp32 throughout."""
    set_comm_phase("fwd")
    route = _route(group)
    q_rank = route.rank if q_rank is None else q_rank
    comms = route.comms()
    k, v = k.contiguous(), v.contiguous()        # they are sent as whole messages
    S = q.shape[1]
    bounds = bounds or [(0, S)]
    o = torch.zeros_like(q)
    lse = torch.full((q.shape[0], q.shape[2], S), float("-inf"), dtype=torch.float32, device=q.device)
    started = False
    for step in range(route.world):
        last = step + 1 == route.world
        if not last:
            lvl = route.level_after(step)
            nk, nv = comms[lvl].send_recv(k), comms[lvl].send_recv(v)
            comms[lvl].commit()
        work = _work(kind, route.src, q_rank, bounds, causal, block_types, route.world)
        if work:
            A.attn_fwd([q], [k], [v], [(o, lse)], A.FwdPlan(_fwd_rows(work, started), q.device), softmax_scale)
            started = True
        if not last:
            comms[lvl].wait()
            route.advance(lvl)
            k, v = nk, nv
    return o, lse


def ring_backward(d_o, q, k, v, o, lse, group, kind: str, causal: bool, softmax_scale=None, bounds=None,
                  q_rank=None, keep_f32: bool = False, block_types=None):
    """``keep_f32``: return the fp32 accumulators instead of casting to the input dtype."""
    set_comm_phase("bwd")
    route = _route(group)
    q_rank = route.rank if q_rank is None else q_rank
    kv_comms, g_comms = route.comms(), route.comms()
    k, v = k.contiguous(), v.contiguous()
    B, S, H, D = q.shape
    bounds = bounds or [(0, S)]
    dvec = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    for b in range(B):
        E.rowdot(o[b], d_o[b], dvec[b])
    dq = torch.zeros(B, S, H, D, dtype=torch.float32, device=q.device)
    dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    side = A.BwdQSide(q, d_o, lse, dvec, dq)
    for step in range(route.world):
        last = step + 1 == route.world
        if not last:
            lvl = route.level_after(step)
            nk, nv = kv_comms[lvl].send_recv(k), kv_comms[lvl].send_recv(v)
            kv_comms[lvl].commit()
        work = _work(kind, route.src, q_rank, bounds, causal, block_types, route.world)
        if work:
            A.attn_bwd([side], [k], [v], [A.BwdKvOut(dk, dv)], A.BwdPlan(_bwd_cols(work), q.device),
                       softmax_scale)
        if not last:
            # the gradient buffers travel with their K/V block
            ndk, ndv = g_comms[lvl].send_recv(dk), g_comms[lvl].send_recv(dv)
            g_comms[lvl].commit()
            kv_comms[lvl].wait()
            g_comms[lvl].wait()
            route.advance(lvl)
            k, v, dk, dv = nk, nv, ndk, ndv
    dk, dv = route.send_home([dk, dv])
    if keep_f32:
        return dq, dk, dv
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


class _RingFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, group, kind, bounds=None, block_types=None):
        o, lse = ring_forward(q, k, v, group, kind, causal, softmax_scale, bounds, block_types=block_types)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.args = (softmax_scale, causal, group, kind, bounds, block_types)
        return o, lse

    @staticmethod
    def backward(ctx, d_o, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, group, kind, bounds, block_types = ctx.args
        dq, dk, dv = ring_backward(d_o.contiguous(), q, k, v, o, lse, group, kind, causal, scale, bounds,
                                   block_types=block_types)
        return dq, dk, dv, None, None, None, None, None, None


def block_sparse_ring_attn_func(q, k, v, pattern, softmax_scale=None, group=None, return_lse: bool = False):
    """Ring attention under a block-sparse pattern: the K/V ring of :func:`ring_flash_attn_func`
    with contiguous shards, where every step computes only the block pairs that the pattern
    allows. This is what a ring-based context-parallel system can do with block sparsity (skip
    compute, still move every block), i.e. the "Ring" baseline of the block-sparse comparisons."""
    world = dist.get_world_size(group)
    n = pattern.table.shape[0]
    par_d = n * world // math.gcd(n, world)
    types = pattern.refined(par_d)
    o, lse = _RingFunc.apply(q, k, v, softmax_scale, False, group, "ring", None, types)
    return (o, lse) if return_lse else o


def _check_unsupported(dropout_p, alibi_slopes, window_size):
    assert dropout_p == 0.0 and alibi_slopes is None and tuple(window_size) == (-1, -1), \
        "dropout, alibi and sliding windows are not part of these baselines"


def _make_func(kind: str):
    def func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
             alibi_slopes=None, deterministic=False, return_attn_probs=False, group=None,
             PROC_INFO=None, opt=False, groups=None):
        group = groups if groups is not None else group        # the reference's keyword is ``groups``
        if kind == "ring" and tuple(int(x) for x in window_size) != (-1, -1) and not isinstance(group, dict):
            # a causal sliding window over the ring's contiguous shards: only the window's keys
            # travel (parallel/halo.py) instead of every shard going round
            _check_unsupported(dropout_p, alibi_slopes, (-1, -1))
            assert not return_attn_probs, "the windowed form returns the output only"
            from .halo import halo_window_attn_func
            return halo_window_attn_func(q, k, v, window_size, softmax_scale, causal, group)
        _check_unsupported(dropout_p, alibi_slopes, window_size)
        o, lse = _RingFunc.apply(q, k, v, softmax_scale, causal, group, kind)
        return (o, lse, None) if return_attn_probs else o
    func.__name__ = _NAMES[kind] + "_func"
    func.__doc__ = (f"{kind} context-parallel attention: q, k, v are this rank's shard "
                    "[batch, tokens, heads, head_dim]; same signature as the reference's function. "
                    "``group`` may also be {'intra': pg, 'inter': pg} for the two-level ring.")
    return func


def _make_varlen_func(kind: str):
    def func(q, k, v, cu_seqlens, max_seqlen=None, dropout_p=0.0, softmax_scale=None, causal=False,
             window_size=(-1, -1), alibi_slopes=None, deterministic=False, return_attn_probs=False,
             group=None):
        _check_unsupported(dropout_p, alibi_slopes, window_size)
        cu = [int(x) for x in cu_seqlens]
        bounds = list(zip(cu[:-1], cu[1:]))
        o, lse = _RingFunc.apply(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), softmax_scale, causal,
                                 group, kind, bounds)
        o = o.squeeze(0)
        return (o, lse.squeeze(0), None) if return_attn_probs else o
    func.__name__ = _NAMES[kind] + "_varlen_func"
    func.__doc__ = (
        f"{kind} context-parallel attention over a packed batch. q, k, v: ``[tokens, heads, head_dim]``, "
        "this rank's shard of every sequence one after the other; ``cu_seqlens`` are the boundaries "
        "of those shards (the same on every rank: each sequence is cut evenly, "
        "ring_flash_attn/ring_flash_attn_varlen.py:24-79; zigzag shards hold chunks r and 2W-1-r of "
        "each sequence, zigzag_ring_flash_attn_varlen.py:23-56). Tokens attend only their own "
        "sequence. ``max_seqlen`` is accepted for signature parity and not needed: the kernels take "
        "(query block, key segment) lists, so the returned lse is already packed ``[heads, tokens]`` "
        "and no flatten / unflatten pass exists.")
    return func


def _packed_variants(func, varlen: bool = False):
    """The (qkv-packed, kv-packed) forms of an attention function: q, k, v stacked along a new
    dimension right after the token dimension."""
    dim = 1 if varlen else 2

    def qkvpacked(qkv, *a, **kw):
        q, k, v = qkv.unbind(dim)
        return func(q, k, v, *a, **kw)

    def kvpacked(q, kv, *a, **kw):
        k, v = kv.unbind(dim)
        return func(q, k, v, *a, **kw)

    base = func.__name__[:-len("_func")]
    qkvpacked.__name__, kvpacked.__name__ = base + "_qkvpacked_func", base + "_kvpacked_func"
    return qkvpacked, kvpacked


ring_flash_attn_func = _make_func("ring")
zigzag_ring_flash_attn_func = _make_func("zigzag")
stripe_flash_attn_func = _make_func("stripe")
ring_flash_attn_varlen_func = _make_varlen_func("ring")
zigzag_ring_flash_attn_varlen_func = _make_varlen_func("zigzag")

ring_flash_attn_qkvpacked_func, ring_flash_attn_kvpacked_func = _packed_variants(ring_flash_attn_func)
zigzag_ring_flash_attn_qkvpacked_func, zigzag_ring_flash_attn_kvpacked_func = \
    _packed_variants(zigzag_ring_flash_attn_func)
stripe_flash_attn_qkvpacked_func, stripe_flash_attn_kvpacked_func = _packed_variants(stripe_flash_attn_func)
ring_flash_attn_varlen_qkvpacked_func, ring_flash_attn_varlen_kvpacked_func = \
    _packed_variants(ring_flash_attn_varlen_func, varlen=True)
zigzag_ring_flash_attn_varlen_qkvpacked_func, zigzag_ring_flash_attn_varlen_kvpacked_func = \
    _packed_variants(zigzag_ring_flash_attn_varlen_func, varlen=True)


# -------------------------------------------------------------------------------------------------
# The per-strategy forward / backward functions and autograd classes under the reference's names
# and positional signatures (ring_flash_attn/ring_flash_attn.py:7-200, zigzag_ring_flash_attn.py:
# 78-356, stripe_flash_attn.py:7-252 and the two *_varlen.py files). They all run the one ring
# above; what differs between the strategies is the mask rule chosen by ``kind``.
# -------------------------------------------------------------------------------------------------
def _bounds_of(cu_seqlens):
    cu = [int(x) for x in cu_seqlens]
    return list(zip(cu[:-1], cu[1:]))


def _make_kernel_level(kind: str, varlen: bool = False):
    base = _NAMES[kind] + ("_varlen" if varlen else "")

    if not varlen:
        def forward(process_group, q, k, v, softmax_scale, dropout_p=0, causal=True, window_size=(-1, -1),
                    alibi_slopes=None, deterministic=False, PROC_INFO=None, opt=False):
            _check_unsupported(dropout_p, alibi_slopes, window_size)
            return ring_forward(q, k, v, process_group, kind, causal, softmax_scale)

        def backward(process_group, dout, q, k, v, out, softmax_lse, softmax_scale, dropout_p=0, causal=True,
                     window_size=(-1, -1), alibi_slopes=None, deterministic=False, PROC_INFO=None, opt=False):
            _check_unsupported(dropout_p, alibi_slopes, window_size)
            return ring_backward(dout.contiguous(), q, k, v, out, softmax_lse, process_group, kind, causal,
                                 softmax_scale)
    elif kind == "zigzag":
        # the reference's zigzag forms carry two precomputed half-sequence indices (zigzag_ring_flash_attn_varlen.py:
        # 58-70, 153-168); the kernels here mask by position, so they are accepted and not needed
        def forward(process_group, q, k, v, cu_seqlens, max_seqlen, half_index0=None, half_index1=None,
                    softmax_scale=None, dropout_p=0, causal=True, window_size=(-1, -1), alibi_slopes=None,
                    deterministic=False):
            _check_unsupported(dropout_p, alibi_slopes, window_size)
            o, lse = ring_forward(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), process_group, kind, causal,
                                  softmax_scale, _bounds_of(cu_seqlens))
            return o.squeeze(0), lse.squeeze(0)

        def backward(process_group, dout, q, k, v, out, softmax_lse, cu_seqlens, max_seqlen, half_index0=None,
                     half_index1=None, softmax_scale=None, dropout_p=0, causal=True, window_size=(-1, -1),
                     alibi_slopes=None, deterministic=False):
            _check_unsupported(dropout_p, alibi_slopes, window_size)
            lse = softmax_lse if softmax_lse.dim() == 3 else softmax_lse.unsqueeze(0)
            grads = ring_backward(dout.unsqueeze(0).contiguous(), q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0),
                                  out.unsqueeze(0), lse, process_group, kind, causal, softmax_scale,
                                  _bounds_of(cu_seqlens))
            return tuple(g.squeeze(0) for g in grads)
    else:
        def forward(process_group, q, k, v, cu_seqlens, max_seqlen, softmax_scale, dropout_p=0, causal=True,
                    window_size=(-1, -1), alibi_slopes=None, deterministic=False):
            _check_unsupported(dropout_p, alibi_slopes, window_size)
            o, lse = ring_forward(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), process_group, kind, causal,
                                  softmax_scale, _bounds_of(cu_seqlens))
            return o.squeeze(0), lse.squeeze(0)

        def backward(process_group, dout, q, k, v, out, softmax_lse, cu_seqlens, max_seqlen, softmax_scale,
                     dropout_p=0, causal=True, window_size=(-1, -1), alibi_slopes=None, deterministic=False):
            _check_unsupported(dropout_p, alibi_slopes, window_size)
            lse = softmax_lse if softmax_lse.dim() == 3 else softmax_lse.unsqueeze(0)
            grads = ring_backward(dout.unsqueeze(0).contiguous(), q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0),
                                  out.unsqueeze(0), lse, process_group, kind, causal, softmax_scale,
                                  _bounds_of(cu_seqlens))
            return tuple(g.squeeze(0) for g in grads)
    forward.__name__, backward.__name__ = base + "_forward", base + "_backward"
    forward.__doc__ = (f"(out, lse) of {kind} attention on this rank's shard; positional signature of the "
                       f"reference's ``{base}_forward``; lse is ``[batch, heads, tokens]`` (packed: ``[heads, tokens]``).")
    backward.__doc__ = f"(dq, dk, dv); positional signature of the reference's ``{base}_backward``."
    return forward, backward


def _make_func_class(kind: str, name: str, varlen: bool = False):
    """An autograd class whose ``apply`` takes the reference's argument list (``..., return_softmax,
    group[, PROC_INFO, opt]``) and returns what the reference's returns (out, or (out, lse, None))."""
    if not varlen:
        def fwd(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes, deterministic,
                return_softmax, group, PROC_INFO=None, opt=False):
            _check_unsupported(dropout_p, alibi_slopes, window_size)
            o, lse = ring_forward(q, k, v, group, kind, causal, softmax_scale)
            ctx.save_for_backward(q, k, v, o, lse)
            ctx.args = (softmax_scale, causal, group, None)
            ctx.n_in = 13
            return (o, lse, None) if return_softmax else o
    else:
        def fwd(ctx, q, k, v, cu_seqlens, max_seqlen, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                deterministic, return_softmax, group):
            _check_unsupported(dropout_p, alibi_slopes, window_size)
            bounds = _bounds_of(cu_seqlens)
            o, lse = ring_forward(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), group, kind, causal,
                                  softmax_scale, bounds)
            ctx.save_for_backward(q, k, v, o, lse)
            ctx.args = (softmax_scale, causal, group, bounds)
            ctx.n_in = 13
            return (o.squeeze(0), lse.squeeze(0), None) if return_softmax else o.squeeze(0)

    def bwd(ctx, dout, *rest):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, group, bounds = ctx.args
        if bounds is None:
            grads = ring_backward(dout.contiguous(), q, k, v, o, lse, group, kind, causal, scale)
        else:
            grads = ring_backward(dout.unsqueeze(0).contiguous(), q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0),
                                  o, lse, group, kind, causal, scale, bounds)
            grads = tuple(g.squeeze(0) for g in grads)
        return tuple(grads) + (None,) * (ctx.n_in - 3)

    return type(name, (torch.autograd.Function,), {"forward": staticmethod(fwd), "backward": staticmethod(bwd),
                                                   "__doc__": f"{kind} attention as an autograd function with the "
                                                              "reference's ``apply`` argument list."})


ring_flash_attn_forward, ring_flash_attn_backward = _make_kernel_level("ring")
zigzag_ring_flash_attn_forward, zigzag_ring_flash_attn_backward = _make_kernel_level("zigzag")
stripe_flash_attn_forward, stripe_flash_attn_backward = _make_kernel_level("stripe")
ring_flash_attn_varlen_forward, ring_flash_attn_varlen_backward = _make_kernel_level("ring", varlen=True)
zigzag_ring_flash_attn_varlen_forward, zigzag_ring_flash_attn_varlen_backward = _make_kernel_level("zigzag", varlen=True)
RingFlashAttnFunc = _make_func_class("ring", "RingFlashAttnFunc")
ZigZagRingFlashAttnFunc = _make_func_class("zigzag", "ZigZagRingFlashAttnFunc")
StripeFlashAttnFunc = _make_func_class("stripe", "StripeFlashAttnFunc")
RingFlashAttnVarlenFunc = _make_func_class("ring", "RingFlashAttnVarlenFunc", varlen=True)
ZigZagRingFlashAttnVarlenFunc = _make_func_class("zigzag", "ZigZagRingFlashAttnVarlenFunc", varlen=True)


def get_half_index(cu_seqlens, *, front: bool):
    """Index (slice for one sequence, boolean mask otherwise) of the front or back half of every
    packed sequence (reference: zigzag_ring_flash_attn_varlen.py:23-40)."""
    cu = [int(x) for x in cu_seqlens]
    if len(cu) == 2:
        half = cu[1] // 2
        return slice(None, half) if front else slice(half, None)
    index = torch.zeros(cu[-1], dtype=torch.bool)
    for a, b in zip(cu[:-1], cu[1:]):
        mid = (a + b) // 2
        if front:
            index[a:mid] = True
        else:
            index[mid:b] = True
    return index


def get_half_lse(lse: torch.Tensor, cu_seqlens, *, front: bool) -> torch.Tensor:
    """The front or back half of every sequence of a padded lse ``[sequences, heads, max_len]``
    (reference: zigzag_ring_flash_attn_varlen.py:42-55)."""
    cu = [int(x) for x in cu_seqlens]
    out = torch.zeros(lse.shape[0], lse.shape[1], lse.shape[2] // 2, dtype=lse.dtype, device=lse.device)
    for i, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        n = b - a
        lo, hi = (0, n // 2) if front else (n // 2, n)
        out[i, :, :hi - lo] = lse[i, :, lo:hi]
    return out


# -------------------------------------------------------------------------------------------------
# input sharding helpers (reference: easy_context/zigzag_ring_attn/prepare_inputs.py:4-40)
# -------------------------------------------------------------------------------------------------
def shard_sequence(x: torch.Tensor, rank: int, world: int, kind: str, dim: int = 1) -> torch.Tensor:
    """This rank's shard of a full-sequence tensor under the layout each strategy expects."""
    if kind in ("ring", "ulysses", "halo"):
        return x.chunk(world, dim=dim)[rank].contiguous()
    if kind == "zigzag":
        ch = x.chunk(2 * world, dim=dim)
        return torch.cat([ch[rank], ch[2 * world - 1 - rank]], dim=dim).contiguous()
    if kind == "stripe":
        idx = torch.arange(rank, x.shape[dim], world, device=x.device)
        return x.index_select(dim, idx).contiguous()
    raise ValueError(kind)


def shard_packed(x: torch.Tensor, cu_seqlens, rank: int, world: int, kind: str):
    """Shard a packed batch ``[tokens, ...]`` sequence by sequence; returns this rank's shard and
    the boundaries of the sequences inside it (every sequence length must divide evenly: by
    ``world`` for the ring, by ``2 * world`` for zigzag)."""
    cu = [int(c) for c in cu_seqlens]
    parts = [shard_sequence(x[a:b], rank, world, kind, dim=0) for a, b in zip(cu[:-1], cu[1:])]
    local = [0]
    for p in parts:
        local.append(local[-1] + p.shape[0])
    return torch.cat(parts, dim=0).contiguous(), local


# -------------------------------------------------------------------------------------------------
# Ulysses
# -------------------------------------------------------------------------------------------------
def deepspeed_ulysses_attn_forward(process_groups, q_s, k_s, v_s, softmax_scale, dropout_p=0, causal=True,
                                   window_size=(-1, -1), alibi_slopes=None, deterministic=False, PROC_INFO=None,
                                   opt=False):
    """Head-parallel forward on sequence shards ``[B, S/sp, H, D]``: all-to-all to ``[B, S, H/sp, D]``,
    attention over whole sequences, all-to-all back. Returns ``(out_s, q_h, k_h, v_h, out_h, lse_h)``:
    the output in the sequence sharding and the head-sharded tensors the backward takes (argument
    list of head_parallel_attn/deepspeed_ulysses_attn.py:10-47, whose compute step is missing)."""
    from ..api import local_plans
    from ..patterns import named
    _check_unsupported(dropout_p, alibi_slopes, (-1, -1))
    a2a = A2AComm(process_groups)
    qh, kh, vh = (a2a.all_to_all(t, 2, 1) for t in (q_s, k_s, v_s))       # [B, S, H/sp, D]
    if tuple(int(x) for x in window_size) != (-1, -1):
        # whole sequences on every rank: a sliding window is the single-device operator
        from ..ops.window import window_forward
        oh, lse = window_forward(qh, kh, vh, window_size, bool(causal), softmax_scale)
        return a2a.all_to_all(oh, 1, 2), qh, kh, vh, oh, lse
    fplan, _ = local_plans(named.causal(1) if causal else named.full(1), qh.shape[1], qh.device)
    oh = torch.empty_like(qh)
    lse = torch.empty(qh.shape[0], qh.shape[2], qh.shape[1], dtype=torch.float32, device=qh.device)
    A.attn_fwd([qh], [kh], [vh], [(oh, lse)], fplan, softmax_scale)
    return a2a.all_to_all(oh, 1, 2), qh, kh, vh, oh, lse


def deepspeed_ulysses_attn_backward(process_group, dout_s, q_h, k_h, v_h, out_h, softmax_lse, softmax_scale=None,
                                    dropout_p=0, causal=True, window_size=(-1, -1), alibi_slopes=None,
                                    deterministic=False, opt=False):
    """Gradients in the sequence sharding from the head-sharded tensors of the forward (argument
    list of head_parallel_attn/deepspeed_ulysses_attn.py:49-95)."""
    from ..api import local_backward, local_plans
    from ..patterns import named
    _check_unsupported(dropout_p, alibi_slopes, (-1, -1))
    a2a = A2AComm(process_group)
    doh = a2a.all_to_all(dout_s.contiguous(), 2, 1)
    if tuple(int(x) for x in window_size) != (-1, -1):
        from ..ops.window import window_backward
        dq, dk, dv = window_backward(doh, q_h, k_h, v_h, out_h, softmax_lse, window_size, bool(causal), softmax_scale)
        return tuple(a2a.all_to_all(t, 1, 2) for t in (dq, dk, dv))
    _, bplan = local_plans(named.causal(1) if causal else named.full(1), q_h.shape[1], q_h.device)
    dq, dk, dv = local_backward(q_h, k_h, v_h, out_h, softmax_lse, doh, bplan, softmax_scale)
    return tuple(a2a.all_to_all(t, 1, 2) for t in (dq, dk, dv))


class DeepSpeedUlyssesAttnFunc(torch.autograd.Function):
    """``apply(q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes, deterministic,
    return_softmax, groups[, PROC_INFO, opt])`` as in the reference (deepspeed_ulysses_attn.py:97-166)."""

    @staticmethod
    def forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes, deterministic,
                return_softmax, groups, PROC_INFO=None, opt=False):
        out_s, qh, kh, vh, oh, lse = deepspeed_ulysses_attn_forward(groups, q, k, v, softmax_scale, dropout_p, causal,
                                                                    window_size, alibi_slopes, deterministic)
        ctx.save_for_backward(qh, kh, vh, oh, lse)
        ctx.args = (softmax_scale, causal, groups, tuple(window_size))
        return (out_s, lse, None) if return_softmax else out_s

    @staticmethod
    def backward(ctx, d_o, *rest):
        qh, kh, vh, oh, lse = ctx.saved_tensors
        scale, causal, groups, window = ctx.args
        grads = deepspeed_ulysses_attn_backward(groups, d_o, qh, kh, vh, oh, lse, scale, causal=causal,
                                                window_size=window)
        return tuple(grads) + (None,) * 10


def deepspeed_ulysses_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                                window_size=(-1, -1), alibi_slopes=None, deterministic=False,
                                return_attn_probs=False, group=None, PROC_INFO=None, groups=None, opt=False):
    """Head-parallel attention: inputs are sequence shards ``[B, S/sp, H, D]``; an all-to-all
    re-shards to ``[B, S, H/sp, D]``, attention runs on whole sequences, a second all-to-all
    restores the sequence sharding. ``groups`` (the reference's keyword) and ``group`` name the
    same process group. ``window_size``: sliding window (``ops/window.py``), the one context-parallel
    strategy here that takes token-exact windows. (The reference's version is a stub whose compute step is missing,
    head_parallel_attn/deepspeed_ulysses_attn.py:43-47.)"""
    return DeepSpeedUlyssesAttnFunc.apply(q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                                          deterministic, return_attn_probs, groups if groups is not None else group,
                                          PROC_INFO, opt)


# -------------------------------------------------------------------------------------------------
# helper functions with the reference's names (ring_flash_attn/utils.py:38-121). The strategies
# above do not need them (the kernels merge in their epilogue and work on packed layouts); they
# serve code written against the reference.
# -------------------------------------------------------------------------------------------------
def update_out_and_lse(out, lse, block_out, block_lse, slice_=None):
    """Merge a block's ``(block_out [B, S, H, D], block_lse [B, H, S])`` into the running
    ``(out [B, S, H, D], lse [B, S, H, 1])`` with the log-sum-exp rule; the first call (``out`` is
    None) adopts the block. ``slice_`` restricts the update to part of the running state. Unlike
    the reference's formula, rows where either side is empty (lse = -inf) stay finite."""
    blse = block_lse.transpose(-2, -1).unsqueeze(-1).float()
    if out is None:
        if slice_ is not None:
            raise RuntimeError("first update_out_and_lse should not pass slice_ args")
        return block_out, blse
    o_run, l_run = (out, lse) if slice_ is None else (out[slice_], lse[slice_])
    new = torch.logaddexp(l_run, blse)
    safe = new.masked_fill(new == float("-inf"), 0.0)
    w_old = torch.where(torch.isfinite(l_run), torch.exp(l_run - safe), torch.zeros_like(new))
    w_new = torch.where(torch.isfinite(blse), torch.exp(blse - safe), torch.zeros_like(new))
    merged = (w_old * o_run.float() + w_new * block_out.float()).to(o_run.dtype)
    if slice_ is None:
        return merged, new
    out[slice_], lse[slice_] = merged, new
    return out, lse


def flatten_varlen_lse(lse: torch.Tensor, cu_seqlens) -> torch.Tensor:
    """Padded ``[n_seq, heads, max_len]`` -> packed ``[heads, total_tokens]``."""
    cu = [int(c) for c in cu_seqlens]
    return torch.cat([lse[i, :, :b - a] for i, (a, b) in enumerate(zip(cu[:-1], cu[1:]))], dim=1)


def unflatten_varlen_lse(lse: torch.Tensor, cu_seqlens, max_seqlen: int) -> torch.Tensor:
    """Packed ``[total_tokens, heads, 1]`` (or ``[total_tokens, heads]``) -> padded
    ``[n_seq, heads, max_seqlen]``; the padding is zero."""
    cu = [int(c) for c in cu_seqlens]
    if lse.dim() == 3:
        lse = lse.squeeze(-1)
    out = torch.zeros(len(cu) - 1, max_seqlen, lse.shape[1], dtype=torch.float32, device=lse.device)
    for i, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        out[i, :b - a] = lse[a:b]
    return out.transpose(1, 2).contiguous()
