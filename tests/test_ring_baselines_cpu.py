"""Ring / zigzag / stripe / Ulysses baselines on CPU ranks over gloo against dense attention."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, cases, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out = {}
        for kind, causal in cases:
            out[f"{kind}-{causal}"] = _one_baseline(rank, world, kind, causal)
        ret[rank] = out
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def _one_baseline(rank, world, kind, causal):
    from ultraattn_b200 import parallel as PL, patterns as P
    S, H, D = 256, 4, 16
    g = torch.Generator().manual_seed(0)
    q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
    if kind.startswith("bsa:"):                     # the ring under a block-sparse pattern
        pat = {"strided": P.strided(8, 4, 2), "global_local": P.global_local(8, 1, 2), "star": P.star(4, 1)}[kind[4:]]
        sh = lambda t: PL.shard_sequence(t, rank, world, "ring")
        ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
        o = PL.block_sparse_ring_attn_func(ql, kl, vl, pat)
        o.backward(sh(d_o))
        o_ref, _, dq, dk, dv = P.dense_attention_with_grads(q, k, v, d_o, pat)
        return max((o - sh(o_ref)).abs().max().item(), (ql.grad - sh(dq)).abs().max().item(),
                   (kl.grad - sh(dk)).abs().max().item(), (vl.grad - sh(dv)).abs().max().item())
    if kind.startswith("halo2:"):                   # two-sided window: halos from both neighbours (or farther)
        left, right = (int(x) for x in kind[6:].split(","))
        sh = lambda t: PL.shard_sequence(t, rank, world, "halo")
        ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
        o = PL.halo_window_attn_func(ql, kl, vl, (left, right), causal=False)
        o.backward(sh(d_o))
        r, c = torch.arange(S)[:, None], torch.arange(S)[None, :]
        mask = (c >= r - left) & (c <= r + right)
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        sc = torch.einsum("bqhd,bkhd->bhqk", qq, kk) / D ** 0.5
        o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc.masked_fill(~mask, float("-inf")), -1), vv)
        o_ref.backward(d_o)
        return max((o - sh(o_ref.detach())).abs().max().item(), (ql.grad - sh(qq.grad)).abs().max().item(),
                   (kl.grad - sh(kk.grad)).abs().max().item(), (vl.grad - sh(vv.grad)).abs().max().item())
    if kind.startswith("halo:"):                    # causal sliding window by halo exchange; the window may span ranks
        left = int(kind[5:])
        sh = lambda t: PL.shard_sequence(t, rank, world, "halo")
        kk2, vv2 = k[:, :, :2], v[:, :, :2]          # grouped-query heads
        ql, kl, vl = (sh(t).requires_grad_() for t in (q, kk2, vv2))
        # through the strategy's own name, and through the ring function's window_size argument
        o = PL.halo_window_attn_func(ql, kl, vl, (left, 0)) if left != 64 else \
            PL.ring_flash_attn_func(ql, kl, vl, causal=True, window_size=(left, 0))
        o.backward(sh(d_o))
        r, c = torch.arange(S)[:, None], torch.arange(S)[None, :]
        mask = (c >= r - left) & (c <= r)
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, kk2, vv2))
        sc = torch.einsum("bqhd,bkhd->bhqk", qq, kk.repeat_interleave(2, 2)) / D ** 0.5
        o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc.masked_fill(~mask, float("-inf")), -1),
                             vv.repeat_interleave(2, 2))
        o_ref.backward(d_o)
        return max((o - sh(o_ref.detach())).abs().max().item(), (ql.grad - sh(qq.grad)).abs().max().item(),
                   (kl.grad - sh(kk.grad)).abs().max().item(), (vl.grad - sh(vv.grad)).abs().max().item())
    if kind == "ulysses-window":                    # head-parallel attention with a token-exact sliding window
        sh = lambda t: PL.shard_sequence(t, rank, world, "ulysses")
        ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
        o = PL.deepspeed_ulysses_attn_func(ql, kl, vl, causal=causal, window_size=(70, 0 if causal else 9))
        o.backward(sh(d_o))
        r, c = torch.arange(S)[:, None], torch.arange(S)[None, :]
        mask = (c >= r - 70) & (c <= r + (0 if causal else 9))
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        sc = torch.einsum("bqhd,bkhd->bhqk", qq, kk) / D ** 0.5
        o_ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc.masked_fill(~mask, float("-inf")), -1), vv)
        o_ref.backward(d_o)
        return max((o - sh(o_ref.detach())).abs().max().item(), (ql.grad - sh(qq.grad)).abs().max().item(),
                   (kl.grad - sh(kk.grad)).abs().max().item(), (vl.grad - sh(vv.grad)).abs().max().item())
    sh = lambda t: PL.shard_sequence(t, rank, world, kind)
    ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
    fn = {"ring": PL.ring_flash_attn_func, "zigzag": PL.zigzag_ring_flash_attn_func,
          "stripe": PL.stripe_flash_attn_func, "ulysses": PL.deepspeed_ulysses_attn_func}[kind]
    o = fn(ql, kl, vl, causal=causal)
    o.backward(sh(d_o))
    pat = P.causal(1) if causal else P.full(1)
    o_ref, _, dq, dk, dv = P.dense_attention_with_grads(q, k, v, d_o, pat)
    return max((o - sh(o_ref)).abs().max().item(), (ql.grad - sh(dq)).abs().max().item(),
               (kl.grad - sh(dk)).abs().max().item(), (vl.grad - sh(dv)).abs().max().item())


def _check(ret, world):
    for r in range(world):
        assert isinstance(ret[r], dict), ret[r]
        for name, err in ret[r].items():
            assert err < 2e-4, (r, name, err)


def test_baselines_world4():
    """Ring (causal and full), zigzag, stripe, Ulysses and the ring under three block-sparse
    patterns on four ranks, one process group."""
    cases = [("ring", True), ("ring", False), ("zigzag", True), ("stripe", True), ("ulysses", True),
             ("ulysses-window", True), ("ulysses-window", False), ("halo:20", True), ("halo:64", True),
             ("halo:150", True), ("halo:1000", True), ("halo2:30,10", False), ("halo2:100,70", False),
             ("halo2:0,64", False), ("bsa:strided", False), ("bsa:global_local", False), ("bsa:star", False)]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(4, 29900 + os.getpid() % 90, cases, ret), nprocs=4, join=True)
    _check(ret, 4)


def _dense_packed(q, k, v, d_o, cu, causal):
    """Dense oracle of a packed batch: every sequence on its own."""
    from ultraattn_b200 import patterns as P
    pat = P.causal(1) if causal else P.full(1)
    outs = [P.dense_attention_with_grads(*(t[None, a:b] for t in (q, k, v, d_o)), pat)
            for a, b in zip(cu[:-1], cu[1:])]
    return [torch.cat([o[i][0] for o in outs], dim=0) for i in (0, 2, 3, 4)]


def _varlen_worker(rank, world, port, cases, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = {f"{kind}-{causal}": _one_varlen(rank, world, kind, causal) for kind, causal in cases}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def _one_varlen(rank, world, kind, causal):
    from ultraattn_b200 import parallel as PL
    H, D = 2, 16
    cu = [0, 64, 64, 192, 224]          # lengths 64, 0, 128, 32
    g = torch.Generator().manual_seed(3)
    q, k, v, d_o = (torch.randn(cu[-1], H, D, generator=g) for _ in range(4))
    sh = lambda t: PL.shard_packed(t, cu, rank, world, kind)[0]
    local_cu = PL.shard_packed(q, cu, rank, world, kind)[1]
    ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
    fn = {"ring": PL.ring_flash_attn_varlen_func, "zigzag": PL.zigzag_ring_flash_attn_varlen_func}[kind]
    o = fn(ql, kl, vl, local_cu, max(b - a for a, b in zip(local_cu[:-1], local_cu[1:])), causal=causal)
    o.backward(sh(d_o))
    # the kv-packed form must give the same output
    kvp = getattr(PL, fn.__name__.replace("_func", "_kvpacked_func"))
    o2 = kvp(ql.detach(), torch.stack([kl.detach(), vl.detach()], dim=1), local_cu, None, causal=causal)
    o_ref, dq, dk, dv = _dense_packed(q, k, v, d_o, cu, causal)
    return max((o - sh(o_ref)).abs().max().item(), (ql.grad - sh(dq)).abs().max().item(),
               (kl.grad - sh(dk)).abs().max().item(), (vl.grad - sh(dv)).abs().max().item(),
               (o2 - o.detach()).abs().max().item())


def test_varlen_baselines_world2():
    """Packed batches through the ring (causal and full) and the zigzag ring on two ranks."""
    cases = [("ring", True), ("ring", False), ("zigzag", True)]
    ret = mp.Manager().dict()
    mp.spawn(_varlen_worker, args=(2, 29700 + os.getpid() % 90, cases, ret), nprocs=2, join=True)
    _check(ret, 2)


def _hierarchy_worker(rank, world, port, cases, ret, per_node=2, S=256):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = {f"{mode}-{causal}": _one_hierarchy(rank, world, causal, mode, per_node, S) for causal, mode in cases}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def _one_hierarchy(rank, world, causal, mode, per_node, S):
    from ultraattn_b200 import parallel as PL, patterns as P
    H, D = 2, 16
    g = torch.Generator().manual_seed(4)
    q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
    kind = "zigzag" if causal else "ring"
    sh = lambda t: PL.shard_sequence(t, rank, world, kind)
    groups = PL.create_hierarchy_groups(tasks_per_node=per_node)
    ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
    o = PL.hierarchy_attn_func(ql, kl, vl, causal=causal, groups=groups, mode=mode)
    o.backward(sh(d_o))
    pat = P.causal(1) if causal else P.full(1)
    o_ref, _, dq, dk, dv = P.dense_attention_with_grads(q, k, v, d_o, pat)
    return max((o - sh(o_ref)).abs().max().item(), (ql.grad - sh(dq)).abs().max().item(),
               (kl.grad - sh(dk)).abs().max().item(), (vl.grad - sh(dv)).abs().max().item())


def test_two_level_ring_2x2():
    """Two nodes of two ranks: both modes, causal (zigzag shards) and full."""
    cases = [(True, "kv"), (False, "kv"), (True, "qo"), (False, "qo")]
    ret = mp.Manager().dict()
    mp.spawn(_hierarchy_worker, args=(4, 29600 + os.getpid() % 90, cases, ret), nprocs=4, join=True)
    _check(ret, 4)


def test_two_level_ring_3_nodes():
    """Three nodes of two ranks: the query / output exchange visits two other nodes (the second
    visitor is requested while the first is computed)."""
    ret = mp.Manager().dict()
    mp.spawn(_hierarchy_worker, args=(6, 29500 + os.getpid() % 90, [(True, "kv"), (True, "qo")], ret, 2, 240),
             nprocs=6, join=True)
    _check(ret, 6)


def test_lightseq_time_steps_match_the_allocation_table():
    """The worker / helper time-step view restates the balanced allocation table: every causal
    tile is computed exactly once, by the rank the table names."""
    from ultraattn_b200.parallel import lightseq as LS
    from ultraattn_b200.planner.dense import get_lightseq_schedule_table
    for w in (2, 4, 5, 8):
        table = get_lightseq_schedule_table(w)
        seen = {}
        for r in range(w):
            for t in range(LS.num_time_steps(w)):
                kind, other = LS.time_step_work(t, r, w)
                tile = (r, other) if kind == "local" else (other, r) if kind == "help" else None
                if tile is not None:
                    assert tile not in seen and table[tile] == r, (w, r, t, tile)
                    seen[tile] = r
        assert len(seen) == w * (w + 1) // 2
    # the reference's predicates on its 8-rank example
    assert [t for t in range(5) if LS.is_last_time(t, 5, 8)] == [4] and LS.is_last_time(2, 2, 8)
    assert [t for t in range(5) if LS.is_compute_for_local_query(t, 1, 8)] == [0, 1]
    assert [r for r in range(8) if LS.is_idle(4, r, 8)] == [0, 1, 2, 3]
    assert [t for t in range(5) if LS.is_sync_from_remote(t, 7, 8)] == [2, 3, 4]
    assert not any(LS.is_sync_from_remote(t, 4, 8) for t in range(5))


def _lightseq_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    try:
        from easy_context.dist_flash_attn import async_communication as AC
        from easy_context.dist_flash_attn.lightseq_async_attn import attention
        from easy_context.dist_flash_attn.prepare_input import extract_local
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.parallel.comm import comm_stats
        AC.initialize_distributed("gloo")
        assert AC.get_sequence_parallel_size() == world and AC.get_sequence_parallel_rank() == rank
        S, H, Hk, D = 256, 4, 2, 16
        g = torch.Generator().manual_seed(9)
        q, d_o = (torch.randn(1, H, S, D, generator=g) for _ in range(2))      # [batch, heads, tokens, dim]
        k, v = (torch.randn(1, Hk, S, D, generator=g) for _ in range(2))
        loc = lambda t: extract_local(t, rank, world, dim=2).contiguous()
        ql, kl, vl = (loc(t).requires_grad_() for t in (q, k, v))
        comm_stats(reset=True)
        o = attention(ql, kl, vl, True, None)
        o.backward(loc(d_o))
        st = comm_stats()
        assert st["fwd_send"] > 0 and st["bwd_recv"] > 0
        tr = lambda t: t.transpose(1, 2)
        o_ref, _, dq, dk, dv = P.dense_attention_with_grads(tr(q), tr(k), tr(v), tr(d_o), P.causal(1))
        ret[rank] = max((o - loc(tr(o_ref))).abs().max().item(), (ql.grad - loc(tr(dq))).abs().max().item(),
                        (kl.grad - loc(tr(dk))).abs().max().item(), (vl.grad - loc(tr(dv))).abs().max().item())
        AC.destroy_sequence_parallel()
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_lightseq_attention_world4():
    port = 29100 + os.getpid() % 90
    ret = mp.Manager().dict()
    mp.spawn(_lightseq_worker, args=(4, port, ret), nprocs=4, join=True)
    for r in range(4):
        assert isinstance(ret[r], float), ret[r]
        assert ret[r] < 2e-4, (r, ret[r])


def _ref_names_worker(rank, world, port, ret):
    """The strategies through the reference's module paths, function names and argument lists."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ultraattn_b200 import parallel as PL, patterns as P
        from ring_flash_attn.ring_flash_attn import ring_flash_attn_backward, ring_flash_attn_forward
        from ring_flash_attn.zigzag_ring_flash_attn import ZigZagRingFlashAttnFunc
        from ring_flash_attn.stripe_flash_attn import StripeFlashAttnFunc
        from ring_flash_attn.ring_flash_attn_varlen import RingFlashAttnVarlenFunc
        from head_parallel_attn.deepspeed_ulysses_attn import DeepSpeedUlyssesAttnFunc
        from hierarchy_attn.hierarchy_attn_impl import HierarchyAttnFunc
        from hierarchy_attn.utils import InterComm, IntraComm
        S, H, D = 256, 4, 16
        g = torch.Generator().manual_seed(0)
        q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
        out = {}
        o_ref, _, dq, dk, dv = P.dense_attention_with_grads(q, k, v, d_o, P.causal(1))

        def err(kind, o, grads):
            sh = lambda t: PL.shard_sequence(t, rank, world, kind)
            return max([(o - sh(o_ref)).abs().max().item()] +
                       [(a - sh(b)).abs().max().item() for a, b in zip(grads, (dq, dk, dv))])

        # kernel-level pair: positional arguments as in the reference
        sh = lambda t: PL.shard_sequence(t, rank, world, "ring")
        o, lse = ring_flash_attn_forward(None, sh(q), sh(k), sh(v), D ** -0.5, 0, True)
        out["ring fwd/bwd"] = err("ring", o, ring_flash_attn_backward(None, sh(d_o), sh(q), sh(k), sh(v), o, lse,
                                                                    D ** -0.5, 0, True))
        # autograd classes: apply(q, k, v, dropout_p, scale, causal, window, alibi, deterministic, return_softmax, group, ...)
        for kind, cls, extra in (("zigzag", ZigZagRingFlashAttnFunc, (None, None, False)),
                                 ("stripe", StripeFlashAttnFunc, (None,)),
                                 ("ulysses", DeepSpeedUlyssesAttnFunc, (None,))):
            sh = lambda t, kind=kind: PL.shard_sequence(t, rank, world, kind)
            ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
            res = cls.apply(ql, kl, vl, 0.0, None, True, (-1, -1), None, False, kind == "stripe", *extra)
            o = res[0] if isinstance(res, tuple) else res
            o.backward(sh(d_o))
            out[cls.__name__] = err(kind, o, (ql.grad, kl.grad, vl.grad))
        # two-level class on a 2 x 2 arrangement (queries visit the other node)
        groups = PL.create_hierarchy_groups(tasks_per_node=2)
        sh = lambda t: PL.shard_sequence(t, rank, world, "zigzag")
        ql, kl, vl = (sh(t).requires_grad_() for t in (q, k, v))
        o = HierarchyAttnFunc.apply(ql, kl, vl, 0.0, None, True, (-1, -1), None, False, False, groups, None, True)
        o.backward(sh(d_o))
        out["HierarchyAttnFunc"] = err("zigzag", o, (ql.grad, kl.grad, vl.grad))
        # packed batch through the varlen class
        full_cu = [0, 96, 256]
        tq, tk, tv, tdo = (torch.randn(full_cu[-1], H, D, generator=g) for _ in range(4))
        ref = _dense_packed(tq, tk, tv, tdo, full_cu, True)
        shp = lambda t: PL.shard_packed(t, full_cu, rank, world, "ring")[0]
        local_cu = PL.shard_packed(tq, full_cu, rank, world, "ring")[1]
        ql, kl, vl = (shp(t).requires_grad_() for t in (tq, tk, tv))
        o = RingFlashAttnVarlenFunc.apply(ql, kl, vl, torch.tensor(local_cu),
                                          max(b - a for a, b in zip(local_cu, local_cu[1:])), 0.0, None, True,
                                          (-1, -1), None, False, False, None)
        o.backward(shp(tdo))
        out["RingFlashAttnVarlenFunc"] = max((a - shp(b)).abs().max().item()
                                             for a, b in zip((o, ql.grad, kl.grad, vl.grad), ref))
        # communicator classes of hierarchy_attn.utils: one ring shift, one query visit
        ring = IntraComm(groups)
        t = torch.full((4,), float(rank))
        got = ring.send_recv(t)
        ring.commit(); ring.wait()
        inter = InterComm(groups)
        visitor = inter.send_recv_q(0, t)
        inter.commit(); inter.wait()
        node, local = rank // 2, rank % 2
        ok_ring = got[0].item() == node * 2 + (local - 1) % 2
        ok_inter = (visitor is None) if node == 1 else visitor[0].item() == rank + 2    # node 1 sends to node 0
        out["comm classes"] = 0.0 if (ok_ring and ok_inter) else 1.0
        ret[rank] = out
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def test_reference_module_paths_and_argument_lists_world4():
    ret = mp.Manager().dict()
    mp.spawn(_ref_names_worker, args=(4, 29900 + os.getpid() % 90, ret), nprocs=4, join=True)
    _check(ret, 4)
