"""Host-side logic of the fused context-parallel path with all ranks simulated in one process.

Peer memory is replaced by ordinary tensors that every simulated rank can see, the in-kernel
staging by host copies, and the kernels by their fp32 restatements; what is checked is everything
the host decides: which blocks are staged where, mailbox slots, source tables, merge lists and the
gradient accumulation through "peer" accumulators."""
import numpy as np
import pytest
import torch

from ultraattn_b200 import patterns as P
from ultraattn_b200.runtime import FakeSpace, FusedContextParallel, plan_allocation


def _run_all_ranks(pattern, world, S, H, D, allocation, seed=0, multicast=False, min_consumers=2,
                   nvls_reduce=False, steps=1, cmap=None):
    table, cmap = plan_allocation(pattern, world, 1, allocation, time_limit=5.0, cmap=cmap)
    if allocation == "lightseq":
        tiles = [int((table == r).sum()) for r in range(world)]
        assert max(tiles) - min(tiles) <= 1, tiles          # the point of the schedule: balance
    registry = {}
    ranks = [FusedContextParallel(table, cmap, pattern, S, H, D, FakeSpace(r, world, registry, multicast=multicast),
                                  dtype=torch.float32, defer_build=True, nvls_min_consumers=min_consumers,
                                  nvls_reduce=nvls_reduce)
             for r in range(world)]
    if multicast:
        assert ranks[0].bc_cols, "the pattern was chosen to have one-to-many blocks"
    for rk in ranks:
        rk.build()
    if nvls_reduce:
        from ultraattn_b200.runtime.verify import verify_fused_tables
        assert all(rk.nvls_reduce for rk in ranks) and verify_fused_tables(ranks) == []
        # the owners' dK/dV of broadcast blocks no longer arrive as per-consumer reductions
        assert sum(rk.traffic["bwd_reduce_in_bytes"] for rk in ranks) > 0
    worst = 0.0
    for step in range(steps):
        worst = max(worst, _one_step(ranks, pattern, world, S, H, D, seed + step))
    return worst, table


def _one_step(ranks, pattern, world, S, H, D, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
    blk = S // ranks[0].par_d
    idx = [torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in rk.owned[rk.rank]]) for rk in ranks]
    shard = lambda t, r: t[:, idx[r]].contiguous()
    # forward, phase by phase in lock step (a barrier separates the phases on real hardware)
    for r, rk in enumerate(ranks):
        if rk.debug_poison:
            rk._poison(("q", "k", "v", "do", "lse", "dvec"))
        rk.fwd_prepare(shard(q, r), shard(k, r), shard(v, r))
    outs = []
    for rk in ranks:
        rk.stage_on_host(rk.f_pieces)
        outs.append(rk.fwd_compute())
    for rk, (o, lse) in zip(ranks, outs):
        rk.fwd_finish(o, lse)
    # backward
    for r, rk in enumerate(ranks):
        rk.bwd_prepare(shard(d_o, r), shard(q, r), shard(k, r), shard(v, r), outs[r][0], outs[r][1], True)
    for rk in ranks:
        rk.stage_on_host(rk.b_pieces)
        rk.bwd_compute(True)
    grads = [rk.bwd_finish() for rk in ranks]
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q, k, v, d_o, pattern)
    worst = 0.0
    for r in range(world):
        worst = max(worst,
                    (outs[r][0] - o_ref[:, idx[r]]).abs().max().item(),
                    (grads[r][0] - dq_ref[:, idx[r]]).abs().max().item(),
                    (grads[r][1] - dk_ref[:, idx[r]]).abs().max().item(),
                    (grads[r][2] - dv_ref[:, idx[r]]).abs().max().item())
        fin = torch.isfinite(lse_ref[:, :, idx[r]])
        worst = max(worst, (outs[r][1][fin] - lse_ref[:, :, idx[r]][fin]).abs().max().item())
    return worst


@pytest.mark.parametrize("name,pattern,world,alloc", [
    ("causal-ilp", lambda: P.causal(1), 4, "ilp"),
    ("causal-naive", lambda: P.causal(1), 4, "naive"),
    ("strided-ilp", lambda: P.strided(8, 4, 2), 4, "ilp"),
    ("global-local-ilp", lambda: P.global_local(8, 1, 2), 2, "ilp"),
    ("star-naive", lambda: P.star(4, 1), 2, "naive"),
    ("full-ilp", lambda: P.full(1), 4, "ilp"),
    ("documents-ilp", lambda: P.document([2, 1, 3, 2]), 4, "ilp"),
    ("causal-lightseq-4", lambda: P.causal(1), 4, "lightseq"),
    ("causal-lightseq-8", lambda: P.causal(1), 8, "lightseq"),
], ids=lambda x: x if isinstance(x, str) else None)
def test_fused_host_logic(name, pattern, world, alloc):
    err, table = _run_all_ranks(pattern(), world, 512, 2, 16, alloc)
    assert err < 2e-4, (err, table)


@pytest.mark.parametrize("name,pattern,world,alloc,minc", [
    ("global-local-4", lambda: P.global_local(8, 1, 2), 4, "ilp", 2),
    ("star-4", lambda: P.star(8, 1), 4, "naive", 2),
    ("causal-2-forced", lambda: P.causal(1), 2, "naive", 1),
], ids=lambda x: x if isinstance(x, str) else None)
def test_fused_host_logic_with_multicast_blocks(name, pattern, world, alloc, minc):
    """Blocks that several ranks need are broadcast by their owner (emulated multicast store)
    instead of being pulled by every consumer; results must not change."""
    err, table = _run_all_ranks(pattern(), world, 512, 2, 16, alloc, multicast=True, min_consumers=minc)
    assert err < 2e-4, (err, table)


@pytest.mark.parametrize("name,pattern,world,alloc,minc", [
    ("global-local-4", lambda: P.global_local(8, 1, 2), 4, "ilp", 2),
    ("star-4", lambda: P.star(8, 1), 4, "naive", 2),
    ("causal-2-forced", lambda: P.causal(1), 2, "naive", 1),
], ids=lambda x: x if isinstance(x, str) else None)
def test_fused_host_logic_with_in_switch_gradient_sum(name, pattern, world, alloc, minc):
    """dK/dV of broadcast blocks: every rank adds into its own replica of the reduction buffer and
    the owner takes the sum over replicas (emulated multimem.ld_reduce). Two steps, so that stale
    contents of the replicas would show."""
    err, table = _run_all_ranks(pattern(), world, 512, 2, 16, alloc, multicast=True, min_consumers=minc,
                                nvls_reduce=True, steps=2)
    assert err < 2e-4, (err, table)


@pytest.mark.parametrize("name,pattern", [("strided", lambda: P.strided(8, 4, 2)), ("causal", lambda: P.causal(1))],
                         ids=lambda x: x if isinstance(x, str) else None)
def test_fused_host_logic_with_searched_ownership(name, pattern):
    """Context remap chosen by the planner (residue classes for the strided pattern, zigzag for
    dense causal): ranks own non-adjacent blocks; results must not change."""
    err, table = _run_all_ranks(pattern(), 4, 512, 2, 16, "ilp", cmap="search")
    assert err < 2e-4, (err, table)


def test_traffic_accounting_causal_two_ranks():
    """Dense causal on two ranks, one block each, row-owner allocation: rank 1 computes tile (1, 0)
    and pulls K/V of block 0; its dK/dV for that block go back; rank 0 moves nothing itself."""
    pat = P.causal(1)
    table = np.array([[0, -1], [1, 1]])
    cmap = np.array([0, 1])
    S, H, D = 256, 2, 16
    registry = {}
    ranks = [FusedContextParallel(table, cmap, pat, S, H, D, FakeSpace(r, 2, registry), dtype=torch.float32,
                                  defer_build=True) for r in range(2)]
    for rk in ranks:
        rk.build()
    blk_elems = (S // 2) * H * D
    t0, t1 = ranks[0].traffic, ranks[1].traffic
    assert all(v == 0 for v in t0.values()), t0
    assert t1["fwd_pull_bytes"] == 2 * blk_elems * 4            # K and V of block 0 (fp32 in this test)
    assert t1["fwd_push_bytes"] == 0 and t1["bwd_pull_bytes"] == 0
    assert t1["bwd_push_bytes"] == 2 * blk_elems * 4            # dK and dV partials (fp32)
    assert ranks[1].metrics()["phases_ms"] == {}


def test_poisoned_mirrors_are_fully_overwritten(monkeypatch):
    """With UA_DEBUG_POISON=1 every staging mirror starts as NaN: a correct result proves that the
    staging lists deliver every block a tile reads."""
    monkeypatch.setenv("UA_DEBUG_POISON", "1")
    err, table = _run_all_ranks(P.strided(8, 4, 2), 4, 512, 2, 16, "ilp")
    assert err < 2e-4, (err, table)


def _build_ranks(pattern, world, S=1024, H=2, D=16, allocation="ilp", multicast=False, min_consumers=2):
    table, cmap = plan_allocation(pattern, world, 1, allocation, time_limit=5.0)
    registry = {}
    ranks = [FusedContextParallel(table, cmap, pattern, S, H, D, FakeSpace(r, world, registry, multicast=multicast),
                                  dtype=torch.float32, defer_build=True, nvls_min_consumers=min_consumers)
             for r in range(world)]
    for rk in ranks:
        rk.build()
    return ranks


@pytest.mark.parametrize("name,world,multicast", [("strided", 4, False), ("global_local", 4, True), ("causal", 2, False)])
def test_static_verifier_accepts_the_tables_and_catches_damage(name, world, multicast):
    """The memory-level plan check: the tables every rank builds pass; a doubled mailbox writer, a
    dropped wait and a tile moved to another rank are each reported."""
    import dataclasses
    from ultraattn_b200.runtime.verify import verify_fused_tables
    pattern = {"strided": P.strided(8, 4, 2), "global_local": P.global_local(8, 1, 2), "causal": P.causal(1)}[name]
    ranks = _build_ranks(pattern, world, allocation="naive" if multicast else "ilp", multicast=multicast,
                         min_consumers=1 if multicast else 2)
    assert verify_fused_tables(ranks) == []
    # 1. a foreign row written into somebody else's slot
    victim = next((rk for rk in ranks if any(r.o_slot != 0 for r in rk.f_rows)), None)
    if victim is not None:
        i = next(i for i, r in enumerate(victim.f_rows) if r.o_slot != 0)
        good = victim.f_rows[i]
        victim.f_rows[i] = dataclasses.replace(good, o_start=good.o_start + victim.blk)
        assert any("mailbox" in p for p in verify_fused_tables(ranks))
        victim.f_rows[i] = good
    # 2. a remote key block read without waiting for its staging flag
    victim = next((rk for rk in ranks if any(s.wait_flag for r in rk.f_rows for s in r.segs)), None)
    if victim is not None:
        i = next(i for i, r in enumerate(victim.f_rows) if any(s.wait_flag for s in r.segs))
        good = victim.f_rows[i]
        segs = tuple(dataclasses.replace(s, wait_flag=0, wait_count=0) for s in good.segs)
        victim.f_rows[i] = dataclasses.replace(good, segs=segs)
        assert any("without a matching wait" in p for p in verify_fused_tables(ranks))
        victim.f_rows[i] = good
    # 3. a tile dropped from one rank's work list
    rk = ranks[-1]
    good = rk.f_rows[-1]
    rk.f_rows[-1] = dataclasses.replace(good, segs=good.segs[:-1])
    assert any("computed by []" in p for p in verify_fused_tables(ranks))
    rk.f_rows[-1] = good
    assert verify_fused_tables(ranks) == []


def test_fused_host_logic_on_random_patterns_property():
    """Property test: random causal-type block tables and rank counts through the fused path's host
    logic (all ranks in one process): the tables pass the static verifier and forward + backward
    match dense attention."""
    from hypothesis import given, settings, strategies as st
    from ultraattn_b200.patterns.blocks import BSA_Repr
    from ultraattn_b200.runtime.verify import verify_fused_tables

    @st.composite
    def causal_tables(draw):
        n = draw(st.sampled_from([4, 8]))
        t = np.zeros((n, n), dtype=np.int8)
        for i in range(n):
            t[i, i] = 2
            for j in range(i):
                t[i, j] = draw(st.sampled_from([0, 1]))
        return t

    @settings(max_examples=8, deadline=None, derandomize=True)
    @given(causal_tables(), st.sampled_from([2, 4]), st.booleans())
    def check(table, world, multicast):
        pat = BSA_Repr(table)
        ranks = _build_ranks(pat, world, S=256, H=1, D=8, allocation="ilp", multicast=multicast)
        assert verify_fused_tables(ranks) == []
        err = _one_step(ranks, pat, world, 256, 1, 8, seed=3)
        assert err < 2e-4, (table.tolist(), world, err)

    check()


def _lock_step(gens):
    """Drive one generator per simulated rank to completion, all of them one barrier at a time."""
    done = [None] * len(gens)
    live = list(range(len(gens)))
    while live:
        channels = set()
        for r in list(live):
            try:
                channels.add(next(gens[r]))
            except StopIteration as fin:
                done[r] = fin.value
                live.remove(r)
        assert len(channels) <= 1, f"ranks met at different barriers: {channels}"
    return done


def test_backward_restages_when_another_forward_ran_in_between():
    """fwd(A); fwd(B); bwd(A); bwd(B): the mirrors hold B's inputs when A's backward runs, so A's
    backward must restage Q / K / V instead of reusing what "the last forward" left there. Only a
    backward that directly follows its own forward may skip the restaging."""
    pattern, world, S, H, D = P.strided(8, 4, 2), 4, 512, 2, 16
    table, cmap = plan_allocation(pattern, world, 1, "ilp", time_limit=5.0)
    registry = {}
    ranks = [FusedContextParallel(table, cmap, pattern, S, H, D, FakeSpace(r, world, registry),
                                  dtype=torch.float32, defer_build=True) for r in range(world)]
    for rk in ranks:
        rk.build()
    assert any(rk.remote_cols or rk.remote_rows for rk in ranks)
    blk = S // ranks[0].par_d
    idx = [torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in rk.owned[rk.rank]]) for rk in ranks]
    shard = lambda t, r: t[:, idx[r]].contiguous()
    data, outs = {}, {}
    for name, seed in (("A", 11), ("B", 12)):
        g = torch.Generator().manual_seed(seed)
        data[name] = tuple(torch.randn(1, S, H, D, generator=g) for _ in range(4))
        q, k, v, _ = data[name]
        outs[name] = _lock_step([rk.forward_steps(shard(q, r), shard(k, r), shard(v, r)) for r, rk in enumerate(ranks)])
    assert all(rk.staged_inputs_match(outs["B"][r][0]) for r, rk in enumerate(ranks))
    assert not any(rk.staged_inputs_match(outs["A"][r][0]) for r, rk in enumerate(ranks))
    for name in ("A", "B"):
        q, k, v, d_o = data[name]
        grads = _lock_step([rk.backward_steps(shard(d_o, r), shard(q, r), shard(k, r), shard(v, r),
                                              outs[name][r][0], outs[name][r][1]) for r, rk in enumerate(ranks)])
        _, _, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q, k, v, d_o, pattern)
        for r in range(world):
            for got, ref in zip(grads[r], (dq_ref, dk_ref, dv_ref)):
                assert (got - ref[:, idx[r]]).abs().max().item() < 2e-4, (name, r)
    # the fast path still exists: a backward right after its own forward reuses the staged inputs
    q, k, v, d_o = data["A"]
    out = _lock_step([rk.forward_steps(shard(q, r), shard(k, r), shard(v, r)) for r, rk in enumerate(ranks)])
    assert all(rk.staged_inputs_match(out[r][0]) for r, rk in enumerate(ranks))


def test_debug_bounds_mode_checks_every_table_entry(monkeypatch):
    """UA_DEBUG_BOUNDS=1: every launch first checks its tables against the tensors it was given
    (the kernels are table driven, so this covers every address they form). A correct fused run
    passes; a table entry that points past a staging mirror is refused before anything runs."""
    from ultraattn_b200.ops import attention as A
    monkeypatch.setenv("UA_DEBUG_BOUNDS", "1")
    err, _ = _run_all_ranks(P.strided(8, 4, 2), 4, 512, 2, 16, "ilp")
    assert err < 2e-4
    q = torch.randn(1, 256, 2, 16)
    k = torch.randn(1, 128, 2, 16)
    o, lse = torch.zeros_like(q), torch.zeros(1, 2, 256)
    good = A.FwdPlan([A.Row(0, 0, 256, (A.Seg(0, 0, 128),), 0, 0, False)])
    A.attn_fwd([q], [k], [k], [(o, lse)], good)
    bad = A.FwdPlan([A.Row(0, 0, 256, (A.Seg(0, 64, 128),), 0, 0, False)])          # keys 64..191 of 128
    with pytest.raises(IndexError, match="exceed 128 tokens"):
        A.attn_fwd([q], [k], [k], [(o, lse)], bad)
    dq = torch.zeros(1, 256, 2, 16)
    side = A.BwdQSide(q, torch.randn_like(q), lse, torch.zeros_like(lse), dq)
    dk, dv = torch.zeros(1, 128, 2, 16), torch.zeros(1, 128, 2, 16)
    badc = A.BwdPlan([A.Col(0, 0, 128, (A.Seg(0, 192, 128),), 0, 0)])                 # queries 192..319 of 256
    with pytest.raises(IndexError, match="rows 192\\+128 exceed 256"):
        A.attn_bwd([side], [k], [k], [A.BwdKvOut(dk, dv)], badc)
