"""Static checks of the fused path's tables, over all ranks at once.

The fused kernels synchronise through memory: staging copies raise per-block flag counters that
compute tiles wait on, partial outputs land in mailbox slots of the owning rank, gradients are
added into accumulators. A wrong table does not fail loudly on the device: a slot written twice
gives a plausible but wrong sum, a wait on a counter nobody raises runs into its time limit. This
module proves, on the host and before anything is launched, that

  * every non-empty tile of the allocation is computed by exactly one forward row and one
    backward column, on the rank the allocation names;
  * every mailbox slot has exactly one writer per call (one flag epoch), lies inside the mailbox,
    and is exactly what its owner merges; no slot that is merged is left unwritten;
  * every wait names a flag that this rank's own staging list raises, with the number of copy
    chunks it will reach; every foreign input is either waited for or comes from the broadcast
    buffer; no two staging pieces write overlapping bytes of a mirror;
  * the backward adds dK/dV of a block into its owner's accumulator at the block's position.

Reference: the only check of this kind in the reference is ``sanity_check_stream_exclusive`` on
the stream schedule (search_algo/execute_plan.py:467-480); it has no memory-level plan to check.
Works on the objects the ranks build themselves, so the test can run every rank of a job in one
process (``FakeSpace``) and a job can run it once at start-up on gathered tables.
"""
from __future__ import annotations

from typing import Sequence


def _overlaps(spans) -> bool:
    spans = sorted(spans)
    return any(a[1] > b[0] for a, b in zip(spans, spans[1:]))


def verify_fused_tables(ranks: Sequence) -> list:
    """``ranks``: the ``FusedContextParallel`` object of every rank, built (``build()`` done), in
    rank order. Returns a list of problems (empty = fine)."""
    problems = []
    r0 = ranks[0]
    par_d, blk, world = r0.par_d, r0.blk, r0.world
    inv = lambda d: {v: k for k, v in d.items()}
    fwd_tiles, bwd_tiles = {}, {}
    writers = {}                        # (owner, slot index) -> [writer ranks]
    for g, rk in enumerate(ranks):
        q_of, kv_of, out_of = inv(rk.f_q_src), inv(rk.f_kv_src), inv(rk.f_out_slot)
        bc_block = inv(rk.bc_slot)
        f_counts = {}
        for flag, _, _ in rk.f_pieces:
            f_counts[flag] = f_counts.get(flag, 0) + 1
        if rk.cuda:
            _, f_counts = rk._device_tasks(rk.f_pieces)
        for kind, pieces in (("forward", rk.f_pieces), ("backward", rk.b_pieces_full)):
            spans = [(dst.data_ptr(), dst.data_ptr() + dst.numel() * dst.element_size()) for _, _, dst in pieces]
            if _overlaps(spans):
                problems.append(f"rank {g}: two {kind} staging pieces write overlapping bytes")
        # ---- forward rows
        for row in rk.f_rows:
            p = q_of[row.q_src]
            r = (rk.owned[p] if p == g else rk.mir_rows[p])[row.q_start // blk]
            if p != g:
                if row.q_wait_flag != r + 1 or row.q_wait_count != f_counts.get(r, -1):
                    problems.append(f"rank {g}: row {r} of rank {p} is read without a matching wait")
                if out_of[row.o_slot] != p:
                    problems.append(f"rank {g}: row {r} is written to the mailbox of the wrong rank")
                slot = row.o_start // blk
                if row.o_start % blk or slot >= len(rk.slots[p]) or rk.slots[p][slot] != (r, g):
                    problems.append(f"rank {g}: row {r} goes to mailbox slot {slot} of rank {p}, which is not its slot")
                writers.setdefault((p, slot), []).append(g)
            elif row.q_wait_flag or row.o_start != rk.lidx[r] * blk or out_of[row.o_slot] != g:
                problems.append(f"rank {g}: own row {r} has a wait or a foreign destination")
            for s in row.segs:
                src = kv_of[s.src]
                if src == "bc":
                    c = bc_block[s.start // blk]
                    if s.wait_flag:
                        problems.append(f"rank {g}: broadcast block {c} must not be waited for")
                else:
                    c = (rk.owned[src] if src == g else rk.mir_cols[src])[s.start // blk]
                    if src != g and (s.wait_flag != par_d + c + 1 or s.wait_count != f_counts.get(par_d + c, -1)):
                        problems.append(f"rank {g}: key block {c} of rank {src} is read without a matching wait")
                    if src == g and s.wait_flag:
                        problems.append(f"rank {g}: own key block {c} has a wait")
                fwd_tiles.setdefault((r, c), []).append(g)
        # ---- backward columns (both variants: mirrors reused from the forward, or staged anew)
        bq_of, bkv_of = inv(rk.b_q_src), inv(rk.b_kv_src)
        for variant, plan in enumerate(rk.b_plans):
            cnt = rk.b_counts[variant]
            if rk.cuda:
                _, cnt = rk._device_tasks(rk.b_pieces if variant == 0 else rk.b_pieces_full)
            for col in plan.cols:
                src = bkv_of[col.kv_src]
                owner = bkv_of[col.g_slot]
                c = bc_block[col.kv_start // blk] if src == "bc" else \
                    (rk.owned[src] if src == g else rk.mir_cols[src])[col.kv_start // blk]
                if owner == "bcg":          # in-switch reduction: own replica, at the block's broadcast slot
                    if c not in rk.bc_slot or col.g_start != rk.bc_slot[c] * blk:
                        problems.append(f"rank {g}: dK/dV of block {c} go to reduction slot {col.g_start // blk}")
                elif owner != int(rk.cmap[c]) or col.g_start != rk.lidx[c] * blk:
                    problems.append(f"rank {g}: dK/dV of block {c} go to rank {owner} at {col.g_start}")
                elif rk.nvls_reduce and c in rk.bc_slot:
                    problems.append(f"rank {g}: dK/dV of broadcast block {c} bypass the reduction buffer")
                staged_kv = cnt.get(par_d + c, 0)
                if src not in ("bc", g) and staged_kv and (col.kv_wait_flag != par_d + c + 1 or col.kv_wait_count != staged_kv):
                    problems.append(f"rank {g}: backward key block {c} is read without a matching wait")
                for s in col.segs:
                    p = bq_of[s.src]
                    r = (rk.owned[p] if p == g else rk.mir_rows[p])[s.start // blk]
                    if p != g and (s.wait_flag != r + 1 or s.wait_count != cnt.get(r, -1)):
                        problems.append(f"rank {g}: backward row {r} of rank {p} is read without a matching wait")
                    if variant == 0:
                        bwd_tiles.setdefault((r, c), []).append(g)
    # ---- tiles: exactly once, on the allocated rank
    for r in range(par_d):
        for c in range(par_d):
            want = int(r0.table[r, c])
            for name, got in (("forward", fwd_tiles.get((r, c), [])), ("backward", bwd_tiles.get((r, c), []))):
                if want < 0 and got:
                    problems.append(f"{name}: empty tile ({r}, {c}) is computed by {got}")
                elif want >= 0 and got != [want]:
                    problems.append(f"{name}: tile ({r}, {c}) belongs to rank {want}, computed by {got}")
    # ---- mailbox slots: one writer each, all inside the mailbox, merged iff written
    for (p, slot), ws in sorted(writers.items()):
        if len(ws) != 1:
            problems.append(f"mailbox slot {slot} of rank {p} has {len(ws)} writers per call: {ws}")
        if slot >= ranks[p].max_slots:
            problems.append(f"mailbox slot {slot} of rank {p} lies outside its mailbox")
    for p, rk in enumerate(ranks):
        merged = sorted(s for _, _, slots in rk.f_merge for s in slots)
        written = sorted(slot for (owner, slot) in writers if owner == p)
        if merged != written:
            problems.append(f"rank {p} merges mailbox slots {merged} but slots {written} are written")
    return problems
