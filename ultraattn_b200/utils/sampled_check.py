"""Check a block-sparse attention result on sampled rows against an fp32 oracle.

A dense oracle needs memory quadratic in the sequence length; at the benchmark shape (512k tokens)
that is out of reach, but any single query row only attends a few blocks and any single key row is
attended by a few blocks. So the check recomputes, in fp32 and from the raw inputs,

* O, lse and dQ of sampled *query rows* (softmax over exactly the keys the pattern allows), and
* dK, dV of sampled *key rows* (sum over the queries that attend them; this part uses the lse and
  D = rowsum(dO * O) of the run under test, whose O / lse are covered by the first part),

and reports, per quantity, the largest error relative to the largest reference magnitude and the
largest per-row relative error (||got - ref|| / ||ref||), which also sees a wrong row of small
magnitude. Inputs are fetched block by block through ``get_block(kind, block)`` so that a rank can
check rows whose keys live on other ranks (the benchmark regenerates them from their seeds).
"""
from __future__ import annotations

import math
from typing import Callable, Sequence

import numpy as np
import torch

from ..patterns.blocks import BSA_Repr, CAUSAL, EMPTY


def _row_errs(pairs) -> float:
    """Largest ||got - ref|| / ||ref|| over rows; a row whose reference is (nearly) zero, such as
    the first token of a causal sequence with dQ = 0, is measured against 1 % of the median norm."""
    if not pairs:
        return 0.0
    norms = torch.stack([r.norm() for _, r in pairs])
    floor = 0.01 * norms.median().clamp_min(1e-20)
    return max(float((g.float() - r).norm() / torch.maximum(r.norm(), floor)) for g, r in pairs)


class SampledCheck:
    """``pattern`` over ``seq_len`` tokens, ``get_block(kind, b)`` -> ``[blk, H, D]`` tensor of the
    global block ``b`` for kind in {"q", "k", "v", "do"}; ``lse_block(b)`` / ``dvec_block(b)`` ->
    ``[H, blk]`` fp32 of the run under test (only needed for :meth:`check_key_rows`)."""

    def __init__(self, pattern: BSA_Repr, seq_len: int, get_block: Callable[[str, int], torch.Tensor],
                 softmax_scale: float | None = None, head_dim: int = 128):
        self.types = np.asarray(pattern.block_table_int)
        self.n = self.types.shape[0]
        assert seq_len % self.n == 0
        self.blk = seq_len // self.n
        self.get = get_block
        self.scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(head_dim)

    # ---------------------------------------------------------------------------------------------
    def query_row(self, t: int):
        """Oracle (O [H, D], lse [H], dQ [H, D]) of global query token ``t``."""
        i, r = divmod(t, self.blk)
        q = self.get("q", i)[r].float()                     # [H, D]
        d_o = self.get("do", i)[r].float()
        cols = [j for j in range(self.n) if self.types[i, j] != EMPTY]
        scores, blocks = [], []
        for j in cols:
            k = self.get("k", j).float()                    # [blk, H, D]
            s = torch.einsum("hd,khd->hk", q, k) * self.scale
            if self.types[i, j] == CAUSAL:
                s[:, r + 1:] = float("-inf")
            scores.append(s)
            blocks.append(j)
            del k
        s_all = torch.cat(scores, dim=1)
        lse = torch.logsumexp(s_all, dim=1)                 # [H]
        o = torch.zeros_like(q)
        dq = torch.zeros_like(q)
        parts = []
        for j, s in zip(blocks, scores):
            p = torch.exp(s - lse[:, None])
            v = self.get("v", j).float()
            o += torch.einsum("hk,khd->hd", p, v)
            parts.append((j, p, torch.einsum("hd,khd->hk", d_o, v)))
            del v
        dvec = (d_o * o).sum(-1)                            # [H]
        for j, p, dp in parts:
            ds = p * (dp - dvec[:, None])
            dq += torch.einsum("hk,khd->hd", ds, self.get("k", j).float()) * self.scale
        return o, lse, dq

    def key_row(self, u: int, lse_block, dvec_block):
        """Oracle (dK [H, D], dV [H, D]) of global key token ``u`` (equal head counts)."""
        j, c = divmod(u, self.blk)
        k = self.get("k", j)[c].float()
        v = self.get("v", j)[c].float()
        dk = torch.zeros_like(k)
        dv = torch.zeros_like(v)
        for i in range(self.n):
            if self.types[i, j] == EMPTY:
                continue
            q = self.get("q", i).float()
            d_o = self.get("do", i).float()
            s = torch.einsum("qhd,hd->hq", q, k) * self.scale
            p = torch.exp(s - lse_block(i).float())
            if self.types[i, j] == CAUSAL:
                p[:, :c] = 0.0
            dv += torch.einsum("hq,qhd->hd", p, d_o)
            dp = torch.einsum("qhd,hd->hq", d_o, v)
            ds = p * (dp - dvec_block(i).float())
            dk += torch.einsum("hq,qhd->hd", ds, q) * self.scale
        return dk, dv

    # ---------------------------------------------------------------------------------------------
    def check_query_rows(self, rows: Sequence[int], fetch: Callable[[int], tuple]) -> dict:
        """``fetch(t)`` -> (O [H, D], lse [H], dQ [H, D] or None) of the run under test."""
        out = {"o": [0.0, 0.0], "lse": [0.0, 0.0], "dq": [0.0, 0.0]}
        refs = {"o": 0.0, "dq": 0.0}
        errs, pairs_o, pairs_dq = [], [], []
        for t in rows:
            o_ref, lse_ref, dq_ref = self.query_row(int(t))
            o, lse, dq = fetch(int(t))
            errs.append((o.float() - o_ref, o_ref, lse.float() - lse_ref, None if dq is None else dq.float() - dq_ref, dq_ref))
            refs["o"] = max(refs["o"], float(o_ref.abs().max()))
            refs["dq"] = max(refs["dq"], float(dq_ref.abs().max()))
            out["lse"][1] = max(out["lse"][1], float((lse.float() - lse_ref).abs().max()))
            pairs_o.append((o, o_ref))
            if dq is not None:
                pairs_dq.append((dq, dq_ref))
        out["o"][1], out["dq"][1] = _row_errs(pairs_o), _row_errs(pairs_dq)
        for eo, _, el, edq, _ in errs:
            out["o"][0] = max(out["o"][0], float(eo.abs().max()) / max(refs["o"], 1e-20))
            out["lse"][0] = max(out["lse"][0], float(el.abs().max()))
            if edq is not None:
                out["dq"][0] = max(out["dq"][0], float(edq.abs().max()) / max(refs["dq"], 1e-20))
        return {k: {"max_abs_over_max_ref": v[0], "max_row_relative": v[1]} for k, v in out.items()}

    def check_key_rows(self, rows: Sequence[int], fetch: Callable[[int], tuple], lse_block, dvec_block) -> dict:
        """``fetch(u)`` -> (dK [H, D], dV [H, D]) of the run under test."""
        got, ref = [], []
        for u in rows:
            ref.append(self.key_row(int(u), lse_block, dvec_block))
            got.append(fetch(int(u)))
        res = {}
        for idx, name in enumerate(("dk", "dv")):
            top = max(float(r[idx].abs().max()) for r in ref) if ref else 1.0
            res[name] = {
                "max_abs_over_max_ref": max((float((g[idx].float() - r[idx]).abs().max()) / max(top, 1e-20)
                                             for g, r in zip(got, ref)), default=0.0),
                "max_row_relative": _row_errs([(g[idx], r[idx]) for g, r in zip(got, ref)])}
        return res


def pick_rows(pattern: BSA_Repr, seq_len: int, owned_blocks: Sequence[int], n: int, seed: int = 0) -> list:
    """``n`` global token indices inside ``owned_blocks``: the first and last token of the first
    and last owned block (the last block is where element offsets are largest), one token on each
    side of a 128-row tile edge, the rest uniformly random."""
    blk = seq_len // pattern.block_table_int.shape[0]
    rng = np.random.default_rng(seed)
    first, last = owned_blocks[0], owned_blocks[-1]
    rows = {first * blk, first * blk + min(127, blk - 1), first * blk + min(128, blk - 1),
            last * blk, last * blk + blk - 1, last * blk + blk // 2}
    while len(rows) < n:
        b = int(rng.choice(list(owned_blocks)))
        rows.add(b * blk + int(rng.integers(0, blk)))
    return sorted(rows)
