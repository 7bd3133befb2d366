"""The sampled-row checker against the dense oracle (the checker is what validates the benchmark
shape, where a dense oracle does not fit in memory)."""
import pytest
import torch

from ultraattn_b200 import patterns as P
from ultraattn_b200.utils.sampled_check import SampledCheck, pick_rows


@pytest.mark.parametrize("pattern", [lambda: P.strided(8, 4, 2), lambda: P.global_local(8, 1, 2), lambda: P.causal(1)],
                         ids=["strided", "global-local", "causal"])
def test_sampled_rows_agree_with_dense_oracle(pattern):
    pat = pattern()
    S, H, D = 512, 2, 16
    g = torch.Generator().manual_seed(3)
    q, k, v, d_o = (torch.randn(1, S, H, D, generator=g) for _ in range(4))
    o, lse, dq, dk, dv = P.dense_attention_with_grads(q, k, v, d_o, pat)
    n = pat.block_table_int.shape[0]
    blk = S // n
    data = {"q": q, "k": k, "v": v, "do": d_o}
    chk = SampledCheck(pat, S, lambda kind, b: data[kind][0, b * blk:(b + 1) * blk], head_dim=D)
    rows = pick_rows(pat, S, list(range(n)), 24, seed=1)
    assert S - 1 in rows and 0 in rows
    res = chk.check_query_rows(rows, lambda t: (o[0, t], lse[0, :, t], dq[0, t]))
    assert all(v["max_row_relative"] < 1e-3 for v in res.values()), res
    dvec = (o * d_o).sum(-1).permute(0, 2, 1)            # [1, H, S]
    res = chk.check_key_rows(rows[:12], lambda u: (dk[0, u], dv[0, u]),
                             lambda b: lse[0, :, b * blk:(b + 1) * blk], lambda b: dvec[0, :, b * blk:(b + 1) * blk])
    assert all(v["max_row_relative"] < 1e-3 for v in res.values()), res
    # a wrong row of small magnitude is seen by the per-row figure
    bad = o.clone()
    bad[0, rows[3]] *= 1.5
    res = chk.check_query_rows(rows, lambda t: (bad[0, t], lse[0, :, t], dq[0, t]))
    assert res["o"]["max_row_relative"] > 0.4
