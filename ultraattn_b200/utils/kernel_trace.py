"""Summaries of the per-CTA time stamps the attention kernels record on request
(``ops.attention.enable_kernel_trace``).

The fused context-parallel kernels move their own data (staging copies by peer loads, partial
results by peer stores), so a profiler timeline shows one launch where the reference's runtime
shows separate NCCL kernels (NVTX ranges by kernel key, orchestrated_attn_impl.py:69,141). The
stamps give the attribution back: how long the SMs spent copying before computing, how busy each
SM was, how long the tail ran with few SMs busy."""
from __future__ import annotations

import numpy as np


def summarize(trace: np.ndarray, n_sms: int = 148) -> dict:
    """``trace``: int64 [n_ctas, 4] from ``read_kernel_trace``. Times in milliseconds."""
    if trace.size == 0:
        return {"ctas": 0}
    t0, t1, t2 = (trace[:, i].astype(np.float64) for i in range(3))
    sm = (trace[:, 3] >> 32).astype(np.int64)
    start, end = t0.min(), t2.max()
    span = (end - start) * 1e-6
    busy = np.zeros(int(sm.max()) + 1)
    np.add.at(busy, sm, (t2 - t0))
    staging = (t1 - t0)
    copying = staging[staging > 2000.0]                 # CTAs that took copy tasks (more than 2 us before computing)
    last_start = (t0.max() - start) * 1e-6
    # tail: time at the end of the launch during which fewer than half of the SMs still had work
    ends_per_sm = np.full(busy.shape[0], start)
    np.maximum.at(ends_per_sm, sm, t2)
    half_idle_from = np.sort(ends_per_sm)[len(ends_per_sm) // 2]
    return {
        "ctas": int(trace.shape[0]),
        "span_ms": round(span, 3),
        "sm_busy_fraction": round(float(busy.sum() / ((end - start) * max(len(busy), 1))), 4),
        "ctas_that_copied": int(copying.size),
        "staging_ms_longest_cta": round(float(staging.max()) * 1e-6, 3),
        "staging_sm_ms_total": round(float(copying.sum()) * 1e-6, 3),
        "staging_done_ms_after_start": round(float((t1[staging > 2000.0].max() - start) * 1e-6) if copying.size else 0.0, 3),
        "last_cta_start_ms": round(last_start, 3),
        "tail_ms_under_half_sms": round(float((end - half_idle_from) * 1e-6), 3),
        "longest_cta_ms": round(float((t2 - t0).max()) * 1e-6, 3),
    }
