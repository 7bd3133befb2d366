"""JSON-lines metrics and the roofline arithmetic used in reports.

The reference logs with ``print`` and keeps its structured results only in the profile JSONs
(``hfu`` / ``time`` / ``sim_time``; search_algo/task1_bsa.py:352-356), and its plot scripts parse
``mfu: ... s/iter`` lines back out of the logs (search_algo/utils.py:274-363). Here every measured
call can be appended as one JSON object per line: time (max over ranks), TFLOP/s per GPU, bytes
moved over NVLink per direction, and the achieved fraction of the roofline, i.e. of the slower of
"FLOPs at the measured GEMM peak" and "NVLink bytes at the measured link bandwidth".
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Optional

# fall-backs when no measured-peaks file is available: earlier measurements on B200
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
NVLINK_GBS_PER_DIRECTION = 770.0        # measured peer copy, one direction, one GPU


def load_peaks(path: Optional[str] = None) -> dict:
    """Measured peaks (``bf16_tflops``, ``bf16_tflops_sustained``, ``hbm_gbs``) from a JSON file
    (default: ``MEASURED_PEAKS.json`` in the working directory or named by ``UA_MEASURED_PEAKS``),
    with ``source`` = "measured" or "fallback"."""
    cand = [path, os.environ.get("UA_MEASURED_PEAKS"), "MEASURED_PEAKS.json"]
    for c in cand:
        if c and Path(c).exists():
            d = json.loads(Path(c).read_text())
            out = {k: float(d[k]) for k in FALLBACK_PEAKS if k in d}
            if len(out) == len(FALLBACK_PEAKS):
                out["source"] = "measured"
                return out
    return dict(FALLBACK_PEAKS, source="fallback")


def roofline(flops_per_gpu: float, nvlink_bytes_per_gpu: float, seconds: float, peaks: Optional[dict] = None,
             sustained: bool = True, link_gbs: float = NVLINK_GBS_PER_DIRECTION) -> dict:
    """Target time = max(compute at peak, bytes over one NVLink direction at link bandwidth);
    ``fraction`` = target / measured. ``nvlink_bytes_per_gpu`` is the larger of the bytes a GPU
    receives and the bytes it sends."""
    peaks = peaks or load_peaks()
    peak = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    t_compute = flops_per_gpu / peak
    t_link = nvlink_bytes_per_gpu / (link_gbs * 1e9)
    target = max(t_compute, t_link)
    return {"t_compute_s": t_compute, "t_link_s": t_link, "bound": "compute" if t_compute >= t_link else "nvlink",
            "target_s": target, "fraction": target / seconds if seconds > 0 else 0.0,
            "tflops_per_gpu": flops_per_gpu / seconds / 1e12 if seconds > 0 else 0.0,
            "peaks": peaks.get("source", "given")}


class MetricsLogger:
    """Append-only JSON-lines file; one object per measured call."""

    def __init__(self, path: Optional[str] = None, **common):
        self.path = Path(path) if path else None
        self.common = common
        self.records: list = []
        if self.path:
            self.path.parent.mkdir(parents=True, exist_ok=True)

    def log(self, name: str, seconds: float, flops_per_gpu: float = 0.0, pull_bytes: int = 0,
            push_bytes: int = 0, **extra) -> dict:
        rec = {"ts": time.time(), "name": name, "ms": seconds * 1e3, **self.common, **extra}
        if flops_per_gpu:
            rec.update(roofline(flops_per_gpu, max(pull_bytes, push_bytes), seconds))
        rec["nvlink_pull_bytes"], rec["nvlink_push_bytes"] = int(pull_bytes), int(push_bytes)
        self.records.append(rec)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        return rec


def read_jsonl(path) -> list:
    return [json.loads(line) for line in Path(path).read_text().splitlines() if line.strip()]
