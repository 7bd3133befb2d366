"""Token-level masks on the block-sparse kernels: correctness against dense masked attention and
forward / forward + backward time per mask.

    python -m ultraattn_b200.drivers.bench_masks [--seq 32768] [--heads 16] [--masks causal,sliding_window,...]

The masks of the reference's mask benchmark (tests/flexattn_tests/flexattn.py:29-43, which times
torch FlexAttention on causal, sliding-window, prefix-LM and document masks as a candidate kernel
backend): here each is a launch plan of the same attention kernels — causal and document masks as
segment lists, prefix-LM as a fully visible prefix item plus a causal item with a shifted
diagonal, the sliding window as the two-part plan of ``ops/window.py``, and ``streaming`` (window
plus attention sinks, the token-exact form of the reference's block-level streaming pattern). Its
score modifications (ALiBi, soft-capping) change the scores themselves and are not available on
these kernels. Prints one JSON line per mask: density of the mask, max error against dense
attention (sequence lengths up to ``--check-limit``), milliseconds and achieved TFLOP/s counted on
the visible pairs only.
"""
from __future__ import annotations

import argparse
import json
import math
import time

import torch

from .. import api
from ..ops.window import sliding_window_attention


def _doc_bounds(seq: int, n_docs: int, seed: int = 0) -> list:
    """``n_docs`` random document lengths that add up to ``seq`` (each at least 1)."""
    g = torch.Generator().manual_seed(seed)
    cuts = sorted(set((torch.randperm(seq - 1, generator=g)[:n_docs - 1] + 1).tolist()))
    return [0] + cuts + [seq]


def build_masks(seq: int, window: int, prefix: int, n_docs: int, sinks: int = 4) -> dict:
    """name -> (callable(q, k, v) -> o with autograd, dense boolean mask builder)."""
    r = lambda: torch.arange(seq)[:, None]
    c = lambda: torch.arange(seq)[None, :]
    cu = _doc_bounds(seq, n_docs)

    def doc_mask():
        m = torch.zeros(seq, seq, dtype=torch.bool)
        for a, b in zip(cu[:-1], cu[1:]):
            m[a:b, a:b] = torch.ones(b - a, b - a, dtype=torch.bool).tril()
        return m

    return {
        "causal": (lambda q, k, v: api.varlen_attention(q, k, v, [0, seq], True), lambda: c() <= r()),
        "sliding_window": (lambda q, k, v: sliding_window_attention(q, k, v, (window - 1, 0), True),
                           lambda: (c() <= r()) & (c() > r() - window)),
        "streaming": (lambda q, k, v: sliding_window_attention(q, k, v, (window - 1, 0), True, sink_tokens=sinks),
                      lambda: (c() <= r()) & ((c() > r() - window) | (c() < sinks))),
        "prefix_lm": (lambda q, k, v: api.prefix_lm_attention(q, k, v, prefix), lambda: (c() <= r()) | (c() < prefix)),
        "document": (lambda q, k, v: api.varlen_attention(q, k, v, cu, True), doc_mask),
    }


def _dense(q, k, v, mask):
    g = q.shape[2] // k.shape[2]
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float().repeat_interleave(g, 2)) / math.sqrt(q.shape[-1])
    s = s.masked_fill(~mask.to(q.device), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float().repeat_interleave(g, 2))


def _time(fn, iters: int, device) -> float:
    """Milliseconds per call: CUDA events on the current stream, host clock on CPU."""
    fn()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / iters
    t = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t) * 1e3 / iters


def run(seq: int, heads: int, kv_heads: int, head_dim: int, masks, window: int, prefix: int, n_docs: int,
        iters: int, check_limit: int, device) -> list:
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    g = torch.Generator().manual_seed(0)
    mk = lambda h: torch.randn(1, seq, h, head_dim, generator=g).to(dtype).to(device).requires_grad_()
    q, k, v = mk(heads), mk(kv_heads), mk(kv_heads)
    d_o = torch.randn(1, seq, heads, head_dim, generator=g).to(dtype).to(device)
    out = []
    table = build_masks(seq, window, prefix, n_docs)
    for name in masks:
        fn, dense_mask = table[name]
        rec = {"mask": name, "seq": seq, "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim,
               "device": device.type, "dtype": str(dtype).split(".")[-1]}
        if seq <= check_limit:
            m = dense_mask()
            rec["density"] = m.float().mean().item()
            with torch.no_grad():
                err = (fn(q, k, v).float() - _dense(q, k, v, m)).abs().max().item()
            rec["max_err"] = err
            pairs = float(m.sum())
        else:
            pairs = None

        def fwd():
            with torch.no_grad():
                return fn(q, k, v)

        def fwd_bwd():
            o = fn(q, k, v)
            o.backward(d_o)
            q.grad = k.grad = v.grad = None

        rec["fwd_ms"] = _time(fwd, iters, device)
        rec["fwd_bwd_ms"] = _time(fwd_bwd, iters, device)
        if pairs is not None:
            flops = 4.0 * pairs * heads * head_dim              # QK^T and PV, 2 flops per multiply-add
            rec["fwd_tflops"] = flops / (rec["fwd_ms"] * 1e-3) / 1e12
            rec["fwd_bwd_tflops"] = 3.5 * flops / (rec["fwd_bwd_ms"] * 1e-3) / 1e12
        out.append(rec)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=32768)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=None)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--masks", default="causal,sliding_window,streaming,prefix_lm,document")
    ap.add_argument("--window", type=int, default=1024)
    ap.add_argument("--prefix", type=int, default=1024)
    ap.add_argument("--docs", type=int, default=12)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--check-limit", type=int, default=16384,
                    help="largest sequence for which the dense mask is built (density, error, TFLOP/s)")
    ap.add_argument("--device", default=None, choices=["cuda", "cpu"])
    a = ap.parse_args(argv)
    device = torch.device(a.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    for rec in run(a.seq, a.heads, a.kv_heads or a.heads, a.head_dim, a.masks.split(","), a.window, a.prefix, a.docs,
                   a.iters, a.check_limit, device):
        print(json.dumps(rec), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
