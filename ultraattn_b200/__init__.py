"""ultraattn_b200 — context-parallel block-sparse attention for B200 (sm_100a).

Layers: ``patterns`` (block tables, named patterns, dense oracle), ``planner`` (tile allocation
ILP, dependent kernel graph, kernel fusion, launch scheduling, cost model), ``plandb`` (plan /
profile database), ``runtime`` (plan executors: gloo CPU reference, NCCL baseline, fused sm_100a),
``parallel`` (process topology, ring / zigzag / stripe / Ulysses strategies), ``ops`` (kernel entry
points), ``models`` (Llama-style model built on the kernels).
"""
from . import patterns  # noqa: F401
from .api import attention, prefix_lm_attention, varlen_attention  # noqa: F401
from .ops.window import sliding_window_attention  # noqa: F401

__version__ = "0.1.0"
