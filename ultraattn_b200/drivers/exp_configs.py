"""Experiment spaces of the planning / profiling campaign (reference: search_algo/exp_configs.py:69-695).

Three classes, selected with ``--exp-class``:
  * ``bsa_train``   strided and global+local patterns, forward and backward
  * ``dense_train`` full and causal attention, forward and backward
  * ``bsa_infer``   star and streaming prefill, forward only
Each yields global (inter-level) :class:`BSA_Config` objects, the distinct per-node (intra-level)
configs obtained by cutting them into ``CP_inter`` x ``CP_inter`` node tiles, and the shapes to
plan for. Defaults describe one 8-GPU NVSwitch box (``CP = (k, 1)``); ``max_nodes`` > 1 adds the
multi-node points of the reference's sweep.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..patterns import named
from ..patterns.blocks import BSA_Config
from ..utils.bsa_helpers import split_to_node_configs
from ..utils.misc import unique_list


@dataclass
class ExpSpace:
    exp_class: str
    fobs: list
    inter_bsa_configs: list
    intra_bsa_configs: list
    Ss: list                       # total sequence lengths
    Nhs: list
    bs: int = 1
    D: int = 128
    S_per_gpu_bounds: tuple = (256, 262144)
    plan_types: list = field(default_factory=lambda: ["Flexflow", "ILP"])

    def shape_configs(self, cp_total: int):
        lo, hi = self.S_per_gpu_bounds
        for S in self.Ss:
            if not (lo <= S // cp_total <= hi):
                continue
            for nh in self.Nhs:
                yield {"S": (S, S), "Nh": (nh, nh), "bs": self.bs, "D": self.D}


def _cps(max_intra: int, max_nodes: int):
    intra = [c for c in (2, 4, 8) if c <= max_intra]
    out = [(c, 1) for c in intra]
    n = 2
    while n <= max_nodes:
        out.append((max_intra, n))
        n *= 2
    return out


def _space(exp_class, fobs, reprs, Ss, Nhs, max_intra, max_nodes, quick):
    inter = [BSA_Config(None, None, {"bsa_repr": r, "CP": cp}) for r in reprs for cp in _cps(max_intra, max_nodes)]
    intra = []
    for c in inter:
        intra += split_to_node_configs(c)
    if quick:
        Ss, Nhs = Ss[:2], Nhs[:1]
    return ExpSpace(exp_class, fobs, inter, unique_list(intra), Ss, Nhs)


def get_bsa_train_configs(max_intra=8, max_nodes=1, quick=False) -> ExpSpace:
    reprs = [named.strided(32, 4, 2), named.global_local(32, 1, 2)]
    Ss = [1 << p for p in range(14, 22)]            # 16k .. 2M
    return _space("bsa_train", [0, 1], reprs, Ss, [1, 32], max_intra, max_nodes, quick)


def get_dense_train_configs(max_intra=8, max_nodes=1, quick=False) -> ExpSpace:
    reprs = [named.full(1), named.causal(1)]
    Ss = [1 << p for p in range(14, 22)]
    return _space("dense_train", [0, 1], reprs, Ss, [1, 32], max_intra, max_nodes, quick)


def get_bsa_infer_configs(max_intra=8, max_nodes=1, quick=False) -> ExpSpace:
    reprs = [named.star(32, 1), named.streaming(32, 1, 2)]
    Ss = [1 << p for p in range(14, 20)]            # 16k .. 512k
    return _space("bsa_infer", [0], reprs, Ss, [1, 32], max_intra, max_nodes, quick)


def get_exp_configs(fobs=(0,), plan_type: str = "manual", transform_mode: str = "greedy",
                    MAX_QUEUE_SIZE: int = 100) -> list:
    """One :class:`Evaluation_Configs` per pass (reference: search_algo/exp_configs.py:13-67; the
    hierarchy is set later, per experiment)."""
    from ..planner.cost import Evaluation_Configs
    return [Evaluation_Configs(plan_type, MAX_QUEUE_SIZE, fob, hierarchy=None, transform_mode=transform_mode)
            for fob in fobs]


def get_exp_train_configs(**kw) -> list:
    return get_exp_configs(fobs=(0, 1), **kw)


def get_exp_infer_configs(**kw) -> list:
    return get_exp_configs(fobs=(0,), **kw)


def step0_top_down_decompose(exp_class: str, max_intra: int = 8, max_nodes: int = 1, quick: bool = False) -> ExpSpace:
    fn = {"bsa_train": get_bsa_train_configs, "dense_train": get_dense_train_configs,
          "bsa_infer": get_bsa_infer_configs}.get(exp_class)
    if fn is None:
        raise ValueError(f"unknown --exp-class {exp_class!r}")
    return fn(max_intra, max_nodes, quick)
