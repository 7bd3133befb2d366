"""Command line + YAML configuration (reference: search_algo/arguments.py:18-67, configs/*.yaml).

YAML keys: ``Parallel.SP``, ``Shape.{Sq,Skv,Nhq,Nhkv,BS,D}``, ``Pattern.{pattern_type,
pattern_sparsity,local_blocks}``, ``Experiment.{transform_mode,lowering_mode}``; command-line flags
override the file.
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field
from typing import Optional

_args = None


@dataclass
class RunConfig:
    SP: tuple = (1, 8)
    Sq: int = 131072
    Skv: int = 131072
    Nhq: int = 32
    Nhkv: int = 32
    BS: int = 1
    D: int = 128
    pattern_type: str = "causal"
    pattern_sparsity: float = 0.125
    local_blocks: int = 2
    global_blocks: int = 1
    n_blocks: int = 32
    stride: int = 4
    transform_mode: str = "greedy"
    lowering_type: str = "Flexflow"
    exp_class: Optional[str] = None
    profiler_with_tensorboard: bool = False
    tb_dir: str = "./prof_results/tb"
    extra: dict = field(default_factory=dict)

    def pattern(self):
        from ..patterns import named
        t = self.pattern_type
        if t == "full":
            return named.full(1)
        if t == "causal":
            return named.causal(1)
        if t in ("stride", "strided"):
            return named.strided(self.n_blocks, self.stride, self.local_blocks)
        if t in ("star",):
            return named.star(self.n_blocks, self.global_blocks)
        if t in ("stream", "streaming"):
            return named.streaming(self.n_blocks, self.global_blocks, self.local_blocks)
        if t in ("local_global", "global_local", "lg"):
            return named.global_local(self.n_blocks, self.global_blocks, self.local_blocks)
        raise ValueError(f"unknown pattern_type {t!r}")


_YAML_MAP = {("Parallel", "SP"): "SP", ("Shape", "Sq"): "Sq", ("Shape", "Skv"): "Skv", ("Shape", "Nhq"): "Nhq",
             ("Shape", "Nhkv"): "Nhkv", ("Shape", "BS"): "BS", ("Shape", "D"): "D",
             ("Pattern", "pattern_type"): "pattern_type", ("Pattern", "pattern_sparsity"): "pattern_sparsity",
             ("Pattern", "local_blocks"): "local_blocks", ("Pattern", "global_blocks"): "global_blocks",
             ("Pattern", "n_blocks"): "n_blocks", ("Pattern", "stride"): "stride",
             ("Experiment", "transform_mode"): "transform_mode", ("Experiment", "lowering_mode"): "lowering_type"}


def load_yaml(path: str, cfg: Optional[RunConfig] = None) -> RunConfig:
    import yaml
    cfg = cfg or RunConfig()
    with open(path) as f:
        data = yaml.safe_load(f) or {}
    for (sec, key), attr in _YAML_MAP.items():
        if isinstance(data.get(sec), dict) and key in data[sec]:
            val = data[sec][key]
            if attr == "SP":
                val = tuple(val) if isinstance(val, (list, tuple)) else (1, int(val))
            setattr(cfg, attr, val)
    return cfg


def parse_args(argv=None) -> RunConfig:
    global _args
    ap = argparse.ArgumentParser(description="UltraAttn-style planning / profiling campaign")
    ap.add_argument("--config", type=str, default=None, help="YAML file (configs/*.yaml)")
    ap.add_argument("--exp-class", type=str, default=None, choices=["bsa_train", "dense_train", "bsa_infer"])
    ap.add_argument("--SP", type=int, nargs=2, default=None)
    for name, typ in (("Sq", int), ("Skv", int), ("Nhq", int), ("Nhkv", int), ("BS", int), ("D", int),
                      ("pattern_type", str), ("pattern_sparsity", float), ("transform_mode", str),
                      ("lowering_type", str)):
        ap.add_argument(f"--{name}", type=typ, default=None)
    ap.add_argument("--profiler-with-tensorboard", action="store_true")
    ap.add_argument("--tb-dir", type=str, default=None)
    ap.add_argument("--quick", action="store_true", help="small configuration space (smoke runs)")
    ns = ap.parse_args(argv)
    cfg = load_yaml(ns.config) if ns.config else RunConfig()
    for k, v in vars(ns).items():
        if v is None or k == "config":
            continue
        k = k.replace("-", "_")
        if k == "SP":
            v = tuple(v)
        if hasattr(cfg, k):
            setattr(cfg, k, v)
        else:
            cfg.extra[k] = v
    _args = cfg
    return cfg


def get_args() -> Optional[RunConfig]:
    return _args


# ---- the reference's helper names (search_algo/arguments.py:4-70) ------------------------------
def parse_parallel_args(parser) -> None:
    parser.add_argument("--SP", type=int, nargs="+", default=None, help="sequence-parallel degrees (intra, inter)")


def parse_shape_args(parser) -> None:
    for name, what in (("Sq", "query tokens"), ("Skv", "key/value tokens"), ("Nhq", "query heads"),
                       ("Nhkv", "key/value heads"), ("BS", "batch size"), ("D", "head dim")):
        parser.add_argument(f"--{name}", type=int, default=None, help=what)


def parse_pattern_args(parser) -> None:
    parser.add_argument("--pattern_type", type=str, default=None,
                        choices=[None, "causal", "full", "star", "stream", "stride", "global_local"])
    parser.add_argument("--pattern_sparsity", type=float, default=None)


def parse_experiment_args(parser) -> None:
    parser.add_argument("--transform_mode", type=str, default=None, choices=[None, "None", "Greedy", "greedy", "bf"])
    parser.add_argument("--lowering_type", type=str, default=None, choices=[None, "Flexflow", "ILP"])


def recursive_update(config, args) -> None:
    """Overwrite the leaves of a nested configuration dict with the command-line values of the
    same name that were given (not None)."""
    if not isinstance(config, dict):
        return
    for key, value in config.items():
        if isinstance(value, dict):
            recursive_update(value, args)
        elif getattr(args, key, None) is not None:
            config[key] = getattr(args, key)


def parse_config(argv=None) -> dict:
    """The YAML file named by ``--config`` as a nested dict, with command-line overrides applied."""
    import yaml
    ap = argparse.ArgumentParser(description="UltraAttn-style configuration")
    ap.add_argument("--config", type=str, required=True)
    for add in (parse_parallel_args, parse_shape_args, parse_pattern_args, parse_experiment_args):
        add(ap)
    ns = ap.parse_args(argv)
    with open(ns.config) as f:
        config = yaml.safe_load(f) or {}
    recursive_update(config, ns)
    return config


def print_args(args) -> None:
    """Print a parsed configuration on rank 0."""
    if int(getattr(args, "rank", 0) or 0) != 0:
        return
    print("------------------------ arguments ------------------------", flush=True)
    items = vars(args).items() if not isinstance(args, dict) else args.items()
    for k, v in sorted(items):
        print(f"  {k} {'.' * max(2, 48 - len(str(k)))} {v}", flush=True)
    print("-------------------- end of arguments ---------------------", flush=True)
