"""Plan / profile database: the campaign's restartable, content-addressed store.

Directory layout and key grammar are those of the reference (search_algo/database.py:25-37,
search_algo/task1_bsa.py:101-102, 137-140, 178-179, 197-237, 296-300, 424-427, 656-661,
search_algo/bsa_utils.py:101-102), byte for byte, so that databases and plots are interchangeable:

    database/<CLUSTER_NAME>/<PLATFORM>/
        m_configs/time*.json  cb_8_*.log  cb_16_*.log        machine micro-profiles
        {intra,inter}_bsa_allocation.json                    key -> {"Par_D", "schedule_table"}
        {intra,inter}_bsa_exe_plans/<id>.pkl (+ <id>.json)   pickled plan + plain-data side-car
        {intra,inter}_bsa_exe_plans_kv.json                  key -> plan id (max + 1 allocation)
        {intra,inter}_bsa_exe_plans_profile.json             key -> {"hfu", "time", "sim_time"}

    prefix = fob={0|1}_CP={(intra, inter)}_shape_config={S=(Sq, Skv)_Nh=(Nh, Ng)_bs={bs}_D={D}}
             _bsa_config={CP=(intra, inter)_repr=[[row][row]...]}
    plan / profile key = prefix + one of ABLATION_SUFFIXES
    shape-free FULL plans: fob=.._CP=.._shape_config=full_ablation=(Y=..,X=..,dim=0)

What is new: every JSON update is written atomically (temp file + rename) so an interrupted
campaign never leaves a truncated file, and each pickle gets a ``<id>.json`` side-car holding the
same plan as plain lists, loadable without importing any class.
"""
from __future__ import annotations

import json
import os
import pickle
import shutil
import tempfile
from pathlib import Path
from typing import Optional

import numpy as np

from ..planner.cost import Machine_Config, convert_shape_config_to_str

ABLATION_SUFFIXES = [
    "_ablation=(w/o_gpu_tile,w/o_kernel_tile,Flexflow)",
    "_ablation=(w/o_kernel_tile,Flexflow)",
    "_ablation=(w_kernel_tile,Flexflow)",
    "_ablation=(w/o_kernel_tile,ILP)",
    "_ablation=(w_kernel_tile,ILP)",
]


def plan_key_prefix(fob: int, CP: tuple, shape_config: dict, bsa_config) -> str:
    return (f"fob={fob}_CP={tuple(CP)}_shape_config={{{convert_shape_config_to_str(shape_config)}}}"
            f"_bsa_config={{{bsa_config}}}")


def allocation_key(fob: int, bsa_config, gpu_tile_type: Optional[str] = None) -> str:
    return f"fob={fob}_bsa_config={{{bsa_config}}}" + ("" if gpu_tile_type is None else f"_{gpu_tile_type}")


def full_plan_key(fob: int, CP: tuple, Y: int, X: int, dim: int = 0) -> str:
    return f"fob={fob}_CP={tuple(CP)}_shape_config=full_ablation=(Y={Y},X={X},dim={dim})"


def full_profile_suffix(kernel_tile: bool, Y: int, X: int, dim: int = 0) -> str:
    return f"_ablation=({'w_kernel_tile' if kernel_tile else 'w/o_kernel_tile'},Y={Y},X={X},dim={dim})"


def _atomic_write_json(path: Path, obj) -> None:
    fd, tmp = tempfile.mkstemp(dir=str(path.parent), prefix=path.name, suffix=".tmp")
    with os.fdopen(fd, "w") as f:
        json.dump(obj, f)
    os.replace(tmp, path)


class Prof_DB:
    def __init__(self, CLUSTER_NAME: Optional[str] = None, PLATFORM: Optional[str] = None,
                 gloo_global_group=None, root: Optional[str] = None, raw_m_config_dir: str = "logs/m_configs"):
        self.CLUSTER_NAME = CLUSTER_NAME or os.environ.get("CLUSTER_NAME", "local")
        self.PLATFORM = PLATFORM or os.environ.get("PLATFORM", "B200")
        base = Path(root) if root is not None else Path(os.environ.get("UA_DATABASE_ROOT", "database"))
        self.DATABASE_ROOT = str(base / self.CLUSTER_NAME / self.PLATFORM)
        r = Path(self.DATABASE_ROOT)
        self.M_CONFIG_DIR = str(r / "m_configs")
        self.RAW_M_CONFIG_DIR = raw_m_config_dir
        for lvl in ("intra", "inter"):
            up = lvl.upper()
            setattr(self, f"{up}_BSA_ALLOCATION", str(r / f"{lvl}_bsa_allocation.json"))
            setattr(self, f"{up}_BSA_EXE_PLANS_DIR", str(r / f"{lvl}_bsa_exe_plans"))
            setattr(self, f"{up}_BSA_EXE_PLANS_KV", str(r / f"{lvl}_bsa_exe_plans_kv.json"))
            setattr(self, f"{up}_BSA_EXE_PLANS_PROFILE", str(r / f"{lvl}_bsa_exe_plans_profile.json"))
        import torch.distributed as dist
        if not dist.is_initialized() or dist.get_rank() == 0:
            r.mkdir(parents=True, exist_ok=True)
            mdir = Path(self.M_CONFIG_DIR)
            if not mdir.is_dir():
                if Path(self.RAW_M_CONFIG_DIR).is_dir():
                    shutil.copytree(self.RAW_M_CONFIG_DIR, mdir)
                else:
                    mdir.mkdir(parents=True)
            for lvl in ("INTRA", "INTER"):
                Path(getattr(self, f"{lvl}_BSA_EXE_PLANS_DIR")).mkdir(exist_ok=True)
                for kind in ("ALLOCATION", "EXE_PLANS_KV", "EXE_PLANS_PROFILE"):
                    p = Path(getattr(self, f"{lvl}_BSA_{kind}"))
                    if not p.exists():
                        _atomic_write_json(p, {})
        if dist.is_initialized():
            dist.barrier(gloo_global_group)
        self.m_config = self.create_m_config()

    # ------------------------------- machine config --------------------------------------------
    def create_m_config(self) -> Machine_Config:
        """Read ``time*.json`` / ``cb_8_*.log`` / ``cb_16_*.log`` if present; parts that are missing
        fall back to the analytic B200 model."""
        mdir = Path(self.M_CONFIG_DIR)
        if not any(mdir.glob("time*.json")) and not any(mdir.glob("cb_*.log")):
            return Machine_Config.b200_default()        # nothing profiled here: the packaged profile
        return Machine_Config.from_dir(mdir)

    def m_config_update_inter_bsa_profile(self) -> None:
        self.m_config.update_inter_bsa_profile(self._load(self.INTRA_BSA_EXE_PLANS_PROFILE))

    # ------------------------------- generic JSON KV --------------------------------------------
    @staticmethod
    def _load(path) -> dict:
        with open(path) as f:
            return json.load(f)

    def _lvl(self, hierarchy: int) -> str:
        return "INTRA" if hierarchy else "INTER"

    # allocations
    def get_allocation(self, key: str, hierarchy: int = 1):
        d = self._load(getattr(self, f"{self._lvl(hierarchy)}_BSA_ALLOCATION"))
        if key not in d:
            return None
        v = d[key]
        table = np.array(v["schedule_table"], dtype=np.int32)
        assert v["Par_D"] == table.shape[-1]
        return {"Par_D": v["Par_D"], "table": table}

    def put_allocation(self, key: str, table: np.ndarray, hierarchy: int = 1) -> None:
        path = Path(getattr(self, f"{self._lvl(hierarchy)}_BSA_ALLOCATION"))
        d = self._load(path)
        d[key] = {"Par_D": int(table.shape[-1]), "schedule_table": np.asarray(table).tolist()}
        _atomic_write_json(path, d)

    # plans
    def has_plan(self, key: str, hierarchy: int = 1) -> bool:
        return key in self._load(getattr(self, f"{self._lvl(hierarchy)}_BSA_EXE_PLANS_KV"))

    def put_plan(self, key: str, plan, hierarchy: int = 1) -> int:
        lvl = self._lvl(hierarchy)
        kv_path = Path(getattr(self, f"{lvl}_BSA_EXE_PLANS_KV"))
        kv = self._load(kv_path)
        pid = kv[key] if key in kv else (max(kv.values()) + 1 if kv else 0)
        d = Path(getattr(self, f"{lvl}_BSA_EXE_PLANS_DIR"))
        from ..planner import bind_reference_class_paths
        bind_reference_class_paths()        # pickles name the reference's module paths when possible
        with open(d / f"{pid}.pkl", "wb") as f:
            pickle.dump(plan, f)
        if hasattr(plan, "to_plain") and (getattr(plan, "d_graph", None) is not None or hasattr(plan, "Y")):
            _atomic_write_json(d / f"{pid}.json", plan.to_plain())
        kv[key] = pid
        _atomic_write_json(kv_path, kv)
        return pid

    def get_plan(self, key: str, hierarchy: int = 1):
        lvl = self._lvl(hierarchy)
        kv = self._load(getattr(self, f"{lvl}_BSA_EXE_PLANS_KV"))
        if key not in kv:
            return None
        with open(Path(getattr(self, f"{lvl}_BSA_EXE_PLANS_DIR")) / f"{kv[key]}.pkl", "rb") as f:
            return pickle.load(f)

    def get_plan_plain(self, key: str, hierarchy: int = 1) -> Optional[dict]:
        lvl = self._lvl(hierarchy)
        kv = self._load(getattr(self, f"{lvl}_BSA_EXE_PLANS_KV"))
        p = Path(getattr(self, f"{lvl}_BSA_EXE_PLANS_DIR")) / f"{kv.get(key, -1)}.json"
        return json.loads(p.read_text()) if p.exists() else None

    def get_plan_from_json(self, key: str, hierarchy: int = 1):
        """The stored plan rebuilt from its JSON side-car (nothing is unpickled); None if absent."""
        plain = self.get_plan_plain(key, hierarchy)
        if plain is None:
            return None
        from ..planner.schedule import Execution_Plan, Fused_Execution_Plan
        if plain.get("format", "").startswith("ultraattn-fused-plan"):
            return Fused_Execution_Plan.from_plain(plain, self.m_config)
        return Execution_Plan.from_plain(plain)

    # profiles
    def get_profile(self, key: str, hierarchy: int = 1) -> Optional[dict]:
        return self._load(getattr(self, f"{self._lvl(hierarchy)}_BSA_EXE_PLANS_PROFILE")).get(key)

    def put_profile(self, key: str, hfu: float, time_s: float, sim_time_s: float, hierarchy: int = 1,
                    **extra) -> None:
        path = Path(getattr(self, f"{self._lvl(hierarchy)}_BSA_EXE_PLANS_PROFILE"))
        d = self._load(path)
        d[key] = {"hfu": hfu, "time": f"{time_s:.3e}", "sim_time": f"{sim_time_s:.3e}", **extra}
        _atomic_write_json(path, d)

    # CRUD aliases of the reference's (empty) interface
    def insert(self, *a, **k): return self.put_profile(*a, **k)
    def read(self, key, hierarchy=1): return self.get_profile(key, hierarchy)
    def update(self, *a, **k): return self.put_profile(*a, **k)

    def delete(self, key: str, hierarchy: int = 1) -> None:
        path = Path(getattr(self, f"{self._lvl(hierarchy)}_BSA_EXE_PLANS_PROFILE"))
        d = self._load(path)
        d.pop(key, None)
        _atomic_write_json(path, d)
