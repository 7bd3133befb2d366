"""Problem descriptors and the cost model of the planner.

* :class:`Dist_Attn_Config` — one distributed-attention problem (shape + pattern + CP degrees),
  :class:`Dist_Attn_Schedule` — a tile -> rank table bound to a problem and a machine
  (reference: search_algo/search_engine.py:39-113, 348-412).
* :class:`FlashAttn_Profile_Map`, :class:`Inter_Comp_Profile_Map`, :class:`Comm_Profile_Map`,
  :class:`Machine_Config` — measured kernel times and link bandwidth, read from the same file
  formats as the reference's profilers (flash JSON ``{"flash_attn": [[[Smin,bs,Nh,D,"p/q",causal],
  [fwd_us,bwd_us,...]],...]}`` and ``SIZE n, REAL_BD .., BD/PAIR x GB/s`` logs; reference parsers at
  search_algo/utils.py:229-272; maps at search_algo/search_engine.py:115-328).

Where a key has not been profiled the maps fall back to an analytic B200 model (kernel throughput
and NVLink bandwidth measured for this framework's own kernels) instead of failing, so that
plans can be made on a machine without a GPU.
"""
from __future__ import annotations

import json
import math
import re
from functools import reduce
from pathlib import Path
from typing import Optional, Sequence

import numpy as np

from ..patterns.blocks import BSA_Config

GIB = 1024 ** 3

# measured on B200 with this repository's kernels (bf16, D = 128): sustained tile throughput
B200_FWD_TFLOPS = 1050.0
B200_BWD_TFLOPS = 1100.0
B200_NVLINK_GBS = 770.0          # peer copy, per direction
B200_LINK_LATENCY_S = 4e-6
B200_SMS = 148
B200_LAUNCH_S = 3e-5            # per-launch floor seen when tiles are tiny (host launch path included)
PACKAGED_M_CONFIG_DIR = Path(__file__).resolve().parents[1] / "data" / "m_configs" / "B200"


def convert_shape_config_to_str(shape_config: dict) -> str:
    return f"S={shape_config['S']}_Nh={shape_config['Nh']}_bs={shape_config['bs']}_D={shape_config['D']}"


class Evaluation_Configs:
    """How a plan is made: plan_type in {'ILP', 'manual', 'Flexflow'}; fob 0 = forward,
    1 = backward; hierarchy 0 = across nodes, 1 = inside a node; transform_mode in
    {'bf', 'greedy'} (reference: search_algo/search_engine.py:22-37)."""

    def __init__(self, plan_type: str, MAX_QUEUE_SIZE: int, fob: int, plan_path: Optional[str] = None,
                 hierarchy: Optional[int] = 1, transform_mode: str = "bf", inter_comp_profile_map=None):
        self.plan_type = plan_type
        self.MAX_QUEUE_SIZE = MAX_QUEUE_SIZE
        self.fob = fob
        self.plan_path = plan_path
        self.hierarchy = hierarchy
        self.transform_mode = transform_mode
        self.inter_comp_profile_map = inter_comp_profile_map
        self.execution_plan = None

    def get_plan_path(self) -> str:
        return self.plan_path


class Dist_Attn_Config:
    """``SP = (inter, intra)``; ``S = (Sq, Skv)`` totals; ``Nh = (Nh, Ng)``; note that
    ``BSA_Config.CP`` is ``(intra, inter)`` — the opposite order."""

    def __init__(self, SP, S, Nh, bs, D, causal=None, hierarchy: int = 1,
                 bsa_config: Optional[BSA_Config] = None):
        assert bsa_config is not None, "a block-sparse pattern (BSA_Config) is required"
        self.SP = tuple(SP)
        self.S = tuple(S)
        self.Nh = tuple(Nh)
        self.bs = bs
        self.D = D
        self.hierarchy = hierarchy
        self.bsa_config = bsa_config

    @classmethod
    def from_bsa_config(cls, bsa_config: BSA_Config, shape_config: dict, hierarchy: int):
        return cls((bsa_config.CP[1], bsa_config.CP[0]), **shape_config, causal=bsa_config.causal,
                   hierarchy=hierarchy, bsa_config=bsa_config)

    @property
    def causal(self) -> bool:
        return self.bsa_config.causal

    @property
    def shape_config(self) -> dict:
        return {"S": self.S, "Nh": self.Nh, "bs": self.bs, "D": self.D}

    @property
    def hierarchy_sp(self) -> int:
        return self.SP[self.hierarchy]

    @property
    def tot_sp(self) -> int:
        return reduce(lambda x, y: x * y, self.SP)

    @property
    def tot_Par_D(self) -> int:
        n = max(self.tot_sp, self.bsa_config.table.shape[0])
        if self.hierarchy == 0 and self.bsa_config.table.shape == (1, 1) and self.bsa_config.table[0, 0] == 2:
            n = self.tot_sp * (CP2ParD_map.get(self.SP[0], self.SP[0]) // self.SP[0])
        return n

    @property
    def S_per_gpu(self):
        return (self.S[0] // self.tot_sp, self.S[1] // self.tot_sp)

    @property
    def S_per_partition(self):
        return (self.S[0] // self.tot_Par_D, self.S[1] // self.tot_Par_D)

    def get_shape_config_str(self) -> str:
        return convert_shape_config_to_str(self.shape_config)

    def __str__(self) -> str:
        s = (f"SP={self.SP},Sg={self.S_per_gpu},S={self.S},Nh={self.Nh},bs={self.bs},D={self.D},"
             f"hierarchy={self.hierarchy}").replace(" ", "")
        return s + f",bsa_config={self.bsa_config}"


# inter-node causal uses a finer partition than the node count (reference: dense_utils.py:12-17)
CP2ParD_map = {1: 1, 2: 4, 4: 8, 8: 8}


# -------------------------------------------------------------------------------------------------
# compute cost
# -------------------------------------------------------------------------------------------------
def attention_flops(sq: int, skv: int, nh: int, bs: int, d: int, causal: bool, fob: int) -> float:
    """Model FLOPs of one tile: 4*Sq*Skv*D per head forward, 2.5x that backward (the reference
    counts 2x model / 2.5x hardware FLOPs for the backward, search_algo/utils.py:92-103)."""
    f = 4.0 * sq * skv * d * nh * bs * (0.5 if causal else 1.0)
    return f if fob == 0 else 2.5 * f


def analytic_tile_time(sq: int, skv: int, nh: int, bs: int, d: int, causal: bool) -> np.ndarray:
    """[fwd_s, bwd_s] of this framework's kernels on B200 for one tile. Small tiles under-fill the
    148 SMs: the forward launches ceil(Sq/256)*Nh CTAs, the backward ceil(Skv/128)*Nh."""
    def wave_eff(ctas: int) -> float:
        waves = ctas / 148.0
        return waves / math.ceil(waves) if ctas > 0 else 1.0
    f_fwd = attention_flops(sq, skv, nh, bs, d, causal, 0)
    f_bwd = attention_flops(sq, skv, nh, bs, d, causal, 1)
    e_f = max(wave_eff(math.ceil(sq / 256) * nh * bs), 0.05)
    e_b = max(wave_eff(math.ceil(skv / 128) * nh * bs), 0.05)
    return np.array([f_fwd / (B200_FWD_TFLOPS * 1e12 * e_f) + B200_LAUNCH_S,
                     f_bwd / (B200_BWD_TFLOPS * 1e12 * e_b) + B200_LAUNCH_S])


class Comp_Profile_Map:
    profile_map: dict

    def get_comp_time_from_map_key(self, map_key) -> np.ndarray:
        raise NotImplementedError

    def get_value_from_map_key(self, map_key):
        return self.get_comp_time_from_map_key(map_key)

    def get_comp_time(self, da_config, batch_degrees, split_degrees) -> np.ndarray:
        return self.get_comp_time_from_map_key(self.get_comp_map_key(da_config, batch_degrees, split_degrees))


class FlashAttn_Profile_Map(Comp_Profile_Map):
    """key ``(min(Sq,Skv), bs, Nh, D, "p/q", causal)`` -> ``[fwd_s, bwd_s]``."""

    def __init__(self, profile_map: Optional[dict] = None, analytic_fallback: bool = True):
        self.profile_map = dict(profile_map or {})
        self.analytic_fallback = analytic_fallback

    @staticmethod
    def _shape_of_key(key):
        smin, bs, nh, d, ratio, causal = key
        p, q = (int(x) for x in ratio.split("/"))
        if p >= q:
            skv = smin
            sq = smin * p // q
        else:
            sq = smin
            skv = smin * q // p
        return sq, skv, nh, bs, d, bool(causal)

    def get_comp_time_from_map_key(self, map_key) -> np.ndarray:
        if map_key in self.profile_map:
            return np.asarray(self.profile_map[map_key], dtype=float)
        if not self.analytic_fallback:
            raise KeyError(f"Key {map_key} not found in profile_map")
        near = self._from_nearest_measured(map_key)
        return near if near is not None else analytic_tile_time(*self._shape_of_key(map_key))

    def _from_nearest_measured(self, map_key) -> Optional[np.ndarray]:
        """A shape outside a measured grid (a fused rectangle, mostly) takes the throughput of the
        nearest measured shape of the same head dim and mask type (nearest in FLOPs, then in aspect
        ratio), scaled by its FLOPs. Mixing a measured profile with the analytic B200 model would
        price the unmeasured shapes for another machine: with the reference's H800 profile, fused
        tiles came out 2.7x faster than their parts."""
        if not self.profile_map:
            return None
        cached = getattr(self, "_near_cache", None)
        if cached is None:
            cached = self._near_cache = {}
        if map_key in cached:
            return cached[map_key]
        sq, skv, nh, bs, d, causal = self._shape_of_key(map_key)
        want = attention_flops(sq, skv, nh, bs, d, causal, 0)
        best, best_d = None, None
        for k, v in self.profile_map.items():
            if k[3] != d or bool(k[5]) != causal:
                continue
            ksq, kskv, knh, kbs, _, _ = self._shape_of_key(k)
            have = attention_flops(ksq, kskv, knh, kbs, d, causal, 0)
            dist = abs(math.log(have / want)) + 0.25 * abs(math.log((ksq / kskv) / (sq / skv)))
            if best_d is None or dist < best_d:
                best, best_d = np.asarray(v, dtype=float) * (want / have), dist
        cached[map_key] = best
        return best

    def get_comp_map_key(self, da_config: Dist_Attn_Config, batch_degrees: Sequence[int],
                         split_degrees: Sequence[int], causal: bool = False) -> tuple:
        sq = da_config.S[0] * batch_degrees[0] // split_degrees[0]
        skv = da_config.S[1] * batch_degrees[1] // split_degrees[1]
        bs = da_config.bs // split_degrees[2]
        nh = da_config.Nh[0] // split_degrees[3]
        g = math.gcd(sq, skv)
        return (min(sq, skv), bs, nh, da_config.D, f"{sq // g}/{skv // g}", causal)

    def merge_comp_map_key(self, k0: tuple, k1: tuple, merge_dim: int) -> tuple:
        """Key of the tile obtained by gluing two non-causal tiles along dim 0 (Sq), 1 (Skv),
        2 (bs) or 3 (Nh)."""
        assert not (k0[5] or k1[5]), "causal tiles are not merged"
        if merge_dim in (0, 1):
            s0 = self._shape_of_key(k0)[:2]
            s1 = self._shape_of_key(k1)[:2]
            assert s0[merge_dim ^ 1] == s1[merge_dim ^ 1]
            s = (s0[0] + s1[0], s0[1]) if merge_dim == 0 else (s0[0], s0[1] + s1[1])
            g = math.gcd(*s)
            return (min(s), k0[1], k0[2], k0[3], f"{s[0] // g}/{s[1] // g}", False)
        out = list(k0)
        out[merge_dim - 1] += k1[merge_dim - 1]
        return tuple(out)


class Inter_Comp_Profile_Map(Comp_Profile_Map):
    """String database key -> measured time of the intra-node plan that implements an inter-node
    compute tile (reference: search_algo/search_engine.py:272-280)."""

    def __init__(self, profile_map: Optional[dict] = None):
        self.profile_map = dict(profile_map or {})

    def get_comp_time_from_map_key(self, map_key) -> np.ndarray:
        v = self.profile_map[map_key]
        if isinstance(v, dict):
            t = float(v["time"])
            return np.array([t, t])
        return np.asarray(v, dtype=float)

    def update(self, other: dict) -> None:
        self.profile_map.update(other)


# -------------------------------------------------------------------------------------------------
# communication cost
# -------------------------------------------------------------------------------------------------
class Comm_Profile_Map:
    """``(bytes,)`` -> GB/s of one peer-to-peer message under a 2-rank bidirectional pattern;
    ``time = bytes / BW(bytes)``, clamped to the largest profiled size."""

    def __init__(self, profile_map: Optional[dict] = None, peak_gbs: float = B200_NVLINK_GBS,
                 latency_s: float = B200_LINK_LATENCY_S):
        self.profile_map = dict(profile_map or {})
        self.sizes = sorted(k[0] for k in self.profile_map)
        self.peak_gbs = peak_gbs
        self.latency_s = latency_s

    def get_comm_map_key(self, da_config: Dist_Attn_Config, batch_degrees, split_degrees) -> tuple:
        """Bytes of one comm unit: one Q-side tile, ``Sq_tile * bs * Nh * D * 2``."""
        sq = da_config.S[0] * batch_degrees[0] // split_degrees[0]
        return (sq * (da_config.bs // split_degrees[2]) * (da_config.Nh[0] // split_degrees[3])
                * da_config.D * 2,)

    def bandwidth_gbs(self, nbytes: float) -> float:
        if not self.sizes:
            if nbytes <= 0:
                return self.peak_gbs
            return nbytes / 1e9 / (self.latency_s + nbytes / (self.peak_gbs * 1e9))
        import bisect
        i = bisect.bisect_left(self.sizes, nbytes)
        i = min(i, len(self.sizes) - 1)
        return self.profile_map[(self.sizes[i],)]

    def get_comm_time_from_map_key(self, map_key) -> float:
        nbytes = map_key[0]
        if nbytes <= 0:
            return 0.0
        return nbytes / 1e9 / self.bandwidth_gbs(nbytes)

    get_value_from_map_key = get_comm_time_from_map_key


class Fused_Transport_Profile:
    """Measured throughput of the transports that only the fused runtime uses, read from the JSON
    table that ``drivers.cluster_profile --comm-fused`` writes (one record per point: ``transport``,
    ``ranks``, ``bytes``, ``gbs_per_rank`` and, for staging pulls, ``copy_ctas``). Every rank was
    active while a point was measured, so the figures already include the contention of an
    all-ranks pattern. A transport without records answers ``None`` and the caller falls back to the
    point-to-point link curve."""

    def __init__(self, records: Optional[Sequence[dict]] = None):
        self.records = list(records or [])

    def _points(self, transport: str, ranks: Optional[int]):
        pts = [r for r in self.records if r.get("transport") == transport]
        if ranks is not None and pts:
            best = min({r["ranks"] for r in pts}, key=lambda n: (abs(n - ranks), -n))
            pts = [r for r in pts if r["ranks"] == best]
        return pts

    def pull_gbs(self, copy_ctas: int, ranks: Optional[int] = None) -> Optional[float]:
        """GB/s into one rank when ``copy_ctas`` CTAs stage peer blocks (linear between measured
        CTA counts, flat outside them)."""
        pts = sorted((r["copy_ctas"], r["gbs_per_rank"]) for r in self._points("peer_pull", ranks))
        if not pts:
            return None
        xs, ys = zip(*pts)
        return float(np.interp(copy_ctas, xs, ys))

    def gbs(self, transport: str, nbytes: float, ranks: Optional[int] = None) -> Optional[float]:
        """GB/s of ``transport`` at a message of ``nbytes`` (log-linear between measured sizes)."""
        pts = sorted((r["bytes"], r["gbs_per_rank"]) for r in self._points(transport, ranks))
        if not pts or nbytes <= 0:
            return None
        xs, ys = zip(*pts)
        return float(np.interp(math.log2(nbytes), [math.log2(x) for x in xs], ys))

    def time_s(self, transport: str, nbytes: float, ranks: Optional[int] = None, **kw) -> Optional[float]:
        g = self.pull_gbs(kw["copy_ctas"], ranks) if transport == "peer_pull" else self.gbs(transport, nbytes, ranks)
        return None if not g else nbytes / (g * 1e9)


class Machine_Config:
    """[inter, intra] compute maps, [inter, intra] communication maps and the fused runtime's
    transport table."""

    def __init__(self, BW=None, comp_profile_maps=None, comm_profile_maps=None, fused_transports=None):
        self.BW = BW or (B200_NVLINK_GBS, B200_NVLINK_GBS)
        self.comp_profile_maps = comp_profile_maps or [Inter_Comp_Profile_Map(), FlashAttn_Profile_Map()]
        self.comm_profile_maps = comm_profile_maps or [Comm_Profile_Map(), Comm_Profile_Map()]
        self.fused_transports = fused_transports or Fused_Transport_Profile()

    def __getstate__(self) -> dict:
        """The transport table travels as its plain records: a pickled plan (which carries its
        machine profile) then names no class that the reference does not have."""
        state = dict(self.__dict__)
        ft = state.pop("fused_transports", None)
        state["fused_transport_records"] = list(ft.records) if ft is not None else []
        return state

    def __setstate__(self, state: dict) -> None:
        self.__dict__.update(state)
        self.fused_transports = Fused_Transport_Profile(self.__dict__.pop("fused_transport_records", []))

    @classmethod
    def b200_default(cls) -> "Machine_Config":
        """The machine profile shipped with the package (``data/m_configs/B200``: the kernel grid
        measured on a B200 with this repository's kernels, in the reference's ``time*.json``
        format, and link curves when present); shapes outside the measured grid use the analytic
        model."""
        return cls.from_dir(PACKAGED_M_CONFIG_DIR)

    @classmethod
    def from_dir(cls, m_config_dir) -> "Machine_Config":
        """Read ``time*.json`` / ``cb_8_*.log`` / ``cb_16_*.log`` / ``fused_comm_*.json`` of a
        directory; what is missing falls back to the analytic B200 model."""
        mdir = Path(m_config_dir)
        flash = sorted(mdir.glob("time*.json")) if mdir.is_dir() else []
        cb8 = sorted(mdir.glob("cb_8_*.log")) if mdir.is_dir() else []
        cb16 = sorted(mdir.glob("cb_16_*.log")) if mdir.is_dir() else []
        comp_intra = FlashAttn_Profile_Map(load_flash_profile(flash[0]) if flash else None)
        comm_intra = Comm_Profile_Map(convert_profile_data_to_comm_map(cb8[0]) if cb8 else None)
        comm_inter = Comm_Profile_Map(convert_profile_data_to_comm_map(cb16[0]) if cb16 else None)
        ft = sorted(mdir.glob("fused_comm_*.json")) if mdir.is_dir() else []
        records = [r for f in ft for r in json.loads(f.read_text())]
        return cls(None, [Inter_Comp_Profile_Map(), comp_intra], [comm_inter, comm_intra],
                   Fused_Transport_Profile(records))

    def update_inter_bsa_profile(self, profile: dict) -> None:
        self.comp_profile_maps[0].update(profile)


# -------------------------------------------------------------------------------------------------
# profile file formats
# -------------------------------------------------------------------------------------------------
def convert_profile_data_to_map(profile_list) -> dict:
    out = {}
    for key, vals in profile_list:
        out[tuple(key)] = np.array(vals[:2], dtype=float) / 1e6      # us -> s
    return out


def load_flash_profile(path) -> dict:
    data = json.loads(Path(path).read_text())
    return convert_profile_data_to_map(data["flash_attn"])


def dump_flash_profile(path, entries) -> None:
    """entries: iterable of (key tuple, fwd_s, bwd_s, fwd_tflops, bwd_tflops)."""
    rows = [[list(k), [f * 1e6, b * 1e6, tf, tb]] for k, f, b, tf, tb in entries]
    Path(path).write_text(json.dumps({"flash_attn": rows}, indent=1))


_UNIT = {"B": 1.0, "KB": 1e3, "MB": 1e6, "GB": 1e9, "TB": 1e12}
_CB_LINE = re.compile(r"^SIZE (\d+),.*?BD/PAIR (\d*(?:\.\d*)?) ([A-Z]+)/s")


def convert_throughput_to_B(size: float, unit: str) -> float:
    """``size`` in ``unit`` (B, KB, MB, ... with decimal steps of 1000) -> bytes."""
    names = ["B", "KB", "MB", "GB", "TB", "PB", "EB", "ZB", "YB"]
    assert unit in names, f"invalid unit {unit!r}"
    return size * 1000 ** names.index(unit)


def create_schedule(da_config, m_config, split_degrees, S_map, schedule_table_func, hierarchy: int = 1):
    """A ``Dist_Attn_Schedule`` (or a list of them) from a function that returns the allocation
    table(s) for a partition (reference: search_algo/search_engine.py:951-957)."""
    tables = schedule_table_func(split_degrees, S_map, da_config=da_config)
    if isinstance(tables, list):
        return [Dist_Attn_Schedule(da_config, m_config, split_degrees, S_map, t, hierarchy) for t in tables]
    return Dist_Attn_Schedule(da_config, m_config, split_degrees, S_map, tables, hierarchy)


def convert_profile_data_to_comm_map(file_name, num_gpus_div: int = 1) -> dict:
    out = {}
    for line in Path(file_name).read_text().splitlines():
        m = _CB_LINE.match(line)
        if m:
            out[(int(m.group(1)),)] = float(m.group(2)) * _UNIT[m.group(3)] / 1e9
    return out


def format_cb_line(size_elems: int, real_gbs: float, pair_gbs: float, time_s: float, vol_mb: float) -> str:
    return (f"SIZE {size_elems}, REAL_BD {real_gbs:.3f} GB/s, BD/PAIR {pair_gbs:.3f} GB/s, "
            f"time {time_s:.3e} s, comm_vol {vol_mb:.3f} MB")


# -------------------------------------------------------------------------------------------------
# schedule
# -------------------------------------------------------------------------------------------------
class Dist_Attn_Schedule:
    """A tile allocation bound to a problem: ``schedule_table[bs, Nh, q_blk, kv_blk]`` = rank
    computing the tile (-1 empty); ``S_map[bs, blk]`` = owner rank of each sequence block;
    ``split_degrees = (Sq_split, Skv_split, bs_split, Nh_split)``.

    Communication units per message kind, [fwd, bwd], in Q-tile units
    (reference: search_algo/search_engine.py:388-409):
    input row (Q | Q+dO) = [1, 2]; input col (K,V) = [2, 2]*r; output row (O | dQ) = [1, 1];
    output col (- | dK,dV) = [0, 2]*r with r the KV/Q size ratio.
    """

    def __init__(self, da_config: Dist_Attn_Config, m_config: Machine_Config, split_degrees,
                 S_map: np.ndarray, schedule_table: np.ndarray, hierarchy: Optional[int] = None):
        self.da_config = da_config
        self.m_config = m_config
        self.split_degrees = tuple(split_degrees)
        self.S_map = np.asarray(S_map)
        self.schedule_table = np.asarray(schedule_table)
        assert self.schedule_table.shape == (split_degrees[2], split_degrees[3], split_degrees[0],
                                             split_degrees[1])
        kv_ratio = ((da_config.S[1] / split_degrees[1]) / (da_config.S[0] / split_degrees[0])
                    * (da_config.Nh[1] / da_config.Nh[0]))
        self.u_inp_row = np.array([1.0, 2.0])
        self.u_inp_col = np.array([2.0, 2.0]) * kv_ratio
        self.u_out_row = np.array([1.0, 1.0])
        self.u_out_col = np.array([0.0, 2.0]) * kv_ratio

    @property
    def tot_sp(self) -> int:
        return self.da_config.tot_sp

    @property
    def hierarchy(self) -> int:
        return self.da_config.hierarchy

    @property
    def hierarchy_sp(self) -> int:
        return self.da_config.hierarchy_sp

    def get_relative_cc_time(self) -> float:
        return 0.0


def get_cc_optimal_schedule_from_table(da_config: Dist_Attn_Config, m_config: Machine_Config,
                                       allocation) -> Dist_Attn_Schedule:
    """Wrap an ILP #1 result (dict-like with 'Par_D', 'cmap', 'table') into a schedule
    (reference: search_algo/search_engine.py:969-987)."""
    par_d = int(allocation["Par_D"])
    table = np.asarray(allocation["table"])
    cmap = np.asarray(allocation["cmap"])
    split = (par_d, par_d, 1, 1)
    s_map = np.tile(cmap[None, :], (1, 1))
    return Dist_Attn_Schedule(da_config, m_config, split, s_map, table[None, None])


# -------------------------------------------------------------------------------------------------
# legacy node-profile logs
# -------------------------------------------------------------------------------------------------
_LEGACY_BASELINES = ("ring_flash_attn_func", "zigzag_ring_flash_attn_func", "stripe_flash_attn_func")


def format_node_profile_lines(fob: int, SP, S, Nh, bs: int, D: int, causal: bool, results: dict) -> list:
    """Log lines of one measured configuration in the format the reference's benchmark prints and
    its cost model parses back (search_algo/utils.py:274-363). ``results`` maps a section name
    (``orchestrated_attn_func``, ``orchestrated_attn_func fused`` or a baseline function name) to
    a list of ``(tflops, seconds_per_iter)`` measurements."""
    lines = [f"fob={fob}",
             f"da_config: SP=({SP[0]},{SP[1]}),Sg=({S[0] // (SP[0] * SP[1])},{S[1] // (SP[0] * SP[1])}),"
             f"S=({S[0]},{S[1]}),Nh=({Nh[0]},{Nh[1]}),bs={bs},D={D},causal={causal},hierarchy=1"]
    for name, runs in results.items():
        lines.append(f"# {name}")
        for tflops, sec in runs:
            lines.append(f"mfu: {tflops:.3f} Tflops/s, hfu: {tflops:.3f} Tflops/s, {1.0 / sec:.3f} iter/s, "
                         f"{sec:.3e} s/iter, (0.000, 0.000, 0.000) sec")
    return lines


def convert_node_profile_data_to_comp_map(file_name, local_size: int = 8) -> dict:
    """Parse a node-profile log into ``{'level0' | 'level1' | 'level2': {key: [fwd_s, bwd_s]}}``
    with ``key = (SP, S_per_gpu, Nh, bs, D, causal)``.

    The log is a sequence of ``fob=<0|1>`` lines, configuration lines (``SP=(a,b),...S=(..),Nh=(..),
    bs=..,D=..,causal=..``), section headers naming the function that was timed and timing lines
    (``... iter/s, <t> s/iter, ...``). Level 0 keeps the best time of the plain orchestrated
    sections, level 1 (and its alias level 2) the best over plain and kernel-tile ("fused")
    sections. Sections of the ring-family baselines are skipped, as in the reference, whose
    authors did not trust those numbers (search_algo/utils.py:311)."""
    import re
    out = {"level0": {}, "level1": {}}
    if file_name is None:
        return out
    rx_fob = re.compile(r"^fob=(\d)")
    rx_cfg = re.compile(r"SP=\((\d+),(\d+)\),.*S=\((\d+),(\d+)\),Nh=\((\d+),(\d+)\),bs=(\d+),D=(\d+),causal=(True|False)")
    rx_time = re.compile(r"iter/s, (-?\d+(?:\.\d+)?(?:e[+-]\d+)?) s/iter")
    fob = key = None
    level = 0
    in_baseline = False
    with open(file_name) as f:
        for line in f:
            if any(b in line for b in _LEGACY_BASELINES):
                in_baseline = True
                continue
            if "orchestrated_attn_func" in line:
                in_baseline = False
                level = 1 if "fused" in line else 0
                continue
            m = rx_time.search(line)
            if m:
                if in_baseline or key is None or fob is None:
                    continue
                t = float(m.group(1))
                for lv in range(level, 2):
                    slot = out[f"level{lv}"].setdefault(key, np.full(2, np.inf, dtype=np.float32))
                    slot[fob] = min(slot[fob], t)
                out["level0"].setdefault(key, np.full(2, np.inf, dtype=np.float32))
                continue
            m = rx_cfg.search(line)
            if m:
                g = [int(x) for x in m.groups()[:8]]
                tot = g[0] * g[1]
                key = ((g[0], g[1]), (g[2] // tot, g[3] // tot), (g[4], g[5]), g[6], g[7], m.group(9) == "True")
                in_baseline = False
                continue
            m = rx_fob.match(line)
            if m:
                fob = int(m.group(1))
    out["level2"] = out["level1"]
    return out


# -------------------------------------------------------------------------------------------------
# time model of the fused runtime
# -------------------------------------------------------------------------------------------------
def fused_step_time(table, cmap, pattern, seq_len: int, n_heads: int, head_dim: int = 128,
                    m_config: Optional["Machine_Config"] = None, n_kv_heads: Optional[int] = None,
                    batch: int = 1, hbm_gbs: float = 6400.0, copy_ctas: int = 148) -> dict:
    """Predicted time of one forward and one backward call of the fused context-parallel runtime
    for an allocation ``table`` (tile -> rank) and ownership ``cmap``.

    Unlike a launch plan's ``end_time`` (one launch and one message per tile, scheduled on three
    streams) the fused runtime runs ONE kernel per pass and rank that walks all of the rank's
    tiles, pulls remote blocks while the first tiles compute and pushes results from its epilogue.
    Its time per rank is therefore modelled as: the sum of the rank's tile times (from the kernel
    grid of the machine profile, at the tile's shape and mask type, minus the per-launch floor that
    a fused launch pays only once) + what the transfers cannot hide (the larger of inbound and
    outbound NVLink bytes over the link curve, overlapped with compute: only the excess counts)
    + the memory-bound passes around the kernels (copy-in of the shards, D = rowsum(dO * O),
    merge of mailbox slots, fp32 -> bf16 cast and clearing of the accumulators). The step ends
    when the slowest rank ends. Returns per-pass times in seconds and the per-rank breakdown.

    Inbound bytes are staged by ``copy_ctas`` CTAs with peer loads and outbound fp32 partial sums
    leave as peer ``red.add``; where the machine profile has measured those transports
    (``Fused_Transport_Profile``) their throughput replaces the point-to-point link curve. The CTAs
    that stage do so before they take their first tile, so staging also costs compute time: its
    duration times the share of the SMs that copy (``stage_s`` in the breakdown). The dQ of foreign
    rows leaves in a launch of its own after the backward kernel (``dq_push_s``)."""
    import numpy as _np
    m = m_config or Machine_Config.b200_default()
    table = _np.asarray(table)
    cmap = _np.asarray(cmap)
    par_d = table.shape[0]
    cp = int(cmap.max()) + 1
    blk = seq_len // par_d
    hk = n_kv_heads or n_heads
    types = pattern.refined(par_d)
    comp = m.comp_profile_maps[1]
    comm = m.comm_profile_maps[1]
    t_tile = {c: _np.maximum(comp.get_comp_time_from_map_key((blk, batch, n_heads, head_dim, "1/1", c))
                             - B200_LAUNCH_S, 1e-7) for c in (False, True)}
    es = 2
    q_blk = batch * blk * n_heads * head_dim * es
    kv_blk = batch * blk * hk * head_dim * es
    shard = seq_len // cp
    out = {"per_rank": []}
    for g in range(cp):
        tiles = [(r, c) for r in range(par_d) for c in range(par_d) if table[r, c] == g]
        comp_t = _np.zeros(2)
        for r, c in tiles:
            comp_t += t_tile[bool(types[r, c] == 2)]
        rows = {r for r, _ in tiles if cmap[r] != g}
        cols = {c for _, c in tiles if cmap[c] != g}
        # forward: pull Q rows and K, V columns; push (O, lse) of foreign rows
        f_in = len(rows) * q_blk + len(cols) * 2 * kv_blk
        f_out = len(rows) * (q_blk + batch * n_heads * blk * 4)
        # backward (inputs staged by the forward are reused): pull dO, lse, D; push dQ (fp32), dK, dV (fp32)
        b_in = len(rows) * (q_blk + 2 * batch * n_heads * blk * 4)
        b_out = len(rows) * 2 * q_blk + len(cols) * 2 * 2 * kv_blk
        ft = m.fused_transports

        def t_in(x):
            return 0.0 if not x else (ft.time_s("peer_pull", x, cp, copy_ctas=copy_ctas)
                                      or comm.get_comm_time_from_map_key((x,)))

        def t_out(x, transport):
            return 0.0 if not x else (ft.time_s(transport, x, cp) or comm.get_comm_time_from_map_key((x,)))

        link = [max(t_in(f_in), t_out(f_out, "peer_store")), max(t_in(b_in), t_out(b_out, "peer_red_add_f32"))]
        own_q = batch * shard * n_heads * head_dim
        own_kv = batch * shard * hk * head_dim
        mem_f = (2 * (own_q + 2 * own_kv) * es + len(rows) * 0 + 3 * own_q * es) / (hbm_gbs * 1e9)
        mem_b = (2 * own_q * es + 2 * own_q * es            # copy-in of dO, D pre-pass reads O and dO
                 + (own_q + 2 * own_kv) * (4 + es + 4)) / (hbm_gbs * 1e9)   # cast + clear of the accumulators
        launch = _np.array([B200_LAUNCH_S * 3, B200_LAUNCH_S * 5])
        share = min(copy_ctas, B200_SMS) / B200_SMS
        stage = [t_in(f_in) * share, t_in(b_in) * share]
        # dQ of foreign rows is accumulated in a local fp32 mirror and pushed to its owner by a
        # separate launch after the backward kernel: not overlapped with compute
        dq_push = t_out(len(rows) * 2 * q_blk, "peer_red_add_f32")
        total = _np.array([max(comp_t[0] + stage[0], link[0]) + mem_f,
                           max(comp_t[1] + stage[1], link[1]) + mem_b + dq_push]) + launch
        out["per_rank"].append({"rank": g, "tiles": len(tiles), "compute_s": comp_t.tolist(), "link_s": link, "stage_s": stage, "dq_push_s": dq_push,
                                "memory_s": [mem_f, mem_b], "total_s": total.tolist()})
    out["fwd_s"] = max(r["total_s"][0] for r in out["per_rank"])
    out["bwd_s"] = max(r["total_s"][1] for r in out["per_rank"])
    out["step_s"] = out["fwd_s"] + out["bwd_s"]
    return out


def ring_step_time(pattern, cp: int, seq_len: int, n_heads: int, head_dim: int = 128,
                   m_config: Optional["Machine_Config"] = None, n_kv_heads: Optional[int] = None,
                   batch: int = 1, kind: str = "ring") -> dict:
    """Predicted forward and backward time of the ring baselines (``parallel/ring.py``) with
    contiguous shards: ``cp`` steps; in every step a rank computes the block pairs that the
    pattern allows between its queries and the visiting K/V shard (one launch) while the next
    shard travels (K and V forward; in the backward also the fp32 dK, dV that ride along).
    ``kind="zigzag"`` models the balanced causal layout (every rank does the same share of every
    step). A block-sparse pattern lets the ring skip compute but not transfers, which is why its
    advantage shrinks with sparsity.

    The ranks are not in lock step: a rank goes on as soon as its own compute and its own exchange
    are done. An exchange (one grouped send + receive) completes one transfer time after the rank
    and BOTH its ring neighbours have reached the step, so a rank with work in a step delays its
    neighbours by one step each, not the whole ring. (Summing the slowest rank of every step, as a
    lock-step model does, doubled the prediction for the prefill patterns, where one rank per step
    has work: star on 8 GPUs 148 ms against 76 ms measured; this recurrence gives 53 ms.)"""
    import numpy as _np
    m = m_config or Machine_Config.b200_default()
    comp, comm = m.comp_profile_maps[1], m.comm_profile_maps[1]
    hk = n_kv_heads or n_heads
    n = pattern.table.shape[0]
    par_d = n * cp // math.gcd(n, cp)
    types = pattern.refined(par_d)
    per = par_d // cp
    blk = seq_len // par_d
    t_tile = {c: _np.maximum(comp.get_comp_time_from_map_key((blk, batch, n_heads, head_dim, "1/1", c))
                             - B200_LAUNCH_S, 1e-7) for c in (False, True)}
    kv_bytes = 2 * batch * (seq_len // cp) * hk * head_dim * 2
    t_kv = comm.get_comm_time_from_map_key((kv_bytes,))
    t_dkv = comm.get_comm_time_from_map_key((2 * kv_bytes,))          # fp32 dK, dV
    work = _np.zeros((cp, cp, 2))                                      # [rank, step, pass]
    for step in range(cp):
        for rank in range(cp):
            src = (rank - step) % cp
            for i in range(per):
                for j in range(per):
                    ty = int(types[rank * per + i, src * per + j])
                    if ty:
                        work[rank, step] += t_tile[ty == 2]
        if kind == "zigzag":
            work[:, step] = work[:, step].sum(axis=0) / cp
    out = []
    for fob, t_x in ((0, t_kv), (1, t_kv + t_dkv)):
        start = _np.zeros(cp)                                          # when each rank enters the step
        for step in range(cp):
            busy = work[:, step, fob]
            done = start + _np.where(busy > 0, busy + B200_LAUNCH_S, 0.0)
            if step + 1 == cp:
                start = done
                break
            posted = _np.maximum(start, _np.maximum(_np.roll(start, 1), _np.roll(start, -1)))
            start = _np.maximum(done, posted + t_x)
        out.append(float(start.max()))
    return {"fwd_s": out[0], "bwd_s": out[1], "step_s": out[0] + out[1]}
