"""Process topology and small communication helpers.

``get_proc_info`` / ``initialize_distribution`` mirror search_algo/initialize.py:29-159 (SLURM,
OpenMPI or torchrun environment -> rank / local rank / node id; NCCL or gloo process group, a gloo
control-plane group with a long timeout for CPU-side solver runs, power-of-two prefix sub-groups).
``RingComm`` and ``A2AComm`` mirror comm_lib/comm_utils.py:11-128 on ``torch.distributed`` only:
the data plane of the fused path does not go through here, these serve the baselines.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist

PROC_INFO: dict = {}
_groups: dict = {}

# bytes this process handed to / asked from torch.distributed point-to-point and all-to-all calls,
# by phase (reference: the per-step byte counters of LightSeq's communication layer,
# easy_context/dist_flash_attn/async_communication.py:499-512)
_comm_stats = {"fwd_send": 0, "fwd_recv": 0, "bwd_send": 0, "bwd_recv": 0}
_comm_phase = ["fwd"]


def set_comm_phase(phase: str) -> None:
    assert phase in ("fwd", "bwd")
    _comm_phase[0] = phase


def count_comm(send_bytes: int = 0, recv_bytes: int = 0) -> None:
    _comm_stats[_comm_phase[0] + "_send"] += int(send_bytes)
    _comm_stats[_comm_phase[0] + "_recv"] += int(recv_bytes)


def comm_stats(reset: bool = False) -> dict:
    out = dict(_comm_stats)
    if reset:
        for k in _comm_stats:
            _comm_stats[k] = 0
    return out


def print_and_reset_comm_stats(rank: Optional[int] = None) -> dict:
    """Print this rank's communicated volume in GB per phase and direction, then clear it."""
    st = comm_stats(reset=True)
    r = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
    print(f"R={r} fwd send: {st['fwd_send'] * 1e-9} fwd recv: {st['fwd_recv'] * 1e-9}; "
          f"bwd send: {st['bwd_send'] * 1e-9}, bwd recv: {st['bwd_recv'] * 1e-9} GB.", flush=True)
    return st


def parse_slurm_tasks_per_node(tasks_per_node: str) -> int:
    """``SLURM_TASKS_PER_NODE`` ("8", "4(x2)", "8,8") -> tasks on the first node."""
    return int(str(tasks_per_node).split("(")[0].split(",")[0])


def initialize_prof_db(gloo_global_group=None):
    """The plan / profile database of this cluster and platform (``CLUSTER_NAME`` / ``PLATFORM``
    from the environment), as the campaign drivers open it (reference: search_algo/initialize.py:19-23)."""
    import os
    from ..plandb.db import Prof_DB
    return Prof_DB(os.environ.get("CLUSTER_NAME"), os.environ.get("PLATFORM"), gloo_global_group)


def get_proc_info() -> dict:
    env = os.environ
    if "SLURM_PROCID" in env and "RANK" not in env:
        rank = int(env["SLURM_PROCID"])
        local_rank = int(env.get("SLURM_LOCALID", 0))
        world = int(env["SLURM_NTASKS"])
        per_node = parse_slurm_tasks_per_node(env.get("SLURM_TASKS_PER_NODE", world))
        node_id = int(env.get("SLURM_NODEID", rank // max(per_node, 1)))
        ip = env.get("SLURM_STEP_NODELIST", "127.0.0.1")
    elif "OMPI_COMM_WORLD_RANK" in env:
        rank = int(env["OMPI_COMM_WORLD_RANK"])
        local_rank = int(env.get("OMPI_COMM_WORLD_LOCAL_RANK", 0))
        world = int(env["OMPI_COMM_WORLD_SIZE"])
        per_node = int(env.get("OMPI_COMM_WORLD_LOCAL_SIZE", world))
        node_id = rank // max(per_node, 1)
        ip = env.get("MASTER_ADDR", "127.0.0.1")
    else:
        rank = int(env.get("RANK", 0))
        local_rank = int(env.get("LOCAL_RANK", rank))
        world = int(env.get("WORLD_SIZE", 1))
        per_node = int(env.get("LOCAL_WORLD_SIZE", world))
        node_id = rank // max(per_node, 1)
        ip = env.get("MASTER_ADDR", "127.0.0.1")
    info = {"rank": rank, "local_rank": local_rank, "world_size": world, "tasks_per_node": per_node,
            "nodeid": node_id, "node_num": max(1, world // max(per_node, 1)), "ip": ip,
            "deviceid": local_rank}
    PROC_INFO.clear()
    PROC_INFO.update(info)
    return info


def initialize_distribution(backend: Optional[str] = None, control_timeout_days: int = 28) -> dict:
    """Initialise torch.distributed for this process and create the control-plane groups."""
    info = get_proc_info()
    use_cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if use_cuda else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if use_cuda:
        torch.cuda.set_device(info["local_rank"])
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", info["local_rank"])
        dist.init_process_group(backend, rank=info["rank"], world_size=info["world_size"], **kw)
    ranks = list(range(info["world_size"]))
    _groups[("gloo", tuple(ranks))] = dist.new_group(
        ranks, backend="gloo", timeout=datetime.timedelta(days=control_timeout_days))
    n = 0
    while (1 << n) <= info["world_size"]:
        sub = list(range(1 << n))
        _groups[("prefix", tuple(sub))] = dist.new_group(sub)
        n += 1
    return info


def get_group(kind: str, ranks) -> Optional[dist.ProcessGroup]:
    return _groups.get((kind, tuple(ranks)))


def control_group():
    for (kind, _), g in _groups.items():
        if kind == "gloo":
            return g
    return None


class RingComm:
    """Neighbour exchange on a ring: ``send_recv`` posts a send to rank+1 and a receive from
    rank-1, ``commit`` launches the batch, ``wait`` completes it."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self._ops = []
        self._reqs = None
        self.send_rank = self._glob((self.rank + 1) % self.world)
        self.recv_rank = self._glob((self.rank - 1) % self.world)

    def _glob(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def send_recv(self, to_send: torch.Tensor, recv_tensor: Optional[torch.Tensor] = None) -> torch.Tensor:
        res = torch.empty_like(to_send) if recv_tensor is None else recv_tensor
        nbytes = to_send.numel() * to_send.element_size()
        count_comm(nbytes, nbytes)
        self._ops.append(dist.P2POp(dist.isend, to_send, self.send_rank, group=self.group))
        self._ops.append(dist.P2POp(dist.irecv, res, self.recv_rank, group=self.group))
        return res

    def commit(self) -> None:
        assert self._reqs is None, "commit called twice"
        self._reqs = dist.batch_isend_irecv(self._ops) if self._ops else []

    def wait(self) -> None:
        assert self._reqs is not None, "wait before commit"
        for r in self._reqs:
            r.wait()
        self._reqs = None
        self._ops = []


class A2AComm:
    """All-to-all re-sharding between the sequence and the head dimension (Ulysses)."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)

    def all_to_all(self, x: torch.Tensor, scatter_dim: int, gather_dim: int) -> torch.Tensor:
        """Split ``x`` along ``scatter_dim`` into ``world`` parts, exchange, concatenate along
        ``gather_dim``."""
        if self.world == 1:
            return x
        ins = [t.contiguous() for t in x.chunk(self.world, dim=scatter_dim)]
        moved = (self.world - 1) * ins[0].numel() * ins[0].element_size()
        count_comm(moved, moved)
        outs = [torch.empty_like(ins[0]) for _ in range(self.world)]
        dist.all_to_all(outs, ins, group=self.group) if x.is_cuda else _a2a_p2p(outs, ins, self.group)
        return torch.cat(outs, dim=gather_dim)


def _a2a_p2p(outs, ins, group) -> None:
    """gloo has no all_to_all: emulate with point-to-point messages."""
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    glob = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    ops = []
    for r in range(world):
        if r == rank:
            outs[r].copy_(ins[r])
        else:
            ops.append(dist.P2POp(dist.isend, ins[r], glob(r), group=group))
            ops.append(dist.P2POp(dist.irecv, outs[r], glob(r), group=group))
    for req in dist.batch_isend_irecv(ops) if ops else []:
        req.wait()
