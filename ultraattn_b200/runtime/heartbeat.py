"""Host-side liveness between steps: who is still taking part in the next step?

A rank announces every step it is about to enter in the job's key-value store (the TCP store
that ``torch.distributed`` already runs for the rendezvous), and before launching anything for
that step the ranks look for peers that have not announced it within a short time limit, or that
said good-bye. Nothing on a GPU waits for a rank that is gone: the survivors learn of it on the
host, before their next launch, and can re-plan for a smaller group
(``ContextParallelAttention.replan``). The reference has no such mechanism: a task that fails
ends the job (scripts/runtime/wrapper_bx.sh:19) and leftover processes are killed by hand
(tools/kill_dead_ps.sh).
"""
from __future__ import annotations

import time
from typing import Optional

import torch.distributed as dist

LEFT = "left"


class ExcludedFromGroup(RuntimeError):
    """The survivors agreed on a member list for a step that does not contain this rank (its
    announcement came too late for the rank whose view was adopted): it must not take part."""


class StepHeartbeat:
    def __init__(self, store=None, rank: Optional[int] = None, world: Optional[int] = None, prefix: str = "ua_hb"):
        if store is None:
            from torch.distributed.distributed_c10d import _get_default_store
            store = _get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix = prefix
        self.alive = list(range(self.world))

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        """Announce that this rank enters ``step``."""
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self) -> None:
        """Say good-bye (between steps, with nothing of this rank in flight)."""
        self.store.set(self._key(self.rank), LEFT)

    def _state(self, r: int):
        key = self._key(r)
        if not self.store.check([key]):
            return None
        val = self.store.get(key).decode()
        return LEFT if val == LEFT else int(val)

    def missing(self, step: int, timeout_s: float = 1.0, poll_s: float = 0.02) -> list:
        """Ranks (of those still counted alive) that do not take part in ``step``: they have not
        announced it within the time limit, or have left. They are dropped from ``alive``.

        Every survivor scans the store against its own deadline, so two survivors can see
        different things (a slow rank's announcement may land between their last polls). The scan
        is therefore only a proposal: the first survivor to finish publishes its member list for
        the step with an atomic compare-and-set, and everybody adopts that list, so that all
        survivors build the same sub-group afterwards. A rank that finds itself outside the
        adopted list raises :class:`ExcludedFromGroup`."""
        deadline = time.monotonic() + timeout_s
        behind = [r for r in self.alive if r != self.rank]
        while True:
            states = {r: self._state(r) for r in behind}
            behind = [r for r, st in states.items() if st == LEFT or st is None or st < step]
            only_leavers = all(states[r] == LEFT for r in behind)       # nobody left to wait for
            if not behind or only_leavers or time.monotonic() >= deadline:
                break
            time.sleep(poll_s)
        proposal = [r for r in self.alive if r not in behind]
        agreed = self._agree(step, proposal)
        gone = [r for r in self.alive if r not in agreed]
        self.alive = [r for r in self.alive if r in agreed]
        if self.rank not in agreed:
            raise ExcludedFromGroup(f"rank {self.rank} is not among the members agreed for step {step}: {agreed}")
        return gone

    def _agree(self, step: int, proposal: list) -> list:
        key = f"{self.prefix}/members/{int(step)}"
        mine = ",".join(str(r) for r in proposal)
        try:
            got = self.store.compare_set(key, "", mine)         # first writer wins; returns what is stored
            got = got.decode() if isinstance(got, bytes) else str(got)
        except (RuntimeError, NotImplementedError, AttributeError):
            return proposal                                     # a store without compare-and-set: local view
        return [int(x) for x in got.split(",") if x != ""] if got else proposal
