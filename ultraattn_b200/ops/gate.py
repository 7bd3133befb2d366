"""A start gate: hold a CUDA stream at a bounded device-side wait until the host says go.

The reference lines its ranks up before every timed region by launching an 8 GiB NCCL all-reduce
(``placeholder_op``, search_algo/benchmark.py:593-594): while the GPUs chew on it the CPU runs
ahead and queues the kernels to be measured, so their launch latency does not show in the timing.
Here a one-thread kernel polls a word of pinned host memory; everything queued behind it on the
stream waits; ``open()`` is a plain host store. Nothing on the GPU has to run for the gate to open
(the waiting kernel does not depend on another launch being resident), and the wait is bounded: if
the host never opens the gate the kernel gives up after ``budget_s``, records that in the device's
status word and the stream runs on.
"""
from __future__ import annotations

import torch

from .. import _lib
from . import attention as A

_GATE_WHERE = 950          # "where" code that the flag-wait kernel writes into the status word


class StartGate:
    def __init__(self, device, budget_s: float = 2.0):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.budget_s = budget_s
        self.epoch = 0
        self.timed_out = False
        # pinned host memory is mapped into the device's address space at the same address
        self.flag = torch.zeros(1, dtype=torch.int32)
        if self.cuda:
            self.flag = self.flag.pin_memory()

    def close(self, stream=None) -> None:
        """Queue the wait on ``stream`` (default: the current stream of the device)."""
        self.epoch += 1
        if not self.cuda:
            return
        stream = stream or torch.cuda.current_stream(self.device)
        rc = _lib.load().ua_wait_flag(self.flag.data_ptr(), self.epoch, self.budget_s,
                                      A.status_buffer(self.device).data_ptr(), stream.cuda_stream)
        _lib.check(rc, "ua_wait_flag")

    def open(self) -> None:
        self.flag[0] = self.epoch

    def check(self) -> bool:
        """After a synchronisation: True if the gate was opened in time. A gate that ran into its
        time limit is not an error of the kernels behind it, so its status entry is cleared here
        (``timed_out`` remembers it); any other status entry is left for ``check_status``."""
        if not self.cuda:
            return True
        st = A.status_buffer(self.device)
        host = st.cpu().tolist()
        if host[0] != 0 and host[1] == _GATE_WHERE:
            st.zero_()
            self.timed_out = True
            return False
        return True
