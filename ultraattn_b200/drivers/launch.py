"""Single-node launcher: one process per GPU with the rendezvous and NCCL settings this framework
expects, in place of the reference's shell wrappers (scripts/runtime/wrapper.sh, executor_bx.sh:
SLURM / mpirun front-ends that export CLUSTER_NAME / PLATFORM and pick NCCL variables).

    python -m ultraattn_b200.drivers.launch --gpus 8 [--port 29500] [--cluster NAME] [--platform B200]
           [--no-nvls] -- -m ultraattn_b200.drivers.task1 --exp-class bsa_train
    python -m ultraattn_b200.drivers.launch --gpus 8 -- bench.py --gpus 8

Everything after ``--`` goes to ``python`` in every rank. Uses ``torch.distributed.run`` with the
loop-back address (container host names need not resolve). Under SLURM or OpenMPI the ranks read
their topology from the scheduler's variables instead (``parallel/comm.py::get_proc_info``) and
this launcher is not needed.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys


def build_command(gpus: int, port: int, rest: list) -> list:
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
            "--master-addr", "127.0.0.1", "--master-port", str(port), *rest]


def build_env(base: dict, cluster: str | None, platform: str | None, no_nvls: bool) -> dict:
    env = dict(base)
    if cluster:
        env["CLUSTER_NAME"] = cluster
    if platform:
        env["PLATFORM"] = platform
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    if no_nvls:
        # in-switch reduction / multicast off in every library (failure-detection runs need this)
        env["NCCL_NVLS_ENABLE"] = "0"
        env["UA_NVLS"] = "0"
        env["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    return env


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--port", type=int, default=29500)
    ap.add_argument("--cluster", default=None)
    ap.add_argument("--platform", default=None)
    ap.add_argument("--no-nvls", action="store_true")
    ap.add_argument("--dry-run", action="store_true", help="print the command and exit")
    a = ap.parse_args(argv)
    if not rest:
        ap.error("nothing to launch: give the program after --")
    cmd = build_command(a.gpus, a.port, rest)
    env = build_env(os.environ, a.cluster, a.platform, a.no_nvls)
    if a.dry_run:
        print(" ".join(cmd))
        return 0
    return subprocess.call(cmd, env=env)


if __name__ == "__main__":
    sys.exit(main())
