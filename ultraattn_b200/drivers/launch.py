"""Launchers: one process per GPU with the rendezvous, NCCL settings, CPU binding and logging this
framework expects, in place of the reference's shell wrappers (scripts/runtime/wrapper.sh,
wrapper_bx.sh, executor_bx.sh and scripts/schedule/*.sh).

    # one node, torchrun underneath (the default)
    python -m ultraattn_b200.drivers.launch --gpus 8 [--port 29500] [--cluster NAME] [--platform B200]
           [--no-nvls] [--exp-name NAME] -- -m ultraattn_b200.drivers.task1 --exp-class bsa_train
    python -m ultraattn_b200.drivers.launch --gpus 8 -- bench.py --gpus 8
    # several nodes under SLURM or OpenMPI: the scheduler starts the ranks, each rank runs the
    # per-rank executor (rank variables, NUMA binding, NIC selection) and then the program
    python -m ultraattn_b200.drivers.launch --launcher slurm --nodes 2 --gpus 8 --partition H800 -- bench.py
    python -m ultraattn_b200.drivers.launch --launcher mpirun --hosts g1:8,g2:8 -- bench.py

Everything after ``--`` goes to ``python`` in every rank. The local launcher uses
``torch.distributed.run`` with the loop-back address (container host names need not resolve).
``--exp-name`` copies the output to ``logs/<name>/output_<timestamp>.log`` as the reference's
wrappers do; ``--nsys`` prefixes every rank with an Nsight Systems command line (the tool itself
is not part of this package). ``--dry-run`` prints the command instead of running it.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import time


# -------------------------------------------------------------------------------------------------
# per-rank executor (reference: scripts/runtime/executor_bx.sh)
# -------------------------------------------------------------------------------------------------
def rank_env(env: dict) -> dict:
    """RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* from the scheduler's variables."""
    out = {}
    if "OMPI_COMM_WORLD_RANK" in env:
        out.update(RANK=env["OMPI_COMM_WORLD_RANK"], WORLD_SIZE=env["OMPI_COMM_WORLD_SIZE"],
                   LOCAL_RANK=env.get("OMPI_COMM_WORLD_LOCAL_RANK", "0"),
                   LOCAL_WORLD_SIZE=env.get("OMPI_COMM_WORLD_LOCAL_SIZE", env["OMPI_COMM_WORLD_SIZE"]))
    elif "SLURM_PROCID" in env:
        world = env.get("SLURM_NTASKS", env.get("SLURM_NPROCS", "1"))
        per_node = str(env.get("SLURM_NTASKS_PER_NODE", env.get("SLURM_TASKS_PER_NODE", world)))
        out.update(RANK=env["SLURM_PROCID"], WORLD_SIZE=world, LOCAL_RANK=env.get("SLURM_LOCALID", "0"),
                   LOCAL_WORLD_SIZE=per_node.split("(")[0].split(",")[0])
    else:
        out.update(RANK=env.get("RANK", "0"), WORLD_SIZE=env.get("WORLD_SIZE", "1"),
                   LOCAL_RANK=env.get("LOCAL_RANK", "0"), LOCAL_WORLD_SIZE=env.get("LOCAL_WORLD_SIZE", "1"))
    if "MASTER_ADDR" not in env:
        nodes = env.get("SLURM_STEP_NODELIST") or env.get("SLURM_JOB_NODELIST")
        # the first host of a plain comma list; a bracketed range needs `scontrol show hostnames`
        out["MASTER_ADDR"] = nodes.split(",")[0] if nodes and "[" not in nodes else "127.0.0.1"
    out.setdefault("MASTER_PORT", env.get("MASTER_PORT", "12215"))
    return out


def parse_cpulist(text: str) -> list:
    """'0-3,8,10-11' -> [0, 1, 2, 3, 8, 10, 11]."""
    cpus = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus += list(range(int(lo), int(hi or lo) + 1))
    return cpus


def numa_nodes(sys_root: str = "/sys/devices/system/node") -> list:
    """CPU lists of the NUMA nodes of this machine, in node order ([] when not exposed)."""
    out = []
    try:
        names = sorted((n for n in os.listdir(sys_root) if n.startswith("node") and n[4:].isdigit()),
                       key=lambda n: int(n[4:]))
        for n in names:
            with open(os.path.join(sys_root, n, "cpulist")) as f:
                out.append(parse_cpulist(f.read()))
    except OSError:
        return []
    return out


def cpus_for_local_rank(local_rank: int, local_world: int, nodes: list) -> list:
    """The cores a rank may use: ranks are spread over the NUMA nodes in order (the first half of
    the local ranks on node 0, ... as the reference binds them, executor_bx.sh:41-46) and the
    ranks of one node share that node's cores."""
    if not nodes:
        return []
    per_node = max(1, -(-local_world // len(nodes)))
    return nodes[min(local_rank // per_node, len(nodes) - 1)]


def rank_exec(rest: list, ib_hca: str | None, bind: bool, nsys_dir: str | None) -> int:
    """Set up this rank's environment and replace the process with the program."""
    env = dict(os.environ)
    env.update(rank_env(env))
    env.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")   # many streams must not share one queue
    if ib_hca:
        env["NCCL_IB_HCA"] = ib_hca
        env["NVSHMEM_HCA_LIST"] = ib_hca
    if bind and hasattr(os, "sched_setaffinity"):
        cpus = cpus_for_local_rank(int(env["LOCAL_RANK"]), int(env["LOCAL_WORLD_SIZE"]), numa_nodes())
        usable = set(cpus) & os.sched_getaffinity(0)
        if usable:
            os.sched_setaffinity(0, usable)
    cmd = [sys.executable, *rest]
    if nsys_dir:
        os.makedirs(nsys_dir, exist_ok=True)
        name = f"{env.get('TRACE_NAME', 'trace')}_w{env['WORLD_SIZE']}_r{env['RANK']}_{time.strftime('%Y%m%d-%H%M%S')}"
        cmd = ["nsys", "profile", "--trace=cuda,nvtx,osrt", f"--output={os.path.join(nsys_dir, name)}", *cmd]
    os.execvpe(cmd[0], cmd, env)
    return 0        # not reached


# -------------------------------------------------------------------------------------------------
# job-level commands
# -------------------------------------------------------------------------------------------------
def _rank_exec_args(a) -> list:
    out = [sys.executable, "-m", "ultraattn_b200.drivers.launch", "--rank-exec"]
    if a.ib_hca:
        out += ["--ib-hca", a.ib_hca]
    if a.no_bind:
        out += ["--no-bind"]
    if a.nsys:
        out += ["--nsys", a.nsys]
    return out + ["--"]


def build_slurm_command(a, rest: list) -> list:
    """``srun`` line (reference: scripts/runtime/wrapper_bx.sh:14-37): one task per GPU, the job
    is killed when any task fails (-K), CPU binding left to the per-rank executor."""
    cmd = ["srun", "-N", str(a.nodes), f"--ntasks-per-node={a.gpus}", f"--gres=gpu:{a.gpus}", "-K",
           "--cpu-bind", "none"]
    if a.partition:
        cmd += ["-p", a.partition]
    if a.hosts:
        cmd += ["-w", a.hosts]
    if a.cpus_per_task:
        cmd += [f"--cpus-per-task={a.cpus_per_task}"]
    return cmd + _rank_exec_args(a) + rest


def build_mpirun_command(a, rest: list) -> list:
    """``mpirun`` line (reference: scripts/runtime/wrapper.sh:158-171). ``--hosts`` is
    ``host:slots,host:slots``."""
    hosts = a.hosts or f"127.0.0.1:{a.gpus}"
    np_total = sum(int(h.split(":")[1]) if ":" in h else a.gpus for h in hosts.split(","))
    cmd = ["mpirun", "-np", str(np_total), "--host", hosts, "--bind-to", "none"]
    for var in ("MASTER_ADDR", "MASTER_PORT", "LD_LIBRARY_PATH", "PATH", "TRACE_NAME", "CLUSTER_NAME", "PLATFORM",
                "NCCL_DEBUG", "NCCL_NET_GDR_LEVEL", "NCCL_IB_DISABLE", "NCCL_NVLS_ENABLE", "UA_NVLS"):
        cmd += ["-x", var]
    return cmd + _rank_exec_args(a) + rest


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
    ap.add_argument("--launcher", default="local", choices=["local", "slurm", "mpirun"])
    ap.add_argument("--gpus", type=int, default=1, help="ranks per node")
    ap.add_argument("--nodes", type=int, default=1)
    ap.add_argument("--port", type=int, default=29500)
    ap.add_argument("--cluster", default=None)
    ap.add_argument("--platform", default=None)
    ap.add_argument("--partition", default=None, help="(slurm) partition")
    ap.add_argument("--hosts", default=None, help="(slurm) node list for -w; (mpirun) host:slots,...")
    ap.add_argument("--cpus-per-task", type=int, default=0)
    ap.add_argument("--ib-hca", default=None, help="NICs to use, e.g. mlx5_0,mlx5_1 (NCCL_IB_HCA)")
    ap.add_argument("--no-bind", action="store_true", help="leave CPU affinity alone")
    ap.add_argument("--nsys", default=None, metavar="DIR", help="profile every rank with Nsight Systems into DIR")
    ap.add_argument("--no-nvls", action="store_true")
    ap.add_argument("--exp-name", default=None, help="copy the output to logs/<name>/output_<timestamp>.log")
    ap.add_argument("--dry-run", action="store_true", help="print the command and exit")
    ap.add_argument("--rank-exec", action="store_true", help="(internal) set up one rank and exec the program")
    a = ap.parse_args(argv)
    if not rest:
        ap.error("nothing to launch: give the program after --")
    if a.rank_exec:
        return rank_exec(rest, a.ib_hca, not a.no_bind, a.nsys)
    if a.launcher == "slurm":
        cmd = build_slurm_command(a, rest)
    elif a.launcher == "mpirun":
        cmd = build_mpirun_command(a, rest)
    else:
        cmd = build_command(a.gpus, a.port, rest)
    env = build_env(os.environ, a.cluster, a.platform, a.no_nvls)
    if a.launcher != "local":
        env.setdefault("MASTER_PORT", str(a.port))
        env.setdefault("NCCL_NET_GDR_LEVEL", "5")
        env.setdefault("NCCL_IB_DISABLE", "0")
        env.setdefault("TRACE_NAME", env.get("CLUSTER_NAME", "trace"))
    if a.dry_run:
        print(" ".join(cmd))
        return 0
    if not a.exp_name:
        return subprocess.call(cmd, env=env)
    log_dir = os.path.join("logs", a.exp_name)
    os.makedirs(log_dir, exist_ok=True)
    path = os.path.join(log_dir, f"output_{time.strftime('%Y.%m.%d-%H:%M:%S')}.log")
    with open(path, "w") as log:
        proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        for line in proc.stdout:
            sys.stdout.write(line)
            log.write(line)
        return proc.wait()


if __name__ == "__main__":
    sys.exit(main())
