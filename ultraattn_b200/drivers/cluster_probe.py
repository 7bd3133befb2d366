"""Cluster probes: run a command on a list of hosts and collect the answers, and poll the job
scheduler for free nodes (reference: cluster_profiler.py, an ssh fan-out of one command, and
cluster_profiler_2.py, an `sinfo` poller).

    python -m ultraattn_b200.drivers.cluster_probe --hosts node1,node2 -- nvidia-smi -L
    python -m ultraattn_b200.drivers.cluster_probe --gpus            # GPU inventory of this host
    python -m ultraattn_b200.drivers.cluster_probe --sinfo --partition gpu --every 30 --count 10

Hosts named ``localhost`` / ``127.0.0.1`` run the command directly; others go through ``ssh`` in
batch mode (no prompts). Everything here only reads: no clocks, power limits or modes are touched.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor

GPU_QUERY = "index,name,memory.total,memory.used,clocks.sm,clocks.max.sm,power.draw,power.limit"


def run_on_host(host: str, cmd: list, timeout: float = 60.0) -> dict:
    local = host in ("localhost", "127.0.0.1", "")
    argv = cmd if local else ["ssh", "-o", "BatchMode=yes", "-o", "ConnectTimeout=10", host, *cmd]
    t0 = time.time()
    try:
        r = subprocess.run(argv, capture_output=True, text=True, timeout=timeout)
        return {"host": host or "localhost", "rc": r.returncode, "stdout": r.stdout, "stderr": r.stderr,
                "seconds": time.time() - t0}
    except (OSError, subprocess.TimeoutExpired) as e:
        return {"host": host or "localhost", "rc": -1, "stdout": "", "stderr": f"{type(e).__name__}: {e}",
                "seconds": time.time() - t0}


def fan_out(hosts: list, cmd: list, timeout: float = 60.0) -> list:
    with ThreadPoolExecutor(max_workers=max(1, min(32, len(hosts)))) as ex:
        return list(ex.map(lambda h: run_on_host(h, cmd, timeout), hosts))


def gpu_inventory(hosts: list) -> list:
    """One record per GPU of every host (read-only nvidia-smi query)."""
    cmd = ["nvidia-smi", f"--query-gpu={GPU_QUERY}", "--format=csv,noheader,nounits"]
    out = []
    for res in fan_out(hosts, cmd):
        if res["rc"] != 0:
            out.append({"host": res["host"], "error": res["stderr"].strip() or f"rc={res['rc']}"})
            continue
        for line in res["stdout"].strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) == len(GPU_QUERY.split(",")):
                out.append(dict(zip(["host"] + GPU_QUERY.split(","), [res["host"]] + f)))
    return out


def parse_sinfo(text: str) -> list:
    """Rows of ``sinfo -h -o '%P %a %D %T'``: partition, availability, node count, state."""
    rows = []
    for line in text.strip().splitlines():
        f = line.split()
        if len(f) >= 4:
            rows.append({"partition": f[0].rstrip("*"), "avail": f[1], "nodes": int(f[2]), "state": f[3]})
    return rows


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("--hosts", default="localhost")
    ap.add_argument("--gpus", action="store_true", help="print the GPU inventory of the hosts")
    ap.add_argument("--sinfo", action="store_true", help="poll the scheduler for idle nodes")
    ap.add_argument("--partition", default=None)
    ap.add_argument("--every", type=float, default=30.0)
    ap.add_argument("--count", type=int, default=1)
    ap.add_argument("--timeout", type=float, default=60.0)
    a = ap.parse_args(argv)
    hosts = [h for h in a.hosts.split(",") if h]
    if a.gpus:
        for rec in gpu_inventory(hosts):
            print(json.dumps(rec))
        return 0
    if a.sinfo:
        for k in range(a.count):
            res = run_on_host("localhost", ["sinfo", "-h", "-o", "%P %a %D %T"], a.timeout)
            rows = parse_sinfo(res["stdout"]) if res["rc"] == 0 else []
            if a.partition:
                rows = [r for r in rows if r["partition"] == a.partition]
            idle = sum(r["nodes"] for r in rows if r["state"].startswith("idle"))
            print(json.dumps({"t": time.time(), "idle_nodes": idle, "rows": rows,
                              "error": None if res["rc"] == 0 else res["stderr"].strip()}))
            if k + 1 < a.count:
                time.sleep(a.every)
        return 0
    if not rest:
        ap.error("nothing to run: give the command after --")
    rc = 0
    for res in fan_out(hosts, rest, a.timeout):
        print(f"==== {res['host']} (rc={res['rc']}, {res['seconds']:.1f}s)")
        sys.stdout.write(res["stdout"])
        if res["stderr"]:
            sys.stderr.write(res["stderr"])
        rc = rc or res["rc"]
    return rc


if __name__ == "__main__":
    sys.exit(main())
