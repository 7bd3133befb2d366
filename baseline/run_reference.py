"""Reference arm of ``bench.py``: the unmodified reference (``baseline/_ref``) on the headline config.

Launched by ``bench.py --impl reference`` as a process of its own (one per GPU under torchrun), with
``sys.path`` pointing at the reference copy and at ``baseline/shims`` only; nothing of this
repository's package, kernels or runtime is importable here.

What runs is the reference's own stack, through its own entry points:

* planning: ``Dist_Attn_Config.from_bsa_config`` -> ``get_general_bsa_cc_optimal_schedule(...,
  gpu_tile_type='naive')`` (its row-owner allocation, ``search_algo/workload_partition.py:550-587``)
  -> ``Dependent_Graph`` -> ``Execution_Plan(plan_type='Flexflow')`` (its list scheduler,
  ``search_algo/execute_plan.py:637-720``). These are the reference's solver-free choices; its two
  integer programs need Gurobi, which cannot be had here. In the reference's own ablation ladder
  this plan is ``(w/o_gpu_tile,w/o_kernel_tile,Flexflow)``.
* execution: ``benchmark_orchestrate_bsa`` (``search_algo/benchmark.py:336-619``) sets up streams,
  one NCCL communicator per rank pair and the buffer carriers, and times forward and backward with
  the reference's own harness (one warm-up, 3 x 1 iterations, reported as ``reference_harness``);
  then the same prepared plans are stepped forward + backward K times through ``orchestrated_attn_func`` / ``orchestrated_attn_backward`` for the figure that is
  compared with this repository's (one step = one forward and one backward).
* kernels: stock flash-attn 2.8 through ``shims/flash_attn_25_api.py`` (the reference's fork of
  2.5.7 is not shipped with it); NCCL: the library PyTorch bundles, at the path the reference's
  ctypes binding computes.

Environment stand-ins, all outside the reference's files: OpenMPI-style rank variables derived
from torchrun's, a loop-back fallback for host-name resolution, ``gurobipy`` / ``pulp`` import-only
modules, an ``int()`` around the peer index the reference passes to ``ncclSend`` / ``ncclRecv`` as a
``numpy.bool`` (NumPy 2 no longer lets ctypes read one as an integer), the machine-profile directory ``logs/m_configs`` the reference copies into its database
(filled with the reference's own H800 kernel profile and link curves).
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import pickle
import shutil
import socket
import statistics
import subprocess
import sys
import threading
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")
METRIC = "cp_attn_fwd_bwd_ms_S512k_strided"
S_TOTAL, N_BLOCKS, N_HEADS, HEAD_DIM = 512 * 1024, 32, 32, 128


def _clean_sys_path() -> None:
    repo_root = os.path.dirname(HERE)
    keep = [p for p in sys.path if os.path.abspath(p or os.getcwd()) not in (repo_root, HERE)]
    # the reference's scripts are started as ``python search_algo/<script>.py``, so that directory is on its path too
    sys.path[:] = [REF, os.path.join(REF, "search_algo"), SHIMS] + keep


def _env_from_torchrun() -> tuple[int, int, int]:
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # the reference reads its rank from SLURM or OpenMPI variables (search_algo/initialize.py:29-57)
    os.environ["OMPI_COMM_WORLD_RANK"] = str(rank)
    os.environ["OMPI_COMM_WORLD_LOCAL_RANK"] = str(local_rank)
    os.environ["OMPI_COMM_WORLD_SIZE"] = str(world)
    os.environ["OMPI_COMM_WORLD_LOCAL_SIZE"] = str(world)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("CLUSTER_NAME", "b200box")
    os.environ.setdefault("PLATFORM", "B200")
    os.environ.setdefault("TRACE_NAME", "refarm")
    # the reference's launcher sets this ("important for cc overlap", scripts/runtime/wrapper.sh:140)
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
    return rank, local_rank, world


def _patch_hostname_resolution() -> None:
    real = socket.gethostbyname

    def gethostbyname(name):
        try:
            return real(name)
        except OSError:
            return "127.0.0.1"
    socket.gethostbyname = gethostbyname


def _numpy2_peer_index_compat() -> None:
    """The reference computes the peer index of a two-rank communicator as ``self.rank <
    global_dst`` on numpy integers (orchestrated_attn/utils.py:308-334), i.e. a ``numpy.bool``, and
    hands it to a ctypes ``c_int`` parameter. NumPy 1.x let ctypes read that through ``__index__``;
    NumPy 2 (installed here) removed it. Convert at the call boundary, outside the reference's files."""
    from tests.distributed.device_communicators.pynccl import PyNcclCommunicator
    send, recv = PyNcclCommunicator.send, PyNcclCommunicator.recv

    def send_int(self, tensor, dst, stream=None):
        return send(self, tensor, int(dst), stream)

    def recv_int(self, tensor, src, stream=None):
        return recv(self, tensor, int(src), stream)
    PyNcclCommunicator.send, PyNcclCommunicator.recv = send_int, recv_int


def _provide_libnccl() -> str:
    """The reference's ctypes binding loads ``third_party/comm_test/third_party/nccl/build/lib/
    libnccl.so.2`` relative to its own file (pynccl_wrapper.py:210). Link PyTorch's bundled NCCL there."""
    want = os.path.join(REF, "third_party", "comm_test", "third_party", "nccl", "build", "lib", "libnccl.so.2")
    if os.path.exists(want):
        return want
    cands = []
    for p in sys.path:
        cands += glob.glob(os.path.join(p, "nvidia", "nccl", "lib", "libnccl.so.2"))
    if not cands:
        import torch
        cands = glob.glob(os.path.join(os.path.dirname(torch.__file__), "lib", "libnccl.so*"))
    if not cands:
        raise FileNotFoundError("no libnccl.so.2 in the Python environment")
    os.makedirs(os.path.dirname(want), exist_ok=True)
    tmp = f"{want}.{os.getpid()}"
    os.symlink(cands[0], tmp)
    os.replace(tmp, want)
    return want


def _provide_machine_profile(workdir: str) -> None:
    """``Prof_DB`` copies ``logs/m_configs`` (relative to the working directory) into its database on
    first use (search_algo/database.py:28,42): one ``time*.json`` and the two link logs."""
    dst = os.path.join(workdir, "logs", "m_configs")
    if os.path.isdir(dst):
        return
    os.makedirs(dst, exist_ok=True)
    fit = os.path.join(REF, "prof_data", "fit")
    for name in ("time_g40_m2_flash_all.json", "cb_8_g42_all.log", "cb_16_g42,44_all.log"):
        shutil.copy(os.path.join(fit, name), os.path.join(dst, name))


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def strided_block_table(n_blocks: int):
    """Query block i attends key block j iff j <= i and (i - j <= 1 or (i - j) % 4 == 0); diagonal
    blocks are causal, the others full (values of the reference's ``Block_Type``)."""
    import numpy as np
    from search_algo.utils import Block_Type
    t = np.full((n_blocks, n_blocks), Block_Type.EMPTY, dtype=object)
    for i in range(n_blocks):
        for j in range(i + 1):
            if i - j <= 1 or (i - j) % 4 == 0:
                t[i, j] = Block_Type.CAUSAL if i == j else Block_Type.FULL
    return t


def make_plans(world: int, seq: int, prof_db, rank: int, gloo_group):
    """Forward and backward intra-node plans of the reference for the strided table on ``world``
    ranks. Rank 0 plans and pickles them into the reference's database directory (as its campaign
    does, search_algo/task1_bsa.py:174-186); every rank then loads the pickles."""
    import torch
    from search_algo.bsa_config import BSA_Repr, BSA_Config
    from search_algo.search_engine import Dist_Attn_Config, Evaluation_Configs
    from search_algo.dependent_graph import Dependent_Graph
    from search_algo.execute_plan import Execution_Plan
    from search_algo.task1_bsa import get_general_bsa_cc_optimal_schedule

    bsa_repr = BSA_Repr(block_table=strided_block_table(N_BLOCKS), cmap=None)
    bsa_config = BSA_Config(None, None, {"bsa_repr": bsa_repr, "CP": (world, 1)})
    shape_config = {"Nh": (N_HEADS, N_HEADS), "S": (seq, seq), "bs": 1, "D": HEAD_DIM}
    da_config = Dist_Attn_Config.from_bsa_config(bsa_config, shape_config=shape_config, hierarchy=1)
    out = []
    for fob in (0, 1):
        exp_config = Evaluation_Configs(plan_type="Flexflow", MAX_QUEUE_SIZE=100, fob=fob, hierarchy=1,
                                        transform_mode="greedy")
        path = os.path.join(prof_db.INTRA_BSA_EXE_PLANS_DIR, f"refarm_w{world}_S{seq}_fob{fob}.pkl")
        if rank == 0:
            schedule = get_general_bsa_cc_optimal_schedule(exp_config, da_config, prof_db, gpu_tile_type="naive")
            d_graph = Dependent_Graph(schedule, fob)
            plan = Execution_Plan(d_graph, fob, plan_type="Flexflow")
            with open(path + ".tmp", "wb") as f:
                pickle.dump(plan, f)
            os.replace(path + ".tmp", path)
        torch.distributed.barrier(gloo_group)
        with open(path, "rb") as f:
            plan = pickle.load(f)
        out.append((exp_config, plan))
    return da_config, bsa_repr, out


def run(args) -> dict:
    rank, local_rank, world = _env_from_torchrun()
    _patch_hostname_resolution()
    workdir = os.path.join(HERE, "_ref_work")
    if rank == 0:
        _provide_machine_profile(workdir)
        _provide_libnccl()
    os.makedirs(workdir, exist_ok=True)
    import torch
    assert torch.cuda.is_available(), "the reference's runtime needs CUDA devices"
    torch.cuda.set_device(local_rank)
    import flash_attn_25_api
    flash_attn_25_api.install()

    # rank 0 has to finish the file set-up before the others load libnccl through the reference
    marker = os.path.join(workdir, f".ready_{os.environ['MASTER_PORT']}")
    if rank == 0:
        open(marker, "w").close()
    else:
        t0 = time.time()
        while not os.path.exists(marker):
            if time.time() - t0 > 120:
                raise TimeoutError("rank 0 did not finish the reference arm's file set-up")
            time.sleep(0.1)
    os.chdir(workdir)

    from search_algo.initialize import initialize_distribution, initialize_prof_db
    from search_algo.benchmark import benchmark_orchestrate_bsa
    from search_algo.execute_plan import Execution_Plan
    from search_algo.utils import filter_kwargs, all_wait_main_stream, main_stream_wait_all
    from search_algo.global_vars import get_global_var as get_global_var_search
    from orchestrated_attn.global_vars import get_global_var as get_global_var_orch
    from orchestrated_attn.orchestrated_attn_impl import orchestrated_attn_func, orchestrated_attn_backward

    _numpy2_peer_index_compat()
    ncclcomm_global, gloo_group = initialize_distribution()
    if rank == 0 and os.path.exists(marker):
        os.remove(marker)
    prof_db = initialize_prof_db(gloo_group)
    da_config, bsa_repr, plans = make_plans(world, args.seq, prof_db, rank, gloo_group)
    dev = torch.device("cuda", local_rank)

    # One buffer for everything, sized as the reference's campaign sizes it (at least the 8 GiB its
    # start-gate all-reduce spans, search_algo/task1_bsa.py:707-714), filled with N(0,1) values.
    sync_size = get_global_var_search("SYNC_SIZE")
    s_gpu = max(da_config.S_per_gpu)
    need = (1 * s_gpu * N_HEADS * HEAD_DIM * 4) * 3
    n_elems = max(need, sync_size // 2)
    tensor_buf = torch.empty(n_elems, device=dev, dtype=torch.bfloat16)
    gen = torch.Generator(device=dev).manual_seed(1)
    chunk = 1 << 26
    for off in range(0, n_elems, chunk):
        n = min(chunk, n_elems - off)
        tensor_buf[off:off + n] = torch.randn(n, generator=gen, dtype=torch.float32, device=dev).to(torch.bfloat16)
    torch.cuda.synchronize()

    class _Args:
        profiler_with_tensorboard = False
        tb_dir = None
    PROC_INFO = get_global_var_search("PROC_INFO")
    node_id = PROC_INFO["nodeid"]
    warmup = max(args.warmup, 3)

    # ---- 1. the reference's own harness: forward and backward timed separately ------------------
    stock, prepared = {}, []
    for exp_config, plan in plans:
        inter_plan = Execution_Plan.create_one_node_exe_plan(exp_config.fob)
        comp_plans = {((1, 1), str(bsa_repr)): plan}
        inter_plan.gpu_kernel_lists[node_id][0].execution_plan = plan
        res = benchmark_orchestrate_bsa(
            _Args(), orchestrated_attn_func, da_config, exp_config, tensor_buf,
            inter_bsa_execution_plans=[inter_plan], inter_comp_plans_dicts=[comp_plans],
            global_group=gloo_group, ncclcomm_global=ncclcomm_global,
            warmup=1, num_iter=1, log=(rank == 0), use_cudagraph=False)
        if rank == 0:
            stock["fwd_s" if exp_config.fob == 0 else "bwd_s"] = float(res[0]["time"])
        prepared.append((exp_config, inter_plan, comp_plans))

    # ---- 2. forward + backward per step, K steps in one timed region ---------------------------
    streams = get_global_var_orch("streams")
    main_stream = streams["intra"][0]
    stream_list = streams["intra"] + streams["inter"]
    calls = []
    for exp_config, inter_plan, comp_plans in prepared:
        f = orchestrated_attn_func if exp_config.fob == 0 else orchestrated_attn_backward
        inputs = {
            "inp_row": inter_plan.buf_dict["inp_row"], "inp_col": inter_plan.buf_dict["inp_col"],
            # diagonal blocks of the strided pattern are causal; the reference's harness passes None here,
            # which runs them as full blocks (search_algo/benchmark.py:393)
            "dropout_p": 0, "causal": True, "deterministic": False,
            "sm_scale": HEAD_DIM ** -0.5, "softmax_scale": HEAD_DIM ** -0.5, "PROC_INFO": PROC_INFO,
            "extra_dict": {"da_config": da_config, "exp_configs": exp_config},
            "execution_plan_dict": {"inter": inter_plan, "intra": comp_plans},
        }
        calls.append((f, filter_kwargs(f, inputs)))

    def step():
        with torch.no_grad():
            for f, kw in calls:
                all_wait_main_stream(stream_list, main_stream)
                f(**kw)
                main_stream_wait_all(stream_list, main_stream)

    def barrier():
        torch.cuda.synchronize()
        torch.distributed.barrier(gloo_group)
        torch.cuda.synchronize()

    def timed(fn, steps, warm):
        with torch.cuda.stream(main_stream):
            for _ in range(warm):
                fn()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(main_stream)
            for _ in range(steps):
                fn()
            e1.record(main_stream)
            barrier()
        t = torch.tensor(e0.elapsed_time(e1) / steps)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=gloo_group)
        return t.item()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(step, args.steps, warmup)
    clocks = sampler.stop() if rank == 0 else None

    # ---- 3. end to end: every step copies this rank's Q/K/V/dO shards from pinned host memory into
    # device memory (same bytes as this repository's arm), steps, and reads a scalar back ----------
    e2e = None
    if not args.no_e2e:
        s_loc = args.seq // world
        shard = s_loc * N_HEADS * HEAD_DIM
        host = []
        for i in range(4):
            h = torch.empty(shard, dtype=torch.bfloat16, pin_memory=True)
            h.copy_(tensor_buf[i * shard:(i + 1) * shard])
            host.append(h)
        # the copies land at the start of the reference's buffer, where every tile's inputs live
        stage = tensor_buf[:4 * shard]
        result = {}

        def step_e2e():
            with torch.cuda.stream(main_stream):
                for i, h in enumerate(host):
                    stage[i * shard:(i + 1) * shard].copy_(h, non_blocking=True)
                step()
                result["v"] = float(tensor_buf[:64].float().sum().cpu())
        e2e_ms = timed(step_e2e, max(1, min(args.steps, 3)), 3)
        e2e = {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": 4 * shard * 2, "d2h_bytes_per_step": 4}

    n_comp = sum(1 for _, plan in plans for k in plan.gpu_kernel_lists[local_rank] if type(k).__name__ == "Comp_Kernel")
    return {
        "impl": "reference", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic N(0,1), seed 1 (the reference's runtime aliases every tile onto one buffer)",
        "config": {"model": "attention-only (Llama2-7B attention shape: 32 heads x 128)",
                   "pattern": "strided: 32 blocks of 16k, j<=i and (i-j<=1 or (i-j)%4==0)",
                   "global_batch": 1, "seq_len": args.seq, "parallelism": f"cp{world}-reference-orchestrated",
                   "reference_plan": "(w/o_gpu_tile,w/o_kernel_tile,Flexflow): row-owner allocation + list scheduler "
                                     "(the reference's solver-free choices; its ILPs need Gurobi)",
                   "kernels": "stock flash-attn 2.8 behind the 2.5 private API; NCCL bundled with PyTorch",
                   "l2": "each tile's Q/K/V (128 + 256 MiB) exceed the 126 MB L2; no flush needed"},
        "reference_harness": stock, "clocks": clocks, "e2e": e2e,
        "gpu_launches": n_comp * args.steps,
        "tokens_per_s": args.seq / (ms * 1e-3) if ms else None,
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seq", type=int, default=S_TOTAL)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--time-limit", type=int, default=int(os.environ.get("UA_REFERENCE_TIME_LIMIT", "1500")),
                    help="seconds after which the arm gives up (a rank that failed leaves the others in a "
                         "collective); default from UA_REFERENCE_TIME_LIMIT")
    args, _ = ap.parse_known_args()
    _clean_sys_path()
    rank = int(os.environ.get("RANK", "0"))

    def give_up():
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              f"the reference's run did not finish within {args.time_limit} s"}), flush=True)
        os._exit(0)
    watchdog = threading.Timer(args.time_limit, give_up)
    watchdog.daemon = True
    watchdog.start()
    try:
        line = run(args)
    except BaseException as e:  # noqa: BLE001  (the arm must always print one line and exit 0)
        if isinstance(e, KeyboardInterrupt):
            raise
        tb = traceback.extract_tb(e.__traceback__)
        where = f"{os.path.relpath(tb[-1].filename, HERE)}:{tb[-1].lineno}" if tb else "?"
        line = {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]} (at {where})"}
        traceback.print_exc(file=sys.stderr)
    if rank == 0:
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
