"""The ctypes NCCL binding (parallel/nccl_binding.py). What needs no GPU runs here on CPU: locating
and loading the library, the checked call path, unique ids, non-member communicators. The
collectives run on 2 GPUs as child processes (explicit side streams, against plain tensor math)."""
import os
import sys

import pytest
import torch

from ultraattn_b200.parallel import nccl_binding as NB

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_is_the_one_pytorch_ships():
    path = NB.find_nccl_library()
    assert "nccl" in os.path.basename(path)
    lib = NB.NcclLibrary()
    assert lib is NB.NcclLibrary()                       # one instance per path
    major, minor, _ = lib.version()
    assert (major, minor) >= (2, 18)


def test_errors_carry_nccl_text():
    lib = NB.NcclLibrary()
    assert lib.error_string(0) == "no error"
    with pytest.raises(NB.NcclError, match="invalid argument"):
        lib.check(4, "ncclFoo")
    lib.check(0, "ncclFoo")


def test_unique_ids_round_trip():
    lib = NB.NcclLibrary()
    a, b = lib.unique_id(), lib.unique_id()
    assert len(a) == NB.NCCL_UNIQUE_ID_BYTES and a != b
    uid = NB.NcclLibrary.unique_id_from_bytes(a)
    assert bytes(bytearray(uid.internal)) == a


def test_env_override_and_missing_library(monkeypatch):
    monkeypatch.setenv("UA_NCCL_LIBRARY", "/nonexistent/libnccl.so.2")
    assert NB.find_nccl_library() == "/nonexistent/libnccl.so.2"
    with pytest.raises(OSError):
        NB.NcclLibrary()


def test_non_member_is_disabled_and_every_dtype_is_mapped():
    comm = NB.NcclCommunicator([5, 7], "cpu")            # this process is rank 0: not a member
    assert comm.disabled and comm.rank == -1
    t = torch.ones(4)
    assert comm.all_reduce(t) is t and comm.async_error() is None
    comm.send(t, 1), comm.recv(t, 1)
    with comm.group():
        pass
    comm.destroy()
    for dt in (torch.bfloat16, torch.float16, torch.float32, torch.int32, torch.int64, torch.uint8):
        assert dt in NB.DTYPES
    assert NB.RED_OPS["sum"] == 0 and NB.RED_OPS["max"] == 2


def _worker(rank, world, port, ret, with_graph):
    # a child that stalls ends by itself with a traceback, and the steps it reached are on record
    import faulthandler
    faulthandler.dump_traceback_later(75, exit=True)
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    steps = []

    def reached(name):
        steps.append(name)
        ret[rank] = {"steps": list(steps)}

    try:
        comm = NB.NcclCommunicator(list(range(world)), dev, control_group=dist.group.WORLD, tag="t")
        assert comm.size_and_rank() == (world, rank)
        reached("init")
        side = torch.cuda.Stream(dev)
        peer = rank ^ 1
        x = torch.full((1 << 20,), float(rank + 1), device=dev, dtype=torch.bfloat16)
        y = torch.empty_like(x)
        torch.cuda.synchronize(dev)
        comm.exchange(x, y, peer, stream=side)
        side.synchronize()
        reached("exchange")
        s = torch.arange(world * 1024, device=dev, dtype=torch.float32) * (rank + 1)
        rs_out = torch.empty(1024, device=dev, dtype=torch.float32)
        rs_in = torch.ones(world * 1024, device=dev, dtype=torch.float32) * (rank + 1)
        ag = torch.empty(world * 8, device=dev, dtype=torch.int32)
        ag_in = torch.full((8,), rank, device=dev, dtype=torch.int32)
        b = torch.full((16,), float(rank), device=dev)
        torch.cuda.synchronize(dev)
        comm.all_reduce(s, stream=side)
        comm.reduce_scatter(rs_out, rs_in, stream=side)
        comm.all_gather(ag, ag_in, stream=side)
        comm.broadcast(b, src=world - 1, stream=side)
        side.synchronize()
        reached("collectives")
        tot = world * (world + 1) // 2
        ok = (bool((y == peer + 1).all()) and bool((s == torch.arange(world * 1024, device=dev) * tot).all())
              and bool((rs_out == tot).all()) and ag.view(world, 8)[:, 0].tolist() == list(range(world))
              and bool((b == world - 1).all()) and comm.async_error() is None)
        if with_graph:
            # the same exchange replayed from a CUDA graph (calls only enqueue on the given stream)
            graph = torch.cuda.CUDAGraph()
            y.zero_()
            torch.cuda.synchronize(dev)
            with torch.cuda.graph(graph, stream=side):
                comm.exchange(x, y, peer, stream=side)
            reached("captured")
            x.fill_(float(10 + rank))
            graph.replay()
            torch.cuda.synchronize(dev)
            reached("replayed")
            ok = ok and bool((y == 10 + peer).all())
            # NCCL keeps a communicator alive while a graph that captured its calls exists:
            # ncclCommDestroy would wait for the graph to go away
            del graph
            torch.cuda.synchronize(dev)
        dist.barrier()
        comm.destroy()
        ret[rank] = {"ok": ok, "steps": list(steps)}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}", "steps": list(steps)}
    finally:
        faulthandler.cancel_dump_traceback_later()
        dist.destroy_process_group()


def _run(with_graph):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    try:
        mp.spawn(_worker, args=(2, 29900 + os.getpid() % 90, ret, with_graph), nprocs=2, join=True)
    except Exception as e:  # noqa: BLE001  (a child that ended by its watchdog)
        pytest.fail(f"a rank stopped after {dict(ret)}: {e}")
    for r in range(2):
        assert "error" not in ret[r], ret[r].get("error")
        assert ret[r]["ok"], ret[r]


@pytest.mark.gpu
def test_collectives_on_explicit_streams_2gpu():
    _run(with_graph=False)


@pytest.mark.gpu
def test_exchange_replays_from_a_cuda_graph_2gpu():
    _run(with_graph=True)
