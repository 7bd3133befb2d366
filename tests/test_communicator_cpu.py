"""Explicit-stream communicators and their registry on gloo CPU ranks."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ultraattn_b200.parallel.communicator import (CommRegistry, IntraComm, IntraComm_fused,
                                                          PyNcclCommunicator, StreamCommunicator)
        assert PyNcclCommunicator is StreamCommunicator
        reg = CommRegistry().create([tuple(range(world))]).for_pairs(range(world)).for_grid(range(world), X=2)
        wc = reg[tuple(range(world))]
        assert wc.rank == rank and wc.world_size == world
        # collectives
        t = torch.full((4,), float(rank + 1))
        wc.all_reduce(t)
        assert t.tolist() == [10.0] * 4
        out = torch.empty(world * 2)
        wc.all_gather(out, torch.full((2,), float(rank)))
        assert out.tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
        rs = torch.empty(1)
        wc.reduce_scatter(rs, torch.arange(world, dtype=torch.float32) * (rank + 1))
        assert rs.item() == rank * 10.0
        # a disabled communicator ignores the call
        with wc.change_state(enable=False):
            t2 = torch.ones(1)
            wc.all_reduce(t2)
            assert t2.item() == 1.0
        # pair communicators: ring exchange of carriers, batched so that nobody blocks
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        ic = IntraComm(reg)
        got = torch.empty(3)
        cs, cr = reg.pair(rank, nxt), reg.pair(rank, prv)
        if cs is cr:                        # world 2: one communicator carries both directions
            cs.group_start()
        ic.send(nxt, torch.full((3,), float(rank)))
        ic.recv(prv, got)
        if cs is cr:
            cs.group_end()
        cs.wait()
        cr.wait()
        assert got.tolist() == [float(prv)] * 3
        # Y x X = 2 x 2 grid: row group gathers, column group reduce-scatters
        fc = IntraComm_fused(reg, range(world), X=2)
        assert fc.groups["r"] == (rank // 2 * 2, rank // 2 * 2 + 1) and fc.groups["c"] == (rank % 2, rank % 2 + 2)
        row = torch.empty(2)
        fc.all_gather("r", row, torch.tensor([float(rank)]))
        assert row.tolist() == [float(rank // 2 * 2), float(rank // 2 * 2 + 1)]
        col = torch.empty(1)
        fc.reduce_scatter("c", col, torch.tensor([1.0, 2.0]) * (rank + 1))
        mates = fc.groups["c"]
        assert col.item() == sum(m + 1 for m in mates) * (1.0 if rank == mates[0] else 2.0)
        wc.barrier()
        ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
    finally:
        dist.destroy_process_group()


def test_stream_communicators_world4():
    port = 29500 + os.getpid() % 90
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(4, port, ret), nprocs=4, join=True)
    for r in range(4):
        assert ret[r] == "ok", ret[r]
