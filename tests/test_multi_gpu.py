"""Context-parallel attention on 2+ real GPUs: the fused peer-memory path and the NCCL baseline
against the dense oracle, plus the bounded-wait time-out path of the device-side flag wait.
Skipped when fewer than two GPUs are visible."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.ops import attention as A
        from ultraattn_b200.runtime import ContextParallelAttention
        pattern = getattr(P, case["pattern"])(*case["args"])
        S, H = case["S"], case["H"]
        rt = ContextParallelAttention(pattern, S, H, 128, device=dev, path=case["path"],
                                      allocation=case.get("allocation", "ilp"), plan_time_limit=5.0,
                                      nvls_min_consumers=case.get("nvls_min_consumers", 2),
                                      nvls_reduce=case.get("nvls_reduce"))
        if case.get("nvls_min_consumers", 2) == 1 and not rt.impl.bc_cols:
            ret[rank] = {"skip": "no NVSwitch multicast address for symmetric memory on this machine"}
            return
        g = torch.Generator().manual_seed(0)
        q, k, v, d_o = (torch.randn(1, S, H, 128, generator=g).to(torch.bfloat16) for _ in range(4))
        par_d = rt.table.shape[0]
        blk = S // par_d
        mine = [b for b in range(par_d) if rt.cmap[b] == rank]
        idx = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in mine])
        ql, kl, vl, dol = (t[:, idx].contiguous().to(dev) for t in (q, k, v, d_o))
        worst = 0.0
        for it in range(2):          # twice: flags, epochs and accumulators must survive reuse
            o, lse = rt.forward(ql, kl, vl)
            dq, dk, dv = rt.backward(dol, ql, kl, vl, o, lse)
            torch.cuda.synchronize()
            A.check_status(dev)
            o_ref, lse_ref, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(
                q.float(), k.float(), v.float(), d_o.float(), pattern)
            for got, ref in ((o, o_ref), (dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
                err = (got.float().cpu() - ref[:, idx]).abs().max().item()
                worst = max(worst, err / (ref.abs().max().item() + 1e-6))
        ret[rank] = {"rel_err": worst}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def _run(world, case):
    port = 29700 + os.getpid() % 200
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, case, ret), nprocs=world, join=True)
    return dict(ret)


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("path", ["fused", "nccl"])
@pytest.mark.parametrize("pattern,args,alloc", [
    ("causal", (1,), "ilp"), ("strided", (8, 4, 2), "ilp"), ("global_local", (8, 1, 2), "naive"),
], ids=["causal", "strided", "global_local"])
def test_context_parallel_2gpu(path, pattern, args, alloc):
    _need(2)
    res = _run(2, {"pattern": pattern, "args": args, "S": 2048, "H": 2, "path": path, "allocation": alloc})
    for r in range(2):
        assert "error" not in res[r], res[r].get("error")
        assert res[r]["rel_err"] < 2e-2, res


def test_context_parallel_2gpu_multicast_blocks():
    """Remote key/value blocks arrive by one multimem store from their owner (forced on for two
    ranks; by default only blocks with at least two consumers are broadcast)."""
    _need(2)
    res = _run(2, {"pattern": "global_local", "args": (8, 1, 2), "S": 2048, "H": 2, "path": "fused",
                   "allocation": "naive", "nvls_min_consumers": 1})
    if any("skip" in res[r] for r in range(2)):
        pytest.skip(res[0].get("skip") or res[1].get("skip"))
    for r in range(2):
        assert "error" not in res[r], res[r].get("error")
        assert res[r]["rel_err"] < 2e-2, res


@pytest.mark.skipif(os.environ.get("UA_TEST_NVLS_REDUCE") != "1",
                    reason="opt-in (UA_TEST_NVLS_REDUCE=1): the in-switch gradient sum is off by default")
def test_context_parallel_2gpu_in_switch_gradient_sum():
    """dK/dV of broadcast blocks summed by multimem.ld_reduce (own-replica accumulation): same
    results as the default delivery by peer reductions."""
    _need(2)
    res = _run(2, {"pattern": "global_local", "args": (8, 1, 2), "S": 2048, "H": 2, "path": "fused",
                   "allocation": "naive", "nvls_min_consumers": 1, "nvls_reduce": True})
    if any("skip" in res[r] for r in range(2)):
        pytest.skip(res[0].get("skip") or res[1].get("skip"))
    for r in range(2):
        assert "error" not in res[r], res[r].get("error")
        assert res[r]["rel_err"] < 2e-2, res


def _nvls_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from ultraattn_b200.ops import attention as A
        from ultraattn_b200.ops import elementwise as E
        from ultraattn_b200.runtime.fused import SymmMemSpace
        sp = SymmMemSpace(dist.group.WORLD, dev)
        n = 1 << 20
        sp.alloc("x", (n,), torch.float32)
        sp.alloc("h", (n,), torch.bfloat16)
        sp.finalize()
        if not sp.has_multicast():
            ret[rank] = {"skip": "no NVSwitch multicast address for symmetric memory on this machine"}
            return
        g = torch.Generator().manual_seed(5)
        parts = [torch.randn(n, generator=g) for _ in range(world)]
        out = {}
        # broadcast: rank 1's data lands in every replica
        if rank == 1:
            sp.multicast_store("x", slice(None), parts[1].to(dev))
        sp.barrier(0)
        out["bcast"] = (sp.local("x").cpu() - parts[1]).abs().max().item()
        sp.barrier(1)
        # reduce: every rank holds a partial; rank 0 pulls the in-switch sum
        sp.local("x").copy_(parts[rank].to(dev))
        sp.local("h").copy_(parts[rank].to(dev).to(torch.bfloat16))
        sp.barrier(2)
        total = sum(parts)
        if rank == 0:
            dst = torch.empty(n, dtype=torch.float32, device=dev)
            E.multimem_reduce(sp.multicast_ptr("x"), dst, n * 4, torch.float32, dev)
            out["reduce"] = (dst.cpu() - total).abs().max().item()
            dsth = torch.empty(n, dtype=torch.bfloat16, device=dev)
            E.multimem_reduce(sp.multicast_ptr("h"), dsth, n * 2, torch.bfloat16, dev)
            ref = sum(p.to(torch.bfloat16).float() for p in parts)
            out["reduce_bf16"] = (dsth.float().cpu() - ref).abs().max().item() / ref.abs().max().item()
        sp.barrier(3)
        # one-shot all-reduce: each rank reduces its slice and stores the sum back into every replica
        sl = n // world
        off = rank * sl * 4
        E.multimem_reduce(sp.multicast_ptr("x") + off, None, sl * 4, torch.float32, dev,
                          mc_out=sp.multicast_ptr("x") + off)
        sp.barrier(4)
        out["allreduce"] = (sp.local("x").cpu() - total).abs().max().item()
        torch.cuda.synchronize()
        A.check_status(dev)
        ret[rank] = out
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def test_nvls_primitives_2gpu():
    """multimem.st broadcast, multimem.ld_reduce reduction (fp32 and bf16) and the one-shot
    all-reduce built from them, against sums computed on the host."""
    _need(2)
    port = 29500 + os.getpid() % 150
    ret = mp.Manager().dict()
    mp.spawn(_nvls_worker, args=(2, port, ret), nprocs=2, join=True)
    res = dict(ret)
    if any("skip" in res[r] for r in range(2)):
        pytest.skip(res[0].get("skip") or res[1].get("skip"))
    for r in range(2):
        assert "error" not in res[r], res[r].get("error")
        assert res[r]["bcast"] == 0.0 and res[r]["allreduce"] < 1e-5, res
    assert res[0]["reduce"] < 1e-5 and res[0]["reduce_bf16"] < 1e-2, res


def _llama_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        import math
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.models.llama import LlamaConfig, LlamaModel
        from ultraattn_b200.ops import attention as A
        from ultraattn_b200.runtime import ContextParallelAttention
        cfg = LlamaConfig(n_layers=2, hidden=256, n_heads=2, head_dim=128, ffn=512, vocab=1000)
        pat = P.global_local(4, 1, 2)
        S = 2048
        rt = ContextParallelAttention(pat, S, cfg.n_heads, 128, device=dev, path="fused", plan_time_limit=5.0)
        par_d = rt.table.shape[0]
        blk = S // par_d
        pos = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in range(par_d) if rt.cmap[b] == rank])
        g = torch.Generator().manual_seed(3)
        ids_all = torch.randint(0, cfg.vocab, (S + 1,), generator=g)
        ids, tgt, posd = ids_all[pos].to(dev), ids_all[pos + 1].to(dev), pos.to(dev)
        out = {}
        for name, nvls in (("nccl", False), ("nvls", None)):
            m = LlamaModel(cfg, device=dev, pattern=pat, runtime=rt, group=dist.group.WORLD, seed=0,
                           nvls_optimizer=nvls)
            out[name] = [m.train_step(ids, tgt, posd, n_total_tokens=S) for _ in range(3)]
            out[name + "_used_nvls"] = m.space is not None
        torch.cuda.synchronize()
        A.check_status(dev)
        out["lnV"] = math.log(cfg.vocab)
        ret[rank] = out
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def test_llama_context_parallel_training_2gpu():
    """Three training steps of a small Llama over two GPUs (fused context-parallel attention,
    sharded Adam): the first loss is ln(vocab), the losses fall, and the optimizer that sums
    gradients inside the switch (when the machine has multicast) tracks the NCCL one."""
    _need(2)
    port = 29350 + os.getpid() % 100
    ret = mp.Manager().dict()
    mp.spawn(_llama_worker, args=(2, port, ret), nprocs=2, join=True)
    res = dict(ret)
    for r in range(2):
        assert "error" not in res[r], res[r].get("error")
        a, b = res[r]["nccl"], res[r]["nvls"]
        assert abs(a[0] - res[r]["lnV"]) < 0.3 and a[2] < a[0], res
        assert all(abs(x - y) < 2e-2 for x, y in zip(a, b)), res
    assert res[0]["nccl"] == res[1]["nccl"]


def _llama_ulysses_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.models.llama import LlamaConfig, LlamaModel
        from ultraattn_b200.ops import attention as A
        from ultraattn_b200.parallel.ulysses_fused import unpermute_qkv_weight
        from ultraattn_b200.runtime import ContextParallelAttention
        cfg = LlamaConfig(n_layers=2, hidden=256, n_heads=2, head_dim=128, ffn=512, vocab=1000)
        pat = P.global_local(4, 1, 2)
        S = 2048
        S_loc = S // world
        g = torch.Generator().manual_seed(3)
        ids_all = torch.randint(0, cfg.vocab, (S + 1,), generator=g)
        # head-parallel model: contiguous token ranges
        pos_u = torch.arange(rank * S_loc, (rank + 1) * S_loc)
        mu = LlamaModel(cfg, device=dev, pattern=pat, group=dist.group.WORLD, seed=0, nvls_optimizer=False,
                        seq_algo="ulysses", seq_len=S)
        assert mu.ulysses is not None
        # context-parallel model with the same weights (its wqkv rows in [q | k | v] order)
        rt = ContextParallelAttention(pat, S, cfg.n_heads, 128, device=dev, path="fused", plan_time_limit=5.0)
        blk = S // rt.table.shape[0]
        pos_c = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in range(rt.table.shape[0]) if rt.cmap[b] == rank])
        mc = LlamaModel(cfg, device=dev, pattern=pat, runtime=rt, group=dist.group.WORLD, seed=0, nvls_optimizer=False)
        with torch.no_grad():
            for li in range(cfg.n_layers):
                mc.p[f"l{li}.wqkv"].copy_(unpermute_qkv_weight(mu.p[f"l{li}.wqkv"], cfg.n_heads, cfg.kv_heads, 128, world))
            mc.master.copy_(mc.flat[rank * mc.shard:(rank + 1) * mc.shard].float())
        lu = [mu.train_step(ids_all[pos_u].to(dev), ids_all[pos_u + 1].to(dev), pos_u.to(dev), n_total_tokens=S) for _ in range(3)]
        lc = [mc.train_step(ids_all[pos_c].to(dev), ids_all[pos_c + 1].to(dev), pos_c.to(dev), n_total_tokens=S) for _ in range(3)]
        torch.cuda.synchronize()
        A.check_status(dev)
        ret[rank] = {"ulysses": lu, "cp": lc}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def test_llama_ulysses_training_matches_context_parallel_2gpu():
    """Three training steps with head-parallel attention (all-to-alls fused into the projection
    GEMMs, forward and backward) follow the context-parallel model started from the same weights."""
    _need(2)
    port = 29450 + os.getpid() % 100
    ret = mp.Manager().dict()
    mp.spawn(_llama_ulysses_worker, args=(2, port, ret), nprocs=2, join=True)
    res = dict(ret)
    for r in range(2):
        assert "error" not in res[r], res[r].get("error")
        u, c = res[r]["ulysses"], res[r]["cp"]
        assert u[2] < u[0] and all(abs(a - b) < 3e-2 for a, b in zip(u, c)), res


def _campaign_worker(rank, world, port, root, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.drivers import report, task1
        from ultraattn_b200.drivers.exp_configs import ExpSpace
        from ultraattn_b200.ops import attention as A
        from ultraattn_b200.patterns.blocks import BSA_Config
        from ultraattn_b200.plandb import ABLATION_SUFFIXES, Prof_DB, plan_key_prefix
        cfg = BSA_Config(None, None, {"bsa_repr": P.star(4, 1), "CP": (2, 1)})
        space = ExpSpace("bsa_infer", [0], [cfg], [cfg], [8192], [4], D=128, S_per_gpu_bounds=(1, 1 << 20))
        db = Prof_DB("unit", "B200", root=root)
        work = task1.step1_generate_intra_bsa_exe_plans(space, db, time_limit=2.0)
        task1.step2_profile_intra_bsa_exe_plans(work, db, dev, world)
        dist.barrier()
        torch.cuda.synchronize()
        A.check_status(dev)
        shape = {"S": (8192, 8192), "Nh": (4, 4), "bs": 1, "D": 128}
        prefix = plan_key_prefix(0, (2, 1), shape, cfg)
        prof = [Prof_DB("unit", "B200", root=root).get_profile(prefix + s) for s in ABLATION_SUFFIXES]
        ok = all(p is not None and float(p["time"]) > 0 and float(p["hfu"]) > 0 for p in prof)
        rows = report.build_rows({prefix + s: p for s, p in zip(ABLATION_SUFFIXES, prof)})
        ret[rank] = {"ok": ok, "ultra": rows[0]["ultraattn"], "n_rows": len(rows)}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def test_planning_campaign_profiles_on_2gpu(tmp_path):
    """Plan generation, measurement of every plan variant with the NCCL executor on two GPUs, the
    profile database and the report table, end to end on a small star-attention prefill."""
    _need(2)
    port = 29250 + os.getpid() % 100
    ret = mp.Manager().dict()
    mp.spawn(_campaign_worker, args=(2, port, str(tmp_path), ret), nprocs=2, join=True)
    res = dict(ret)
    for r in range(2):
        assert "error" not in res[r], res[r].get("error")
        assert res[r]["ok"] and res[r]["n_rows"] == 1 and res[r]["ultra"] > 0, res


def test_context_parallel_4gpu_fused():
    _need(4)
    res = _run(4, {"pattern": "strided", "args": (8, 4, 2), "S": 4096, "H": 2, "path": "fused"})
    for r in range(4):
        assert "error" not in res[r], res[r].get("error")
        assert res[r]["rel_err"] < 2e-2, res


@pytest.mark.parametrize("path", ["fused", "nccl"])
@pytest.mark.parametrize("pattern,args", [("strided", (32, 4, 2)), ("global_local", (32, 1, 2))],
                         ids=["strided", "global_local"])
def test_context_parallel_8gpu(path, pattern, args):
    """The benchmark's block tables (32 blocks) on all eight GPUs of a box, two iterations."""
    _need(8)
    res = _run(8, {"pattern": pattern, "args": args, "S": 8192, "H": 2, "path": path})
    for r in range(8):
        assert "error" not in res[r], res[r].get("error")
        assert res[r]["rel_err"] < 2e-2, res


def _interleaved_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.ops import attention as A
        from ultraattn_b200.runtime import ContextParallelAttention
        pattern = P.strided(8, 4, 2)
        S, H = 2048, 2
        rt = ContextParallelAttention(pattern, S, H, 128, device=dev, path="fused", plan_time_limit=5.0)
        blk = S // rt.table.shape[0]
        idx = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in range(rt.table.shape[0]) if rt.cmap[b] == rank])
        data, outs, worst = {}, {}, 0.0
        for name, seed in (("A", 1), ("B", 2)):
            g = torch.Generator().manual_seed(seed)
            data[name] = [torch.randn(1, S, H, 128, generator=g).to(torch.bfloat16) for _ in range(4)]
            ql, kl, vl, _ = (t[:, idx].contiguous().to(dev) for t in data[name])
            outs[name] = (ql, kl, vl) + tuple(rt.forward(ql, kl, vl))
        for name in ("A", "B"):             # A's backward comes after B's forward
            ql, kl, vl, o, lse = outs[name]
            q, k, v, d_o = data[name]
            dq, dk, dv = rt.backward(d_o[:, idx].contiguous().to(dev), ql, kl, vl, o, lse)
            torch.cuda.synchronize()
            A.check_status(dev)
            _, _, dq_ref, dk_ref, dv_ref = P.dense_attention_with_grads(q.float(), k.float(), v.float(), d_o.float(), pattern)
            for got, ref in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
                worst = max(worst, (got.float().cpu() - ref[:, idx]).abs().max().item() / (ref.abs().max().item() + 1e-6))
        ret[rank] = {"rel_err": worst}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def test_backward_after_another_forward_2gpu():
    """fwd(A); fwd(B); bwd(A); bwd(B) on the fused path: A's backward must not reuse the peers'
    Q / K / V that B's forward left in the staging mirrors."""
    _need(2)
    port = 29700 + os.getpid() % 200
    ret = mp.Manager().dict()
    mp.spawn(_interleaved_worker, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        assert "error" not in ret[r], ret[r].get("error")
        assert ret[r]["rel_err"] < 2e-2, dict(ret)


def _ulysses_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.ops import attention as A
        from ultraattn_b200.parallel.ulysses_fused import FusedUlyssesAttention, permute_qkv_weight
        S, hidden, H = 1024, 512, 4
        g = torch.Generator().manual_seed(0)
        x = (torch.randn(S, hidden, generator=g) * 0.5).to(torch.bfloat16)
        wqkv = (torch.randn(3 * H * 128, hidden, generator=g) * 0.05).to(torch.bfloat16)
        wo = (torch.randn(hidden, H * 128, generator=g) * 0.05).to(torch.bfloat16)
        mod = FusedUlyssesAttention(dist.group.WORLD, dev, S, hidden, H)
        S_loc = S // world
        xl = x[rank * S_loc:(rank + 1) * S_loc].contiguous().to(dev)
        wp = permute_qkv_weight(wqkv, H, H, 128, world).to(dev)
        worst = 0.0
        for _ in range(2):
            y = mod.forward(xl, wp, wo.to(dev))
            torch.cuda.synchronize()
            A.check_status(dev)
            qkv = (x.float() @ wqkv.float().t()).to(torch.bfloat16).float()
            q, k, v = (qkv[:, i * H * 128:(i + 1) * H * 128].reshape(1, S, H, 128) for i in range(3))
            o, _ = P.dense_attention(q, k, v, P.causal(1).token_mask(S))
            y_ref = o.to(torch.bfloat16).float().reshape(S, H * 128) @ wo.float().t()
            err = (y.float().cpu() - y_ref[rank * S_loc:(rank + 1) * S_loc]).abs().max().item()
            worst = max(worst, err / (y_ref.abs().max().item() + 1e-6))
        ret[rank] = {"rel_err": worst}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def test_fused_ulysses_projections_2gpu():
    """QKV projection with the all-to-all in its epilogue and output projection with the
    all-to-all in its operand load, against the unfused computation."""
    _need(2)
    ret = mp.Manager().dict()
    mp.spawn(_ulysses_worker, args=(2, 29930 + os.getpid() % 50, ret), nprocs=2, join=True)
    for r in range(2):
        assert "error" not in ret[r], ret[r].get("error")
        assert ret[r]["rel_err"] < 3e-2, dict(ret)


def _ulysses_grad_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from ultraattn_b200 import patterns as P
        from ultraattn_b200.ops import attention as A, elementwise as E
        from ultraattn_b200.parallel.ulysses_fused import (FusedUlyssesAttention, permute_qkv_weight,
                                                            unpermute_qkv_weight, unfused_reference)
        S, hidden, H = 1024, 512, 4
        pattern = P.strided(8, 4, 2)
        g = torch.Generator().manual_seed(0)
        x = (torch.randn(S, hidden, generator=g) * 0.5).to(torch.bfloat16)
        wqkv = (torch.randn(3 * H * 128, hidden, generator=g) * 0.05).to(torch.bfloat16)
        wo = (torch.randn(hidden, H * 128, generator=g) * 0.05).to(torch.bfloat16)
        dy = (torch.randn(S, hidden, generator=g) * 0.5).to(torch.bfloat16)
        cos, sin = E.rope_tables(S, 128, 10000.0, dev)
        mod = FusedUlyssesAttention(dist.group.WORLD, dev, S, hidden, H, pattern=pattern)
        S_loc = S // world
        sl = slice(rank * S_loc, (rank + 1) * S_loc)
        wp = permute_qkv_weight(wqkv, H, H, 128, world)
        assert torch.equal(unpermute_qkv_weight(wp, H, H, 128, world), wqkv)
        res = {}
        for name in ("fused", "unfused"):
            xl = x[sl].contiguous().to(dev).requires_grad_()
            w1 = wp.to(dev).requires_grad_()
            w2 = wo.to(dev).requires_grad_()
            for _ in range(2):                    # twice: buffers and barriers must survive reuse
                for t in (xl, w1, w2):
                    t.grad = None
                if name == "fused":
                    y = mod(xl, w1, w2, cos, sin)
                else:
                    y = unfused_reference(xl, w1, w2, dist.group.WORLD, H, H, 128, pattern, cos, sin)
                y.backward(dy[sl].to(dev))
                torch.cuda.synchronize()
                A.check_status(dev)
            # weight gradients of the ranks add up (every rank saw its own tokens)
            gw1, gw2 = w1.grad.float(), w2.grad.float()
            dist.all_reduce(gw1)
            dist.all_reduce(gw2)
            res[name] = (y.detach().float().cpu(), xl.grad.float().cpu(), gw1.cpu(), gw2.cpu())
        # CPU fp32 autograd of the same block on the whole sequence
        xf = x.float().requires_grad_()
        wq = wqkv.float().requires_grad_()
        wof = wo.float().requires_grad_()
        qkv = xf @ wq.t()
        q, k, v = (qkv[:, i * H * 128:(i + 1) * H * 128].reshape(S, H, 128) for i in range(3))
        pos = torch.arange(S)
        rot = lambda t: torch.cat([t[..., :64] * cos.cpu()[pos][:, None] - t[..., 64:] * sin.cpu()[pos][:, None],
                                   t[..., 64:] * cos.cpu()[pos][:, None] + t[..., :64] * sin.cpu()[pos][:, None]], -1)
        o, _ = P.dense_attention(rot(q)[None], rot(k)[None], v[None], pattern.token_mask(S))
        yf = o[0].reshape(S, H * 128) @ wof.t()
        yf.backward(dy.float())
        oracle = (yf.detach()[sl], xf.grad[sl], permute_qkv_weight(wq.grad, H, H, 128, world), wof.grad)
        rel = lambda a, b: (a - b).abs().max().item() / (b.abs().max().item() + 1e-6)
        ret[rank] = {"fused_vs_unfused": max(rel(a, b) for a, b in zip(res["fused"], res["unfused"])),
                     "fused_vs_oracle": max(rel(a, b) for a, b in zip(res["fused"], oracle))}
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def test_fused_ulysses_backward_2gpu():
    """Gradients of the head-parallel block through the fused projections (dO scattered by the
    dy @ Wo GEMM, dQKV gathered by the dx GEMM, weight gradients from peer operands) against the
    same block with plain GEMMs + all_to_all, and against fp32 autograd on the whole sequence."""
    _need(2)
    ret = mp.Manager().dict()
    mp.spawn(_ulysses_grad_worker, args=(2, 29880 + os.getpid() % 50, ret), nprocs=2, join=True)
    for r in range(2):
        assert "error" not in ret[r], ret[r].get("error")
        assert ret[r]["fused_vs_unfused"] < 3e-2 and ret[r]["fused_vs_oracle"] < 4e-2, dict(ret)


def test_flag_wait_times_out_cleanly():
    """A device-side wait on a flag that nothing sets gives up after its budget, records an error
    code in the status word and leaves the context usable (no trap, no hang)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from ultraattn_b200 import _lib
    from ultraattn_b200.ops import attention as A
    dev = torch.device("cuda", 0)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    st = A.status_buffer(dev)
    st.zero_()
    rc = _lib.load().ua_wait_flag(flag.data_ptr(), 1, 0.2, st.data_ptr(),
                                  torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "ua_wait_flag")
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="code=2"):
        A.check_status(dev)
    x = torch.ones(4, device=dev) * 2        # the context still works
    assert x.sum().item() == 8
    flag.fill_(1)                            # and a satisfied wait returns without error
    rc = _lib.load().ua_wait_flag(flag.data_ptr(), 1, 0.2, st.data_ptr(),
                                  torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize()
    A.check_status(dev)


def _grid_varlen_worker(rank, world, port, ret):
    """Kernel-tile grid executor (NCCL collectives around one launch) and the packed
    variable-length zigzag ring on real GPUs, against the dense oracle."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from ultraattn_b200 import parallel as PL, patterns as P
        from ultraattn_b200.ops import attention as A
        from ultraattn_b200.runtime import GridExecutor
        S, H = 2048, 2
        g = torch.Generator().manual_seed(21)
        q, k, v, d_o = (torch.randn(1, S, H, 128, generator=g).to(torch.bfloat16) for _ in range(4))
        sl = slice(rank * S // world, (rank + 1) * S // world)
        ql, kl, vl, dol = (t[:, sl].contiguous().to(dev) for t in (q, k, v, d_o))
        out = {}
        for name, (Y, X, causal) in {"grid_1x2_causal": (1, 2, True), "grid_2x1_full": (2, 1, False)}.items():
            ex = GridExecutor(Y, X, device=dev, causal=causal)
            o, lse = ex.forward(ql, kl, vl)
            dq, dk, dv = ex.backward(dol, ql, kl, vl, o, lse)
            torch.cuda.synchronize()
            A.check_status(dev)
            ref = P.dense_attention_with_grads(q.float(), k.float(), v.float(), d_o.float(),
                                               P.causal(1) if causal else P.full(1))
            worst = 0.0
            for got, r in ((o, ref[0]), (dq, ref[2]), (dk, ref[3]), (dv, ref[4])):
                worst = max(worst, (got.float().cpu() - r[:, sl]).abs().max().item() / (r.abs().max().item() + 1e-6))
            out[name] = worst
        # packed batch of two sequences, zigzag shards, causal
        cu = [0, 1024, 1536]
        qp, kp, vp, dop = (t[0, :cu[-1]] for t in (q, k, v, d_o))
        sh = lambda t: PL.shard_packed(t, cu, rank, world, "zigzag")[0]
        local_cu = PL.shard_packed(qp, cu, rank, world, "zigzag")[1]
        qz, kz, vz = (sh(t).to(dev).requires_grad_() for t in (qp, kp, vp))
        oz = PL.zigzag_ring_flash_attn_varlen_func(qz, kz, vz, local_cu, None, causal=True)
        oz.backward(sh(dop).to(dev))
        torch.cuda.synchronize()
        A.check_status(dev)
        worst = 0.0
        refs = [P.dense_attention_with_grads(*(t[None, a:b].float() for t in (qp, kp, vp, dop)), P.causal(1))
                for a, b in zip(cu[:-1], cu[1:])]
        for got, i in ((oz, 0), (qz.grad, 2), (kz.grad, 3), (vz.grad, 4)):
            r = torch.cat([x[i][0] for x in refs], dim=0)
            worst = max(worst, (got.float().cpu() - sh(r)).abs().max().item() / (r.abs().max().item() + 1e-6))
        out["zigzag_varlen"] = worst
        ret[rank] = out
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = {"error": f"{type(e).__name__}: {e}\n{traceback.format_exc()}"}
    finally:
        dist.destroy_process_group()


def test_grid_executor_and_varlen_ring_2gpu():
    _need(2)
    port = 29300 + os.getpid() % 200
    ret = mp.Manager().dict()
    mp.spawn(_grid_varlen_worker, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        assert "error" not in ret[r], ret[r].get("error")
        for name, err in ret[r].items():
            assert err < 2e-2, (r, name, err)
