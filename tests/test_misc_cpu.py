"""Utilities, configuration, data carriers and model glue (CPU)."""
import os

import numpy as np
import pytest
import torch

from ultraattn_b200 import patterns as P


def test_reference_import_paths():
    import comm_lib.comm_utils
    import easy_context
    import head_parallel_attn
    import hierarchy_attn
    import orchestrated_attn
    import ring_flash_attn
    import search_algo.bsa_config as bc
    import search_algo.bsa_utils as bu
    import search_algo.execute_plan as ep
    import search_algo.search_engine as se
    import search_algo.utils as su
    from search_algo.dependent_graph import Comm_Kernel, Comp_Kernel, Dependent_Graph  # noqa: F401
    from search_algo.graph_transformation_engine import Graph_Transformation_Engine  # noqa: F401
    from search_algo.workload_partition import naive_allocate_strategy, solve_sparse_from_bsa  # noqa: F401
    r = bc.BSA_Repr(bu.create_bsa_block_table(2), None)
    cfg = bc.BSA_Config(None, None, {"bsa_repr": r, "CP": (4, 1)})
    assert su.Block_Type.CAUSAL.value == 2 and r.block_table_raw[1, 1] is su.Block_Type.CAUSAL
    assert cfg.to_string() == "CP=(4, 1)_repr=[[2000][1200][1020][1002]]"
    assert bu.bsa_is_causal(bc.BSA_Config.create_causal((2, 1))) and not bu.bsa_is_dense(cfg)
    assert hasattr(ep, "Execution_Plan") and hasattr(ep, "Fused_Execution_Plan") and hasattr(se, "Machine_Config")
    assert callable(orchestrated_attn.orchestrated_attn_func) and callable(ring_flash_attn.stripe_flash_attn_func)
    assert callable(head_parallel_attn.deepspeed_ulysses_attn_func) and callable(easy_context.prepare_seq_parallel_inputs)
    assert len(bu.split_to_node_configs(bc.BSA_Config(None, None, {"bsa_repr": P.causal(1), "CP": (4, 2)}))) == 3
    m = bu.get_b2f_suf_map(8)
    assert "_ablation=(w/o_kernel_tile,Y=4,X=2,dim=0)" in m["_ablation=(w/o_kernel_tile,ILP)"]


def test_utils():
    from ultraattn_b200.utils.misc import FinitePriorityQueue, calc_flops, get_block_table_type, unique_list
    q = FinitePriorityQueue(3)
    for x in [5, 1, 9, 3, 7, 2]:
        q.push(x)
    assert q.items() == [1, 2, 3]
    model, hw = calc_flops(1, 1024, 2, 128, causal=True, fob=1)
    assert hw == 1.25 * model and model == 2 * 4 * 1024 * 1024 * 2 * 128 * 0.5
    assert unique_list([1, 2, 1, 3, 2]) == [1, 2, 3]
    assert get_block_table_type(np.array([[1, 0]])).name == "PARTIAL"


def test_yaml_and_cli(tmp_path):
    from ultraattn_b200.drivers.arguments import parse_args
    cfg = parse_args(["--config", "configs/stream.yaml", "--Nhq", "8", "--exp-class", "bsa_infer"])
    assert cfg.SP == (1, 8) and cfg.Nhq == 8 and cfg.exp_class == "bsa_infer"
    assert cfg.pattern() == P.streaming(32, 1, 2)
    from ultraattn_b200.drivers.exp_configs import step0_top_down_decompose
    sp = step0_top_down_decompose("dense_train", max_intra=8, max_nodes=2, quick=True)
    assert any(c.CP == (8, 2) for c in sp.inter_bsa_configs) and sp.intra_bsa_configs
    assert all(s["S"][0] // 8 >= 256 for s in sp.shape_configs(8))


def test_carriers_reduce():
    from ultraattn_b200.ops.elementwise import lse_merge_reference
    from ultraattn_b200.runtime.orchestrated import Input_Row_Bwd, Output_Col_Bwd, Output_Row_Fwd
    a = Output_Row_Fwd.from_shapes(1, 8, 8, 2, 2, 16, torch.float32)
    b = Output_Row_Fwd.from_shapes(1, 8, 8, 2, 2, 16, torch.float32)
    for c in (a, b):
        c.O.copy_(torch.randn_like(c.O))
        c.lse.copy_(torch.randn_like(c.lse))
    ref_o, ref_l = lse_merge_reference([(a.O[0].clone(), a.lse[0].clone()), (b.O[0], b.lse[0])])
    a.reduce(b)
    assert torch.allclose(a.O[0], ref_o, atol=1e-6) and torch.allclose(a.lse[0], ref_l, atol=1e-6)
    assert a.data.dtype == torch.uint8 and a.data.is_contiguous()      # one flat buffer
    r = Input_Row_Bwd.from_shapes(1, 8, 8, 2, 2, 16, torch.float32)
    assert r.data.numel() == (2 * 8 * 2 * 16 + 2 * 2 * 8) * 4
    g1 = Output_Col_Bwd.from_shapes(1, 8, 8, 2, 2, 16)
    g2 = Output_Col_Bwd.from_shapes(1, 8, 8, 2, 2, 16)
    g1.dK.fill_(1)
    g2.dK.fill_(2)
    g1.reduce(g2)
    assert g1.dK.eq(3).all()


def test_prepare_seq_parallel_inputs():
    from ultraattn_b200.models.glue import prepare_seq_parallel_inputs
    ids = torch.arange(16)[None]
    out = prepare_seq_parallel_inputs("zigzag_ring_attn", ids, ids, ids, rank=1, world_size=2)
    assert out["local_input_ids"].tolist() == [[4, 5, 6, 7, 8, 9, 10, 11]]
    out = prepare_seq_parallel_inputs("stripe_attn", ids, ids, None, rank=1, world_size=4)
    assert out["local_input_ids"].tolist() == [[1, 5, 9, 13]] and out["local_target_ids"] is None


def test_varlen_attention_cpu():
    import math
    from ultraattn_b200.api import varlen_attention
    torch.manual_seed(0)
    cu = [0, 37, 100, 228, 256]
    T, H, D = 256, 2, 16
    q, k, v = (torch.randn(T, H, D, requires_grad=True) for _ in range(3))
    o = varlen_attention(q, k, v, cu, causal=True)
    d_o = torch.randn_like(o)
    o.backward(d_o)
    mask = torch.zeros(T, T, dtype=torch.bool)
    for a, b in zip(cu[:-1], cu[1:]):
        mask[a:b, a:b] = torch.tril(torch.ones(b - a, b - a, dtype=torch.bool))
    q2, k2, v2 = (t.detach().clone().requires_grad_() for t in (q, k, v))
    s = (torch.einsum("qhd,khd->hqk", q2, k2) / math.sqrt(D)).masked_fill(~mask, float("-inf"))
    o2 = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v2)
    o2.backward(d_o)
    for a, b in ((o, o2), (q.grad, q2.grad), (k.grad, k2.grad), (v.grad, v2.grad)):
        assert (a - b).abs().max().item() < 1e-5


def test_launcher_command_and_env():
    from ultraattn_b200.drivers import launch
    cmd = launch.build_command(8, 29511, ["bench.py", "--gpus", "8"])
    assert cmd[1:4] == ["-m", "torch.distributed.run", "--nnodes=1"]
    assert "--nproc-per-node=8" in cmd and cmd[-3:] == ["bench.py", "--gpus", "8"]
    assert cmd[cmd.index("--master-addr") + 1] == "127.0.0.1"
    env = launch.build_env({}, "pool", "B200", True)
    assert env["CLUSTER_NAME"] == "pool" and env["PLATFORM"] == "B200"
    assert env["NCCL_NVLS_ENABLE"] == "0" and env["UA_NVLS"] == "0"
    assert launch.main(["--gpus", "2", "--dry-run", "--", "-m", "x"]) == 0


def test_cluster_probe_local_and_sinfo_parsing():
    from ultraattn_b200.drivers import cluster_probe as cp
    res = cp.fan_out(["localhost", "127.0.0.1"], ["echo", "hello"])
    assert [r["rc"] for r in res] == [0, 0] and all(r["stdout"].strip() == "hello" for r in res)
    assert cp.run_on_host("localhost", ["definitely-not-a-command-xyz"])["rc"] == -1
    rows = cp.parse_sinfo("gpu* up 4 idle\ngpu* up 12 alloc\ncpu up 3 idle~\n")
    assert rows[0] == {"partition": "gpu", "avail": "up", "nodes": 4, "state": "idle"} and len(rows) == 3
    assert cp.main(["--hosts", "localhost", "--", "true"]) == 0


def test_offloaded_checkpoint_matches_plain_backward():
    """A layer run through OffloadedCheckpoint gives the gradients of the plain call."""
    from easy_context.unsloth_offloaded_gradient_checkpoint import OffloadedCheckpoint
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 8)
    layer = lambda h, scale: torch.tanh(lin(h)) * scale
    x = torch.randn(4, 8, requires_grad=True)
    layer(x, 2.0).sum().backward()
    gx, gw = x.grad.clone(), lin.weight.grad.clone()
    x.grad = None
    lin.weight.grad = None
    OffloadedCheckpoint.apply(layer, x, 2.0).sum().backward()
    assert torch.allclose(x.grad, gx) and torch.allclose(lin.weight.grad, gw)


def test_hf_llama_with_offloaded_checkpoints_and_registered_attention():
    """The reference's glue names on a tiny HuggingFace Llama: offloaded gradient checkpointing
    reproduces the plain gradients; the family-name form of the monkey patch registers an
    attention function."""
    import easy_context
    from transformers import AttentionInterface, LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=64)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).train()
    ids = torch.randint(0, 64, (1, 16))
    model(input_ids=ids, labels=ids).loss.backward()
    ref = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    from ultraattn_b200.models import glue
    calls = []
    orig = glue.OffloadedCheckpoint.forward
    glue.OffloadedCheckpoint.forward = staticmethod(lambda ctx, *a: (calls.append(1), orig(ctx, *a))[1])
    try:
        easy_context.apply_unsloth_offloaded_gradient_checkpoint_monkey_patch(model)
        model(input_ids=ids, labels=ids).loss.backward()
    finally:
        glue.OffloadedCheckpoint.forward = orig
    assert len(calls) == cfg.num_hidden_layers
    for n, p in model.named_parameters():
        assert torch.allclose(p.grad, ref[n], atol=1e-6), n
    name = easy_context.apply_seq_parallel_monkey_patch("zigzag_ring_attn", "llama")
    assert name == "ultraattn_zigzag_ring_attn" and name in AttentionInterface().valid_keys()
    assert easy_context.prepare_dataloader("zigzag_ring_attn", [1, 2]) == [1, 2]
    d = easy_context.prepare_zigzag_ring_attn_inputs(torch.arange(8)[None], torch.arange(8)[None], None, 1, 2)
    assert d["local_input_ids"].tolist() == [[2, 3, 4, 5]] and d["local_target_ids"] is None


def test_reference_helper_names_and_legacy_log_roundtrip(tmp_path):
    """Helper names of the reference's search_algo modules, and the legacy node-profile log:
    written by format_node_profile_lines, parsed back by convert_node_profile_data_to_comp_map."""
    import search_algo.bsa_utils as BU
    import search_algo.exp_configs as EC
    import search_algo.utils as U
    import search_algo.workload_partition as WP
    from ultraattn_b200.planner.cost import format_node_profile_lines
    assert U.get_factors(12) == [1, 2, 3, 4, 6, 12] and str(U.closest_fraction(0.3333, 8)) == "1/3"
    assert U.combine_list_to_0([1, 2], [2, 3]) == [1, 2, 3]
    assert U.filter_kwargs(lambda a, b=1: 0, {"a": 1, "c": 2}) == {"a": 1}
    bac = U.Block_Attention_Config.from_causal(2, 4, [0, 0, 1, 1])
    assert bac.block_table_value.tolist() == [[2, 0, 0, 0], [1, 2, 0, 0], [1, 1, 2, 0], [1, 1, 1, 2]]
    al = WP.Quad_LP_GUROBI_from_block_config(bac, fob=0, hierarchy=1, ParD=4, time_limit=3.0)
    assert al["table"].shape == (4, 4) and (al["table"][np.tril_indices(4)] >= 0).all()
    assert [c.fob for c in EC.get_exp_train_configs()] == [0, 1] and EC.get_exp_configs()[0].plan_type == "manual"
    # compute-balanced allocation of dense causal on 4 ranks: perfectly even, unlike the row owner
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.patterns.blocks import BSA_Config
    cfg = BSA_Config(None, None, {"bsa_repr": P.causal(1), "CP": (4, 1)})
    bal, naive = WP.comp_balance_allocate_strategy(cfg, fob=0), WP.naive_allocate_strategy(cfg, fob=0, ParD=8)
    assert bal.comp_max < naive.comp_max and bal.comp_max == (28 + 8 * 0.5) / 4
    # FULL node tiles: profile key -> plan key / kernel-tile plan
    pre = "fob=1_CP=(8, 1)_shape_config={S=(4096, 16384)_Nh=(1, 1)_bs=1_D=128}_bsa_config={CP=(8, 1)_repr=[[1]]}"
    assert BU.convert_intra_profile_key_to_exe_key_or_plan(pre + "_ablation=(w/o_kernel_tile,Y=2,X=4,dim=0)") == \
        "fob=1_CP=(8, 1)_shape_config=full_ablation=(Y=2,X=4,dim=0)"
    fp = BU.convert_intra_profile_key_to_exe_key_or_plan(pre + "_ablation=(w_kernel_tile,Y=4,X=2,dim=0)")
    assert (fp.Y, fp.X, fp.fob) == (4, 2, 1)
    assert BU.convert_intra_profile_key_to_exe_key_or_plan(pre + "_ablation=(w_kernel_tile,ILP)").endswith("ILP)")
    # legacy log
    lines = []
    for fob in (0, 1):
        lines += format_node_profile_lines(fob, (1, 8), (2048, 2048), (1, 1), 1, 128, False, {
            "orchestrated_attn_func": [(1.0, 3e-4 * (fob + 1)), (1.2, 2e-4 * (fob + 1))],
            "orchestrated_attn_func fused": [(3.0, 1e-4 * (fob + 1))],
            "ring_flash_attn_func": [(9.0, 1e-6)]})
    log = tmp_path / "node.log"
    log.write_text("\n".join(lines) + "\n")
    m = U.convert_node_profile_data_to_comp_map(str(log), 8)
    key = ((1, 8), (256, 256), (1, 1), 1, 128, False)
    assert np.allclose(m["level0"][key], [2e-4, 4e-4]) and np.allclose(m["level1"][key], [1e-4, 2e-4])
    assert m["level2"] is m["level1"]


def test_create_buf_dict_regions_do_not_overlap():
    import search_algo.benchmark as B
    from ultraattn_b200 import patterns as P
    from ultraattn_b200.planner import make_plan
    from ultraattn_b200.planner.schedule import Fused_Execution_Plan
    plan = make_plan(pattern=P.causal(1), cp=2, seq_len=256, n_heads=2, head_dim=16, fob=1,
                     allocation="naive", plan_type="Flexflow")
    d = B.create_buf_dict(plan.da_config, 1, plan, level_rank=0, dtype=torch.float32, device="cpu")
    carriers = [v for k, v in d.items() if isinstance(k, tuple)]
    spans = sorted((c.data.data_ptr(), c.data.data_ptr() + c.nbytes()) for c in carriers if c.nbytes())
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    assert d["inp_row"].Q.shape == (1, 128, 2, 16) and d["out_col"].dV.dtype == torch.float32
    with pytest.raises(ValueError):
        B.create_buf_dict(plan.da_config, 1, plan, tensor_buf=torch.zeros(64, dtype=torch.uint8), dtype=torch.float32)
    f = B.create_buf_dict(plan.da_config, 0, Fused_Execution_Plan(2, 2, None, 0), level_rank=3, fused=True,
                          dtype=torch.float32, device="cpu")
    assert f["graph_type"] == "fused" and len(f["ir_slots"]) == 2 and f["inp_row"] is f[("ir", 1)]
    assert f["ir"].numel() >= 2 * f["inp_row"].nbytes()


def test_cluster_launchers_and_rank_setup(tmp_path, capsys):
    """SLURM / OpenMPI command lines, scheduler variables -> rank variables, NUMA core lists, and a
    real per-rank exec that runs a child with the derived environment."""
    import subprocess
    import sys
    from ultraattn_b200.drivers import launch
    assert launch.main(["--launcher", "slurm", "--nodes", "2", "--gpus", "8", "--partition", "H800",
                        "--ib-hca", "mlx5_0,mlx5_1", "--dry-run", "--", "bench.py"]) == 0
    line = capsys.readouterr().out
    assert line.startswith("srun -N 2 --ntasks-per-node=8 --gres=gpu:8 -K") and "--rank-exec --ib-hca mlx5_0,mlx5_1 -- bench.py" in line
    assert launch.main(["--launcher", "mpirun", "--hosts", "g1:8,g2:4", "--dry-run", "--", "bench.py"]) == 0
    assert capsys.readouterr().out.startswith("mpirun -np 12 --host g1:8,g2:4")
    e = launch.rank_env({"SLURM_PROCID": "9", "SLURM_NTASKS": "16", "SLURM_LOCALID": "1",
                         "SLURM_NTASKS_PER_NODE": "8", "SLURM_JOB_NODELIST": "g1,g2"})
    assert (e["RANK"], e["WORLD_SIZE"], e["LOCAL_RANK"], e["LOCAL_WORLD_SIZE"], e["MASTER_ADDR"]) == ("9", "16", "1", "8", "g1")
    e = launch.rank_env({"OMPI_COMM_WORLD_RANK": "3", "OMPI_COMM_WORLD_SIZE": "4", "OMPI_COMM_WORLD_LOCAL_RANK": "3",
                         "MASTER_ADDR": "10.0.0.1"})
    assert e["RANK"] == "3" and "MASTER_ADDR" not in e and e["MASTER_PORT"] == "12215"
    assert launch.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    for n, cpus in enumerate(["0-3", "4-7"]):
        (tmp_path / f"node{n}").mkdir()
        (tmp_path / f"node{n}" / "cpulist").write_text(cpus + "\n")
    nodes = launch.numa_nodes(str(tmp_path))
    assert nodes == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert launch.cpus_for_local_rank(1, 8, nodes) == [0, 1, 2, 3] and launch.cpus_for_local_rank(6, 8, nodes) == [4, 5, 6, 7]
    assert launch.cpus_for_local_rank(0, 8, []) == []
    env = dict(os.environ, SLURM_PROCID="5", SLURM_NTASKS="8", SLURM_LOCALID="5", SLURM_NTASKS_PER_NODE="8")
    env.pop("RANK", None)
    out = subprocess.run([sys.executable, "-m", "ultraattn_b200.drivers.launch", "--rank-exec", "--ib-hca", "mlx5_9",
                          "--", "-c", "import os; print(os.environ['RANK'], os.environ['WORLD_SIZE'], "
                          "os.environ['NCCL_IB_HCA'], os.environ['CUDA_DEVICE_MAX_CONNECTIONS'])"],
                         env=env, capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(__file__)))
    assert out.stdout.split() == ["5", "8", "mlx5_9", "32"], out.stderr


def test_ring_utils_and_dense_helpers(tmp_path):
    """update_out_and_lse equals one softmax over both blocks; flatten / unflatten of packed lse;
    write_plan round trip; the causal-only allocation names."""
    import math
    import search_algo.dense_utils as DU
    import search_algo.workload_partition as WP
    from ring_flash_attn.utils import flatten_varlen_lse, unflatten_varlen_lse, update_out_and_lse
    torch.manual_seed(0)
    B, S, H, D = 1, 8, 2, 4
    q, k1, k2, v1, v2 = (torch.randn(B, S, H, D) for _ in range(5))

    def block(k, v):
        s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(D)
        return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v), torch.logsumexp(s, -1)
    o1, l1 = block(k1, v1)
    o2, l2 = block(k2, v2)
    out, lse = update_out_and_lse(None, None, o1, l1)
    out, lse = update_out_and_lse(out, lse, o2, l2)
    o_ref, l_ref = block(torch.cat([k1, k2], 1), torch.cat([v1, v2], 1))
    assert torch.allclose(out, o_ref, atol=1e-5) and torch.allclose(lse.squeeze(-1).transpose(1, 2), l_ref, atol=1e-5)
    half = (slice(None), slice(0, 4))
    out2, lse2 = update_out_and_lse(o1.clone(), l1.transpose(1, 2).unsqueeze(-1).clone(), o2[:, :4], l2[:, :, :4], slice_=half)
    assert torch.allclose(out2[:, :4], o_ref[:, :4], atol=1e-5) and torch.allclose(out2[:, 4:], o1[:, 4:])
    cu = [0, 3, 8]
    padded = torch.randn(2, H, 5)
    flat = flatten_varlen_lse(padded, cu)
    assert flat.shape == (H, 8) and torch.equal(flat[:, :3], padded[0, :, :3])
    back = unflatten_varlen_lse(flat.t().unsqueeze(-1), cu, 5)
    assert torch.equal(back[0, :, :3], padded[0, :, :3]) and torch.equal(back[1], padded[1])
    plan = DU.create_plan_for_full(4, 2, 0)
    path = DU.write_plan(plan, str(tmp_path))
    assert os.path.exists(path) and os.path.exists(path[:-4] + ".json")
    full, causal = DU.split_dense_configs([WP._causal_config(2), P.BSA_Config.create_full((2, 1))])
    assert len(full) == 1 and len(causal) == 1
    al = WP.ILP(2)
    assert al["table"].tolist()[0][0] == 0 and al["table"][1, 1] == 1


def test_start_gate_is_a_no_op_on_cpu():
    from ultraattn_b200.drivers.benchmark import benchmark_ops
    from ultraattn_b200.ops.gate import StartGate
    g = StartGate("cpu")
    g.close()
    g.open()
    assert g.check() and g.epoch == 1 and int(g.flag[0]) == 1
    assert benchmark_ops(lambda: None, warmup=1, num_iter=2, repeats=1, device=torch.device("cpu"), start_gate=True) >= 0


def test_inputs_sharded_by_remapped_ownership():
    from ultraattn_b200.models.glue import prepare_seq_parallel_inputs, shard_by_ownership
    ids = torch.arange(16)[None]
    cmap = P.cmap_strided(8, 4)                       # rank r owns blocks r and r + 4 (2 tokens each)
    out = prepare_seq_parallel_inputs("ultra_attn", ids, ids, None, rank=1, world_size=4, cmap=cmap)
    assert out["local_input_ids"].tolist() == [[2, 3, 10, 11]] and out["local_target_ids"] is None
    assert shard_by_ownership(torch.arange(8), P.cmap_zigzag(4, 2), 0, dim=0).tolist() == [0, 1, 6, 7]


def test_every_reference_module_path_imports_and_exports():
    """Every module path of the reference that this distribution mirrors imports, and exports the
    names code written against the reference uses."""
    import importlib
    surface = {
        "search_algo.bsa_config": ["BSA_Repr", "BSA_Config"],
        "search_algo.bsa_utils": ["create_bsa_block_table", "split_to_node_configs", "get_b2f_suf_map",
                                  "select_best_profile_comp_key", "convert_intra_profile_key_to_exe_key_or_plan",
                                  "convert_shape_config_to_str", "bsa_is_full", "bsa_is_causal", "bsa_is_dense"],
        "search_algo.custom_sparse_pattern": ["create_block_sparse_pattern"],
        "search_algo.utils": ["Block_Type", "Block_Table_Type", "Block_Comp_Volume", "Block_Attention_Config",
                              "FinitePriorityQueue", "calc_flops", "report_memory", "print_rank_0", "parse_args",
                              "all_wait_main_stream", "main_stream_wait_all", "convert_profile_data_to_map",
                              "convert_profile_data_to_comm_map", "convert_node_profile_data_to_comp_map",
                              "get_factors", "closest_fraction", "unique_list", "use_all_cpus"],
        "search_algo.workload_partition": ["solve_sparse_from_bsa", "naive_allocate_strategy",
                                           "Quad_LP_GUROBI_from_block_config", "comp_balance_allocate_strategy",
                                           "Quad_LP_GUROBI", "ILP", "solve_global_causal", "solve_custom_sparse",
                                           "print_lp_result", "convert_result_to_np", "main"],
        "search_algo.manual_schedules": ["get_qo_schedule_table", "get_kv_schedule_table", "get_cc_optimal_schedule_table"],
        "search_algo.dense_utils": ["CP2ParD_map", "get_block_schedule_table_for_full", "create_plan_for_full",
                                    "create_ablation_configs_for_full", "create_plan_key_suffixes_for_full",
                                    "write_plan", "split_dense_configs"],
        "search_algo.search_engine": ["Evaluation_Configs", "Dist_Attn_Config", "Dist_Attn_Schedule", "Machine_Config",
                                      "FlashAttn_Profile_Map", "Inter_Comp_Profile_Map", "Comm_Profile_Map",
                                      "get_cc_optimal_schedule_from_table"],
        "search_algo.dependent_graph": ["Dependent_Graph", "Cuda_Kernel", "Comp_Kernel", "Comm_Kernel"],
        "search_algo.graph_transformation_engine": ["Graph_Transformation_Engine", "Comp_Fusion_Substitution",
                                                    "Comp_Fusion_Transformation", "Graph_Substitution",
                                                    "Graph_Transformation", "Comm_Rebuild_Engine"],
        "search_algo.execute_plan": ["Execution_Plan", "Fused_Execution_Plan"],
        "search_algo.search_comm": ["Brute_Force_Search_Engine", "get_configs"],
        "search_algo.database": ["Prof_DB"],
        "search_algo.initialize": ["get_proc_info", "initialize_distribution", "initialize_prof_db",
                                   "parse_slurm_tasks_per_node"],
        "search_algo.exp_configs": ["get_exp_configs", "get_exp_train_configs", "get_exp_infer_configs",
                                    "get_bsa_train_configs", "get_dense_train_configs", "get_bsa_infer_configs",
                                    "step0_top_down_decompose"],
        "search_algo.benchmark": ["benchmark_ops", "benchmark_orchestrate_bsa", "prepare_inter_comp_plans", "create_buf_dict"],
        "search_algo.arguments": ["parse_args", "get_args", "parse_config", "recursive_update", "print_args",
                                  "parse_parallel_args", "parse_shape_args", "parse_pattern_args", "parse_experiment_args"],
        "search_algo.global_vars": ["get_global_var", "set_global_var", "TASK_STATUS"],
        "search_algo.task1_bsa": ["main", "get_general_bsa_cc_optimal_schedule", "step1_generate_intra_bsa_exe_plans",
                                  "step1_generate_intra_full_exe_plans", "step2_profile_intra_bsa_exe_plans",
                                  "step2_profile_intra_full_exe_plans", "step3_generate_inter_bsa_exe_plans",
                                  "step3_generate_inter_dense_exe_plans", "generate_intra_bsa_execution_plans",
                                  "generate_inter_bsa_execution_plans", "generate_general_full_execution_plans",
                                  "profile_all_intra_BSA", "profile_all_intra_full",
                                  "get_general_bsa_cc_optimal_schedule_old"],
        "search_algo.task2_bsa": ["main", "step4_profile_inter_bsa_exe_plans", "step4_profile_inter_full_exe_plans",
                                  "profile_all_inter_BSA", "profile_all_inter_full"], "search_algo.main": ["main"],
        "search_algo.fusion_evaluate": ["main"], "search_algo.intra_attn_gen": ["main"],
        "orchestrated_attn": ["orchestrated_attn_func", "orchestrated_attn_backward", "OrchestratedAttnFunc",
                              "Input_Row_Fwd", "Input_Col_Fwd", "Output_Row_Fwd", "Output_Col_Fwd",
                              "Input_Row_Bwd", "Input_Col_Bwd", "Output_Row_Bwd", "Output_Col_Bwd"],
        "orchestrated_attn.orchestrated_attn_impl": ["orchestrated_attn_forward", "orchestrated_attn_backward",
                                                     "fused_attn_forward", "fused_attn_backward",
                                                     "intra_attn_forward", "intra_attn_backward"],
        "orchestrated_attn.utils": ["IntraComm", "InterComm", "IntraComm_fused", "InterComm_fused", "Integrated_Data",
                                    "Comm_Fused", "get_Q_shape_from_da_config", "get_K_shape_from_da_config",
                                    "get_lse_shape_from_da_config", "print_rank_0"],
        "orchestrated_attn.global_vars": ["FULL_DTYPE", "ncclcomm_dict", "cpu_group_dict", "streams",
                                          "is_exist_global_var"],
        "ring_flash_attn": ["ring_flash_attn_func", "ring_flash_attn_kvpacked_func", "ring_flash_attn_qkvpacked_func",
                            "ring_flash_attn_backward", "ring_flash_attn_varlen_func",
                            "zigzag_ring_flash_attn_func", "zigzag_ring_flash_attn_varlen_func",
                            "zigzag_ring_flash_attn_varlen_qkvpacked_func", "stripe_flash_attn_func",
                            "stripe_flash_attn_kvpacked_func"],
        "ring_flash_attn.utils": ["update_out_and_lse", "flatten_varlen_lse", "unflatten_varlen_lse"],
        "hierarchy_attn": ["hierarchy_attn_func"], "head_parallel_attn": ["deepspeed_ulysses_attn_func"],
        "comm_lib.comm_utils": ["RingComm", "RingCommOld", "RingCommNew", "A2AComm"],
        "easy_context": ["prepare_seq_parallel_inputs", "apply_seq_parallel_monkey_patch", "prepare_dataloader",
                         "prepare_zigzag_ring_attn_inputs", "prepare_dist_flash_attn_inputs",
                         "apply_zigzag_ring_attn_monkey_patch_llama", "apply_zigzag_ring_attn_monkey_patch_mistral",
                         "apply_dist_flash_attn_monkey_patch_llama",
                         "apply_unsloth_offloaded_gradient_checkpoint_monkey_patch"],
        "ring_flash_attn.ring_flash_attn": ["ring_flash_attn_forward", "ring_flash_attn_backward", "RingFlashAttnFunc",
                                            "ring_flash_attn_func", "ring_flash_attn_qkvpacked_func"],
        "ring_flash_attn.zigzag_ring_flash_attn": ["zigzag_ring_flash_attn_forward", "zigzag_ring_flash_attn_backward",
                                                   "ZigZagRingFlashAttnFunc", "zigzag_ring_flash_attn_func"],
        "ring_flash_attn.stripe_flash_attn": ["stripe_flash_attn_forward", "stripe_flash_attn_backward",
                                              "StripeFlashAttnFunc", "stripe_flash_attn_func"],
        "ring_flash_attn.ring_flash_attn_varlen": ["ring_flash_attn_varlen_forward", "ring_flash_attn_varlen_backward",
                                                   "RingFlashAttnVarlenFunc", "ring_flash_attn_varlen_func"],
        "ring_flash_attn.zigzag_ring_flash_attn_varlen": ["get_half_index", "get_half_lse", "ZigZagRingFlashAttnVarlenFunc",
                                                          "zigzag_ring_flash_attn_varlen_forward",
                                                          "zigzag_ring_flash_attn_varlen_func"],
        "ring_flash_attn.triton_utils": ["flatten_varlen_lse", "unflatten_varlen_lse"],
        "head_parallel_attn.deepspeed_ulysses_attn": ["deepspeed_ulysses_attn_forward", "deepspeed_ulysses_attn_backward",
                                                      "DeepSpeedUlyssesAttnFunc", "deepspeed_ulysses_attn_func"],
        "hierarchy_attn.hierarchy_attn_impl": ["intra_attn_forward", "hierarchy_attn_forward", "hierarchy_attn_backward",
                                               "overlapped_hierarchy_attn_forward", "overlapped_hierarchy_attn_backward",
                                               "HierarchyAttnFunc", "hierarchy_attn_func"],
        "hierarchy_attn.utils": ["IntraComm", "InterComm", "OverlappedInterComm", "wait_recursively",
                                 "update_out_and_lse", "print_rank_0"],
        "easy_context.zigzag_ring_attn.monkey_patch": ["apply_zigzag_ring_attn_monkey_patch_llama",
                                                       "apply_zigzag_ring_attn_monkey_patch_mistral"],
        "easy_context.zigzag_ring_attn.prepare_inputs": ["extract_local", "prepare_zigzag_ring_attn_inputs"],
        "easy_context.dist_flash_attn.monkey_patch": ["apply_dist_flash_attn_monkey_patch_llama"],
        "easy_context.unsloth_offloaded_gradient_checkpoint.monkey_patch": [
            "Unsloth_Offloaded_Gradient_Checkpointer", "apply_unsloth_offloaded_gradient_checkpoint_monkey_patch"],
        "easy_context.dist_flash_attn.lightseq_async_attn": ["attention"],
        "easy_context.dist_flash_attn.async_communication": ["initialize_distributed", "get_sequence_parallel_group",
                                                            "get_sequence_parallel_rank", "get_sequence_parallel_size",
                                                            "is_last_time", "is_compute_for_local_query", "is_idle",
                                                            "is_sync_from_remote", "print_and_reset_comm_stats"],
        "easy_context.dist_flash_attn.prepare_input": ["extract_local", "prepare_dist_flash_attn_inputs"],
        "easy_context.zigzag_ring_attn": ["prepare_zigzag_ring_attn_inputs"],
        "easy_context.unsloth_offloaded_gradient_checkpoint": ["apply_unsloth_offloaded_gradient_checkpoint_monkey_patch"],
    }
    missing = []
    for mod, names in surface.items():
        m = importlib.import_module(mod)
        missing += [f"{mod}.{n}" for n in names if not hasattr(m, n)]
    assert not missing, missing


def test_kernel_trace_summary_on_a_synthetic_launch():
    """`utils.kernel_trace.summarize` on a hand-made trace: 4 SMs, two waves of 1 ms CTAs, the first
    wave spends 0.2 ms copying, one SM gets a third CTA (the tail)."""
    import numpy as np
    from ultraattn_b200.utils.kernel_trace import summarize
    ms = 1_000_000
    rows = []
    for sm in range(4):
        rows.append((0, int(0.2 * ms), 1 * ms, sm << 32 | sm))                 # first wave: copies, then computes
        rows.append((1 * ms, 1 * ms + 500, 2 * ms, sm << 32 | (4 + sm)))       # second wave: no copying
    rows.append((2 * ms, 2 * ms, 3 * ms, 0 << 32 | 8))                          # tail on SM 0
    out = summarize(np.array(rows, dtype=np.int64), n_sms=4)
    assert out["ctas"] == 9 and out["span_ms"] == 3.0
    assert out["ctas_that_copied"] == 4 and out["staging_sm_ms_total"] == 0.8 and out["staging_done_ms_after_start"] == 0.2
    assert out["longest_cta_ms"] == 1.0 and out["last_cta_start_ms"] == 2.0
    assert out["tail_ms_under_half_sms"] == 1.0                               # three of four SMs are done at 2 ms
    assert abs(out["sm_busy_fraction"] - 9 / 12) < 1e-4
    assert summarize(np.zeros((0, 4), dtype=np.int64)) == {"ctas": 0}


def test_planner_helpers_accept_the_reference_argument_lists():
    """`search_algo.manual_schedules` / `dense_utils` / `utils.calc_flops` called the way the
    reference's own code calls them; expected values were produced by the reference's functions."""
    import numpy as np
    from search_algo.dense_utils import (create_ablation_configs_for_full, create_plan_for_full,
                                         create_plan_key_suffixes_for_full, get_block_schedule_table_for_full)
    from search_algo.manual_schedules import get_kv_schedule_table, get_qo_schedule_table
    from search_algo.utils import calc_flops
    S_map = np.array([[3, 2, 1, 0]])
    qo = get_qo_schedule_table([4, 4, 1, 1], S_map, True)
    assert qo.shape == (1, 1, 4, 4) and qo[0, 0].tolist() == [[3, -1, -1, -1], [3, 2, -1, -1], [3, 2, 1, -1], [3, 2, 1, 0]]
    kv = get_kv_schedule_table([4, 4, 1, 1], S_map, True)
    assert kv[0, 0].tolist() == [[3, -1, -1, -1], [2, 2, -1, -1], [1, 1, 1, -1], [0, 0, 0, 0]]
    assert get_kv_schedule_table(3, True).tolist() == [[0, -1, -1], [1, 1, -1], [2, 2, 2]]       # short form
    grid = get_block_schedule_table_for_full([4, 4, 1, 1], S_map, 2, None)
    assert grid[0, 0].tolist() == [[3, 2, 3, 2], [3, 2, 3, 2], [1, 0, 1, 0], [1, 0, 1, 0]]
    assert [list(calc_flops(2, (1024, 2048), 8, 128, f, 0.5)) for f in (0, 1, 2)] == \
        [[8589934592.0, 8589934592.0], [17179869184.0, 21474836480.0], [25769803776.0, 30064771072.0]]
    assert create_ablation_configs_for_full(4)[1] == {"Y": 2, "X": 2, "first_dim": 0, "KERNEL_TILE_TYPE": "w/o_kernel_tile"}
    assert create_plan_key_suffixes_for_full(8) == ["_ablation=(Y=8,X=1,dim=0)", "_ablation=(Y=4,X=2,dim=0)",
                                                    "_ablation=(Y=2,X=4,dim=0)", "_ablation=(Y=1,X=8,dim=0)"]
    from ultraattn_b200.patterns.blocks import BSA_Config
    from ultraattn_b200.planner.cost import Dist_Attn_Config, Machine_Config
    da = Dist_Attn_Config.from_bsa_config(BSA_Config.create_full((4, 1)),
                                          {"S": (4096, 4096), "Nh": (2, 2), "bs": 1, "D": 128}, hierarchy=1)
    plan = create_plan_for_full(da, Machine_Config.b200_default(), 2, 1, 0)
    assert plan.X == 2 and plan.fob == 1 and plan.verify() == []
    assert create_plan_for_full(4, 2, 0).X == 2                                                  # short form


def test_solver_result_helpers_of_workload_partition(capsys):
    """``convert_result_to_np`` / ``print_lp_result`` read a solver's variable dictionary
    (``x_i_j_k`` with a value attribute) into the allocation table; ``solve_custom_sparse`` solves
    one parametric pattern and every non-empty tile gets a rank."""
    import numpy as np
    from search_algo.workload_partition import convert_result_to_np, print_lp_result, solve_custom_sparse

    class Var:
        def __init__(self, x):
            self.X = x
    own = {(1, 0): 0, (2, 0): 1, (2, 1): 1}
    Vars = {f"x_{i}_{j}_{k}": Var(1.0 if r == k else 0.0) for (i, j), r in own.items() for k in range(2)}
    table = convert_result_to_np(2, 3, Vars, "X", np.array([0, 1, 1]))
    assert table.tolist() == [[0, -1, -1], [0, 1, -1], [1, 1, 1]]
    print_lp_result(2, 3, Vars, "X", np.array([0, 1, 1]))
    out = capsys.readouterr().out
    assert "Allocation Matrix:" in out and out.strip().splitlines()[-1].split() == ["1", "1", "1"]
    al = solve_custom_sparse(CP=2, Par_D=4, local_blocks=2, time_limit=5.0)
    t = np.asarray(al.table)
    assert t.shape == (4, 4) and (t[np.arange(4), np.arange(4)] >= 0).all() and t[0, 3] == -1
