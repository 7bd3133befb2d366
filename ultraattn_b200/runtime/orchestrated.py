"""The reference's runtime entry points, made functional.

``orchestrated_attn_func`` / ``orchestrated_attn_backward`` keep the reference's signature
(orchestrated_attn/orchestrated_attn_impl.py:622, 763) and its data carriers
(orchestrated_attn/utils.py:34-298: every bundle is ONE flat contiguous buffer with typed views, so
one message moves the whole bundle). In the reference the forward returns ``None``, the backward
asserts and the carriers' ``reduce`` methods are empty; here the call executes the plan and the
carriers reduce for real: forward partial outputs merge with the log-sum-exp rule, backward
partial gradients add.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import elementwise as E
from .executor import PlanExecutor


class Integrated_Data:
    """A bundle of tensors laid out back to back in one byte buffer."""
    fields: tuple = ()

    def __init__(self, specs, buf: Optional[torch.Tensor] = None, device=None):
        nbytes = 0
        offs = []
        for _, dtype, shape in specs:
            n = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
            offs.append((nbytes, n))
            nbytes += (n + 15) // 16 * 16
        self.data = buf[:nbytes] if buf is not None else torch.zeros(nbytes, dtype=torch.uint8, device=device)
        for (name, dtype, shape), (o, n) in zip(specs, offs):
            setattr(self, name, self.data[o:o + n].view(dtype).view(*shape))
        self.specs = specs

    @classmethod
    def from_da_config_with_buf(cls, da_config, buf=None, batch_degree: int = 1, dtype=torch.bfloat16, device=None):
        sq, skv = da_config.S_per_partition
        return cls.from_shapes(da_config.bs, sq * batch_degree, skv * batch_degree, da_config.Nh[0],
                               da_config.Nh[1], da_config.D, dtype, buf, device)

    def nbytes(self) -> int:
        return self.data.numel()


def _carrier(name, spec_fn, doc):
    def from_shapes(cls, bs, sq, skv, nh, ng, d, dtype=torch.bfloat16, buf=None, device=None):
        return cls(spec_fn(bs, sq, skv, nh, ng, d, dtype), buf, device)
    return type(name, (Integrated_Data,), {"from_shapes": classmethod(from_shapes), "__doc__": doc})


f32 = torch.float32
Input_Row_Fwd = _carrier("Input_Row_Fwd", lambda b, sq, sk, nh, ng, d, dt: [("Q", dt, (b, sq, nh, d))], "Q")
Input_Col_Fwd = _carrier("Input_Col_Fwd", lambda b, sq, sk, nh, ng, d, dt: [("K", dt, (b, sk, ng, d)), ("V", dt, (b, sk, ng, d))], "K | V")
Input_Row_Bwd = _carrier("Input_Row_Bwd", lambda b, sq, sk, nh, ng, d, dt: [
    ("Q", dt, (b, sq, nh, d)), ("dO", dt, (b, sq, nh, d)), ("D", f32, (b, nh, sq)), ("lse", f32, (b, nh, sq))],
    "Q | dO | D | lse")
Input_Col_Bwd = _carrier("Input_Col_Bwd", lambda b, sq, sk, nh, ng, d, dt: [("K", dt, (b, sk, ng, d)), ("V", dt, (b, sk, ng, d))], "K | V")
Output_Col_Fwd = _carrier("Output_Col_Fwd", lambda b, sq, sk, nh, ng, d, dt: [], "(empty)")


class Output_Row_Fwd(Integrated_Data):
    """O | lse. ``reduce`` merges another partial output into this one."""

    @classmethod
    def from_shapes(cls, bs, sq, skv, nh, ng, d, dtype=torch.bfloat16, buf=None, device=None):
        return cls([("O", dtype, (bs, sq, nh, d)), ("lse", f32, (bs, nh, sq))], buf, device)

    def reduce(self, other: "Output_Row_Fwd") -> None:
        for b in range(self.O.shape[0]):
            E.lse_merge([(self.O[b], self.lse[b]), (other.O[b], other.lse[b])], (self.O[b], self.lse[b]))


class Output_Row_Bwd(Integrated_Data):
    """dQ (fp32). ``reduce`` adds."""

    @classmethod
    def from_shapes(cls, bs, sq, skv, nh, ng, d, dtype=torch.bfloat16, buf=None, device=None):
        return cls([("dQ", f32, (bs, sq, nh, d))], buf, device)

    def reduce(self, other: "Output_Row_Bwd") -> None:
        self.dQ.add_(other.dQ)


class Output_Col_Bwd(Integrated_Data):
    """dK | dV (fp32). ``reduce`` adds."""

    @classmethod
    def from_shapes(cls, bs, sq, skv, nh, ng, d, dtype=torch.bfloat16, buf=None, device=None):
        return cls([("dK", f32, (bs, skv, ng, d)), ("dV", f32, (bs, skv, ng, d))], buf, device)

    def reduce(self, other: "Output_Col_Bwd") -> None:
        self.dK.add_(other.dK)
        self.dV.add_(other.dV)


_executors: dict = {}


def _executor(execution_plan_dict: dict, PROC_INFO, device):
    """The object that runs the plans of ``execution_plan_dict``: a :class:`PlanExecutor` for
    launch plans ('fwd' / 'bwd', or 'intra'), a grid executor for a kernel-tile plan ('fused': a
    ``Fused_Execution_Plan``). Cached per plan object."""
    fused = execution_plan_dict.get("fused")
    if fused is not None:
        key = ("fused", id(fused))
        if key not in _executors:
            from .grid import GridExecutor
            _executors[key] = GridExecutor.from_plan(fused, execution_plan_dict.get("group"), device,
                                                     execution_plan_dict.get("registry"))
        return _executors[key]
    key = (id(execution_plan_dict.get("fwd") or execution_plan_dict.get("intra")), id(execution_plan_dict.get("bwd")))
    if key not in _executors:
        pf = execution_plan_dict.get("fwd") or execution_plan_dict.get("intra")
        pb = execution_plan_dict.get("bwd")
        _executors[key] = PlanExecutor(pf, pb, group=execution_plan_dict.get("group"), device=device,
                                       p2p_groups=execution_plan_dict.get("p2p_groups"))
    return _executors[key]


class OrchestratedAttnFunc(torch.autograd.Function):
    """Differentiable form on plain tensors (the reference's class of this name has a forward that
    returns nothing and a backward that asserts, orchestrated_attn_impl.py:688-761):
    ``OrchestratedAttnFunc.apply(q, k, v, softmax_scale, execution_plan_dict)`` -> O of this
    rank's shard; gradients flow to q, k, v."""

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, execution_plan_dict):
        ex = _executor(execution_plan_dict, None, q.device)
        o, lse = ex.forward(q, k, v, softmax_scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.ex, ctx.scale = ex, softmax_scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ctx.ex.backward(d_o.contiguous(), q, k, v, o, lse, ctx.scale)
        return dq, dk, dv, None, None


def orchestrated_attn_func(inp_row, inp_col, dropout_p: float = 0.0, softmax_scale=None, causal: bool = False,
                           window_size=(-1, -1), alibi_slopes=None, deterministic: bool = False,
                           return_attn_probs: bool = False, PROC_INFO=None, execution_plan_dict=None,
                           extra_dict=None):
    """Forward of the planned distributed attention. ``inp_row`` carries this rank's Q shard,
    ``inp_col`` its K | V shard; ``execution_plan_dict`` = {'fwd': plan, 'bwd': plan, 'group': pg}.
    Returns an :class:`Output_Row_Fwd` (O, lse) for this rank's shard."""
    assert dropout_p == 0.0 and alibi_slopes is None
    ex = _executor(execution_plan_dict, PROC_INFO, inp_row.Q.device)
    o, lse = ex.forward(inp_row.Q, inp_col.K, inp_col.V, softmax_scale)
    out = Output_Row_Fwd.from_shapes(o.shape[0], o.shape[1], o.shape[1], o.shape[2], inp_col.K.shape[2],
                                     o.shape[3], o.dtype, None, o.device)
    out.O.copy_(o)
    out.lse.copy_(lse)
    return out


def orchestrated_attn_backward(inp_row, inp_col, out_fwd=None, dropout_p: float = 0.0, softmax_scale=None,
                               causal: bool = False, window_size=(-1, -1), alibi_slopes=None,
                               deterministic: bool = False, PROC_INFO=None, execution_plan_dict=None,
                               extra_dict=None):
    """Backward. ``inp_row`` is an :class:`Input_Row_Bwd` (Q | dO | D | lse; D is recomputed from
    ``out_fwd`` when given), ``inp_col`` K | V. Returns (Output_Row_Bwd, Output_Col_Bwd)."""
    ex = _executor(execution_plan_dict, PROC_INFO, inp_row.Q.device)
    o = out_fwd.O if out_fwd is not None else None
    if o is None:
        raise ValueError("the forward output (O, lse) is needed to form D = rowsum(dO * O)")
    dq, dk, dv = ex.backward(inp_row.dO, inp_row.Q, inp_col.K, inp_col.V, o, inp_row.lse, softmax_scale)
    r = Output_Row_Bwd.from_shapes(dq.shape[0], dq.shape[1], dk.shape[1], dq.shape[2], dk.shape[2], dq.shape[3],
                                   dq.dtype, None, dq.device)
    c = Output_Col_Bwd.from_shapes(dq.shape[0], dq.shape[1], dk.shape[1], dq.shape[2], dk.shape[2], dq.shape[3],
                                   dq.dtype, None, dq.device)
    r.dQ.copy_(dq)
    c.dK.copy_(dk)
    c.dV.copy_(dv)
    return r, c


# -------------------------------------------------------------------------------------------------
# one buffer for every carrier of a plan
# -------------------------------------------------------------------------------------------------
def _carrier_types(fob: int) -> dict:
    return {("i", "r"): Input_Row_Fwd if fob == 0 else Input_Row_Bwd,
            ("i", "c"): Input_Col_Fwd if fob == 0 else Input_Col_Bwd,
            ("o", "r"): Output_Row_Fwd if fob == 0 else Output_Row_Bwd,
            ("o", "c"): Output_Col_Fwd if fob == 0 else Output_Col_Bwd}


def _fusion_degrees(execution_plan, level_rank: int) -> tuple:
    """(row degrees, column degrees) of the compute kernels of one rank: a fused kernel spans
    several Q rows / KV columns, a plain one spans one of each."""
    rows, cols = {1}, {1}
    lists = getattr(execution_plan, "gpu_kernel_lists", None) or {}
    for k in (lists.get(level_rank, []) if isinstance(lists, dict) else lists[level_rank]):
        if getattr(k, "type", None) == "comp":
            r, c = k.key[2], k.key[3]
            rows.add(len(r) if isinstance(r, tuple) else 1)
            cols.add(len(c) if isinstance(c, tuple) else 1)
    return sorted(rows), sorted(cols)


def create_buf_dict(da_config, fob: int, execution_plan=None, batch_degrees=(1, 1), tensor_buf=None,
                    level_rank: int = 0, fused: bool = False, dtype=torch.bfloat16, device=None) -> dict:
    """Carve the data carriers of a plan out of ONE byte buffer (reference: search_algo/benchmark.py:
    231-334, where every carrier aliases offset 0 of the buffer because results are discarded;
    here every carrier has its own 256-byte aligned region, so the buffers hold real data).

    General plans: ``buf_dict[((io, rc), degree)]`` for ``io`` in 'i'/'o', ``rc`` in 'r'/'c' and
    every fusion degree of the rank's compute kernels, plus the aliases ``inp_row``, ``inp_col``,
    ``out_row``, ``out_col`` (degree 1). Kernel-tile plans (``fused=True``, a
    ``Fused_Execution_Plan``): regions ``ir`` / ``or`` with X slots and ``ic`` / ``oc`` with Y slots
    (the gather / reduce-scatter operands), ``inp_row`` / ``inp_col`` being this rank's own slot.
    ``tensor_buf=None`` allocates exactly what is needed; a buffer that is too small is an error.
    """
    types = _carrier_types(fob)
    cursor = 0
    pending = []            # (key, cls, batch_degree, offset, nbytes)

    def reserve(key, cls, degree):
        nonlocal cursor
        probe = cls.from_da_config_with_buf(da_config, None, degree, dtype, "meta")
        n = probe.nbytes()
        pending.append((key, cls, degree, cursor, n))
        cursor += (n + 255) // 256 * 256

    out: dict = {"graph_type": "fused" if fused else "general"}
    if not fused:
        row_deg, col_deg = _fusion_degrees(execution_plan, level_rank) if execution_plan is not None else ([1], [1])
        for io in ("i", "o"):
            for deg in row_deg:
                reserve(((io, "r"), deg), types[(io, "r")], batch_degrees[0] * deg)
            for deg in col_deg:
                reserve(((io, "c"), deg), types[(io, "c")], batch_degrees[1] * deg)
    else:
        X, Y = execution_plan.X, execution_plan.Y
        for name, rc, n_slots in (("ir", "r", X), ("ic", "c", Y), ("or", "r", X), ("oc", "c", Y)):
            io = name[0]
            for slot in range(n_slots):
                reserve((name, slot), types[(io, rc)], batch_degrees[0 if rc == "r" else 1])
    if tensor_buf is None:
        tensor_buf = torch.zeros(max(cursor, 1), dtype=torch.uint8, device=device)
    buf = tensor_buf.view(torch.uint8).view(-1) if tensor_buf.dtype != torch.uint8 else tensor_buf.view(-1)
    if buf.numel() < cursor:
        raise ValueError(f"tensor_buf holds {buf.numel()} bytes, the plan's carriers need {cursor}")
    for key, cls, degree, off, n in pending:
        out[key] = cls.from_da_config_with_buf(da_config, buf[off:off + max(n, 0)], degree, dtype)
    out["tensor_buf"], out["nbytes"] = tensor_buf, cursor
    if not fused:
        out["inp_row"], out["inp_col"] = out[(("i", "r"), 1)], out[(("i", "c"), 1)]
        out["out_row"], out["out_col"] = out[(("o", "r"), 1)], out[(("o", "c"), 1)]
    else:
        x_id, y_id = level_rank % X, level_rank // X
        for name, n_slots in (("ir", X), ("ic", Y), ("or", X), ("oc", Y)):
            first, last = pending_offsets(pending, name)
            out[name] = buf[first:last]
            out[name + "_slots"] = [out[(name, s)] for s in range(n_slots)]
        out["inp_row"], out["inp_col"] = out[("ir", x_id)], out[("ic", y_id)]
        out["out_row"], out["out_col"] = out[("or", x_id)], out[("oc", y_id)]
    return out


def pending_offsets(pending, name: str) -> tuple:
    """Byte range [first, last) that the slots of region ``name`` cover."""
    spans = [(off, off + n) for key, _, _, off, n in pending if key[0] == name]
    return min(s for s, _ in spans), max(e for _, e in spans)
