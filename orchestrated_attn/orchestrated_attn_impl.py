"""Reference: orchestrated_attn/orchestrated_attn_impl.py (general executor :62-213, kernel-tile
path :222-298 / :433-552, entry points :622-792)."""
from ultraattn_b200.runtime.executor import PlanExecutor  # noqa: F401
from ultraattn_b200.runtime.grid import GridExecutor  # noqa: F401
from ultraattn_b200.runtime.orchestrated import (OrchestratedAttnFunc, orchestrated_attn_backward,  # noqa: F401
                                                 orchestrated_attn_func)

orchestrated_attn_forward = orchestrated_attn_func


def fused_attn_forward(execution_plan, inp_row, inp_col, softmax_scale=None, group=None, **kw):
    """Kernel-tile forward of a ``Fused_Execution_Plan``: carriers in, ``Output_Row_Fwd`` out."""
    return orchestrated_attn_func(inp_row, inp_col, softmax_scale=softmax_scale,
                                  execution_plan_dict={"fused": execution_plan, "group": group}, **kw)


def fused_attn_backward(execution_plan, inp_row, inp_col, out_fwd, softmax_scale=None, group=None, **kw):
    """Kernel-tile backward: returns ``(Output_Row_Bwd, Output_Col_Bwd)``."""
    return orchestrated_attn_backward(inp_row, inp_col, out_fwd, softmax_scale=softmax_scale,
                                      execution_plan_dict={"fused": execution_plan, "group": group}, **kw)


intra_attn_forward = orchestrated_attn_func
intra_attn_backward = orchestrated_attn_backward


def stream_wait_event(stream, event) -> None:
    """Make a stream, or both streams of a pair, wait for an event (reference: :215-220)."""
    for s in (stream if isinstance(stream, (list, tuple)) else [stream]):
        s.wait_event(event)
