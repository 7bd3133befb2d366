"""Reference: search_algo/benchmark.py.

``benchmark_orchestrate_bsa`` accepts the reference's argument list (``args, raw_f, da_config,
exp_config, tensor_buf, inter_bsa_execution_plans, inter_comp_plans_dicts, ...``) as well as this
framework's short form (``plan_fwd, plan_bwd, fob, device, ...``)."""
from ultraattn_b200.drivers import benchmark as _bench
from ultraattn_b200.drivers.benchmark import benchmark_ops  # noqa: F401
from ultraattn_b200.drivers.task2 import prepare_inter_comp_plans  # noqa: F401
from ultraattn_b200.runtime.orchestrated import create_buf_dict  # noqa: F401


def benchmark_orchestrate_bsa(*args, **kw):
    first = args[0] if args else kw.get("plan_fwd")
    if hasattr(first, "gpu_kernel_lists"):               # an Execution_Plan: the short form
        return _bench.benchmark_orchestrate_bsa(*args, **kw)
    return _bench.benchmark_orchestrate_bsa_reference_form(*args, **kw)
