"""Reference: search_algo/initialize.py."""
from ultraattn_b200.parallel import comm as _comm
from ultraattn_b200.parallel.comm import (PROC_INFO, get_proc_info, initialize_prof_db,  # noqa: F401
                                          parse_slurm_tasks_per_node)


def initialize_distribution(*args, **kw):
    """Start torch.distributed and the control-plane groups; returns, like the reference
    (initialize.py:92-159), ``(communicator over all ranks, gloo group of all ranks)``. The process
    information lands in ``PROC_INFO`` (also ``search_algo.global_vars.get_global_var('PROC_INFO')``).
    ``ultraattn_b200.parallel.comm.initialize_distribution`` is the form that returns that dict."""
    from search_algo.global_vars import set_global_var
    from ultraattn_b200.parallel.communicator import StreamCommunicator
    info = _comm.initialize_distribution(*args, **kw)
    set_global_var("PROC_INFO", dict(info))
    import torch.distributed as dist
    world = StreamCommunicator(list(range(info["world_size"])), group=dist.group.WORLD)
    return world, _comm.control_group()
