"""Reference: orchestrated_attn/utils.py (data carriers :34-298, communication wrappers :300-380)."""
from ultraattn_b200.parallel.communicator import (InterComm, InterComm_fused, IntraComm,  # noqa: F401
                                                  IntraComm_fused)
from ultraattn_b200.runtime.orchestrated import (Input_Col_Bwd, Input_Col_Fwd, Input_Row_Bwd,  # noqa: F401
                                                 Input_Row_Fwd, Integrated_Data, Output_Col_Bwd,
                                                 Output_Col_Fwd, Output_Row_Bwd, Output_Row_Fwd)
from ultraattn_b200.utils.misc import print_rank_0  # noqa: F401,E402

Comm_Fused = IntraComm_fused        # the reference's common base of the row / column collectives


def get_Q_shape_from_da_config(da_config, batch_degree: int) -> tuple:
    """Shape of a query-side tile that covers ``batch_degree`` partitions."""
    return (da_config.bs, da_config.S_per_partition[0] * batch_degree, da_config.Nh[0], da_config.D)


def get_K_shape_from_da_config(da_config, batch_degree: int) -> tuple:
    """Shape of a key-side tile (the reference sizes it with the query head count, utils.py:28-29)."""
    return (da_config.bs, da_config.S_per_partition[1] * batch_degree, da_config.Nh[0], da_config.D)


def get_lse_shape_from_da_config(da_config, batch_degree: int) -> tuple:
    return (da_config.bs, da_config.Nh[0], da_config.S_per_partition[0] * batch_degree)
