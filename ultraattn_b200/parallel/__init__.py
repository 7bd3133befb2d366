from .comm import A2AComm, PROC_INFO, RingComm, get_proc_info, initialize_distribution
from .communicator import (CommRegistry, InterComm, InterComm_fused, IntraComm, IntraComm_fused,
                           PyNcclCommunicator, StreamCommunicator)
from .hierarchy import create_hierarchy_groups, hierarchy_attn_func
from .halo import HaloWindowAttnFunc, halo_window_attn_func  # noqa: F401
from .ring import (block_sparse_ring_attn_func, deepspeed_ulysses_attn_func, ring_backward, ring_flash_attn_func,
                   ring_flash_attn_kvpacked_func, ring_flash_attn_qkvpacked_func,
                   ring_flash_attn_varlen_func, ring_flash_attn_varlen_kvpacked_func,
                   ring_flash_attn_varlen_qkvpacked_func, ring_forward, shard_packed, shard_sequence,
                   stripe_flash_attn_func, stripe_flash_attn_kvpacked_func,
                   stripe_flash_attn_qkvpacked_func, zigzag_ring_flash_attn_func,
                   zigzag_ring_flash_attn_kvpacked_func, zigzag_ring_flash_attn_qkvpacked_func,
                   zigzag_ring_flash_attn_varlen_func, zigzag_ring_flash_attn_varlen_kvpacked_func,
                   zigzag_ring_flash_attn_varlen_qkvpacked_func)
