"""Reference: easy_context/dist_flash_attn/async_communication.py."""
from ultraattn_b200.parallel.lightseq import (_initialize_sequence_parallel, destroy_sequence_parallel,  # noqa: F401
                                              get_sequence_parallel_group, get_sequence_parallel_rank,
                                              get_sequence_parallel_size, initialize_distributed,
                                              is_compute_for_local_query, is_idle, is_last_time,
                                              is_sync_from_remote, print_and_reset_comm_stats)
