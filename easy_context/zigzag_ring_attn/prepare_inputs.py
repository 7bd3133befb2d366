"""Reference: easy_context/zigzag_ring_attn/prepare_inputs.py."""
from ultraattn_b200.models.glue import prepare_zigzag_ring_attn_inputs  # noqa: F401
from ultraattn_b200.parallel.ring import shard_sequence as _shard


def extract_local(value, rank, world_size, device=None, dim=1):
    """This rank's zigzag shard of ``value`` along ``dim`` (chunks ``rank`` and ``2 * world_size - 1 - rank``
    of ``2 * world_size``), optionally moved to ``device`` (reference: prepare_inputs.py:4-13)."""
    out = _shard(value, rank, world_size, "zigzag", dim=dim)
    return out if device is None else out.to(device)
