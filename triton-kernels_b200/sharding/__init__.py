from .gather import all_gather_outputs, all_gather_ragged
from .planner import balance_sequences, batch_head_units, contiguous_shard, kv_head_shard

__all__ = [
    "all_gather_outputs",
    "all_gather_ragged",
    "balance_sequences",
    "batch_head_units",
    "contiguous_shard",
    "kv_head_shard",
]
