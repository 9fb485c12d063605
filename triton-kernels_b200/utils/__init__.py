from .launch_config import (
    decode_chunk_tokens,
    decode_items,
    decode_plan,
    paged_box_rows,
    prefill_items,
)
from .validation import (
    AttentionProblem,
    detect_layout,
    validate_decode,
    validate_prefill,
)

__all__ = [
    "AttentionProblem",
    "decode_chunk_tokens",
    "decode_items",
    "decode_plan",
    "detect_layout",
    "paged_box_rows",
    "prefill_items",
    "validate_decode",
    "validate_prefill",
]
