"""B200-native attention kernels behind the reference's public names
(kernels/__init__.py:1-51 of the reference; only the attention hot path and its closest sibling, the row softmax, are provided)."""
from .attention import (
    flash_attention_v1,
    flash_attention_v2,
)
from .decode import decode_attention
from .paged_cache import append_paged_kv
from .softmax import (
    log_softmax,
    softmax,
)
from .speculative_decode import (
    speculative_decode_attention,
)

__all__ = [
    "flash_attention_v1",
    "flash_attention_v2",
    "speculative_decode_attention",
    "decode_attention",
    "append_paged_kv",
    "softmax",
    "log_softmax",
]
