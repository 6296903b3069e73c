"""B200-native (sm_100a) causal FlashAttention-2 with the public surface of flash-attention-triton.

Exports the same four names as the reference package (``src/flash_attention_triton/__init__.py:13``)
plus the autograd function.
"""

from .api import (
    FlashAttentionV2Function,
    KernelsConfigV2,
    flash_attention_v2,
    flash_attention_v2_custom,
    init_to_zero_v2,
)
from .partition import shard_range, shard_slab

__version__ = "0.1.0"

__all__ = [
    "FlashAttentionV2Function",
    "KernelsConfigV2",
    "flash_attention_v2",
    "flash_attention_v2_custom",
    "init_to_zero_v2",
    "shard_range",
    "shard_slab",
]
