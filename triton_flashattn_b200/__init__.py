"""B200-native flash attention (forward + backward) with an optional trainable bias.

Public interface (same names and signatures as the reference project):
    flash_attention_fn, flash_attention_qkvpacked_fn,
    FlashAttentionFn, FlashAttentionQKVPackedFn
"""
from .flash_attention import (  # noqa: F401
    FlashAttentionFn,
    FlashAttentionQKVPackedFn,
    flash_attention_fn,
    flash_attention_qkvpacked_fn,
)
from .sharding import shard_batch_heads  # noqa: F401

__all__ = [
    "FlashAttentionFn",
    "FlashAttentionQKVPackedFn",
    "flash_attention_fn",
    "flash_attention_qkvpacked_fn",
    "shard_batch_heads",
]
