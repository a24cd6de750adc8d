"""B200-native flash attention (forward + backward) with an optional trainable bias.

Public interface (same names and signatures as the reference project):
    flash_attention_fn, flash_attention_qkvpacked_fn,
    FlashAttentionFn, FlashAttentionQKVPackedFn
plus, with no counterpart in the reference: FlashAttention (nn.Module), flash_attention_op
(the same call through torch.library operators) and shard_batch_heads.
"""
from .flash_attention import (  # noqa: F401
    FlashAttentionFn,
    FlashAttentionQKVPackedFn,
    flash_attention_fn,
    flash_attention_qkvpacked_fn,
)
from .module import FlashAttention, flash_attention_op  # noqa: F401
from .sharding import shard_batch_heads  # noqa: F401

__all__ = [
    "FlashAttentionFn",
    "FlashAttentionQKVPackedFn",
    "flash_attention_fn",
    "flash_attention_qkvpacked_fn",
    "FlashAttention",
    "flash_attention_op",
    "shard_batch_heads",
]
