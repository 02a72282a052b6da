"""Public operator API, mirroring ``ejkernel.modules`` for the operators this package covers."""

from .operations import (
    PageAttentionConfig,
    page_attention,
    RaggedPageAttention,
    RaggedPageAttentionConfig,
    RaggedPageAttentionv3Config,
    ragged_page_attention,
    ragged_page_attention_v3,
)

__all__ = [
    "PageAttentionConfig",
    "page_attention",
    "RaggedPageAttention",
    "RaggedPageAttentionConfig",
    "RaggedPageAttentionv3Config",
    "ragged_page_attention",
    "ragged_page_attention_v3",
]
