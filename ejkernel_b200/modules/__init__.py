"""Public operator API, mirroring ``ejkernel.modules`` for the one operator this package covers."""

from .operations import RaggedPageAttention, RaggedPageAttentionConfig, ragged_page_attention

__all__ = ["RaggedPageAttention", "RaggedPageAttentionConfig", "ragged_page_attention"]
