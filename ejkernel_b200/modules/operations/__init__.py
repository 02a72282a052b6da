from .configs import BaseOperationConfig, RaggedPageAttentionConfig
from .ragged_page_attention import RaggedPageAttention, ragged_page_attention

__all__ = ["BaseOperationConfig", "RaggedPageAttention", "RaggedPageAttentionConfig", "ragged_page_attention"]
