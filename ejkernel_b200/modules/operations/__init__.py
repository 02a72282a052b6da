from .configs import BaseOperationConfig, RaggedPageAttentionConfig
from .page_attention import PageAttentionConfig, page_attention
from .ragged_page_attention import RaggedPageAttention, ragged_page_attention
from .ragged_page_attention_v3 import RaggedPageAttentionv3Config, ragged_page_attention_v3

__all__ = [
    "BaseOperationConfig",
    "PageAttentionConfig",
    "page_attention",
    "RaggedPageAttention",
    "RaggedPageAttentionConfig",
    "RaggedPageAttentionv3Config",
    "ragged_page_attention",
    "ragged_page_attention_v3",
]
