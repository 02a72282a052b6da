from ._interface import ragged_page_attention_v3

__all__ = ["ragged_page_attention_v3"]
