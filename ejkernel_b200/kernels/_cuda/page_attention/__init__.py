from ._interface import page_attention

__all__ = ["page_attention"]
