"""CUDA platform implementations (the reference ships this package empty:
ejkernel/kernels/_cuda/__init__.py:1-15)."""

from .page_attention import page_attention
from .ragged_page_attention import ragged_page_attention
from .ragged_page_attention_v3 import ragged_page_attention_v3

__all__ = ["page_attention", "ragged_page_attention", "ragged_page_attention_v3"]
