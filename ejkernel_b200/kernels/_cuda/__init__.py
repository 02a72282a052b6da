"""CUDA platform implementations (the reference ships this package empty:
ejkernel/kernels/_cuda/__init__.py:1-15)."""

from .ragged_page_attention import ragged_page_attention

__all__ = ["ragged_page_attention"]
