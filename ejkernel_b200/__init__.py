"""B200-native (sm_100a) ragged paged attention behind the ejkernel operator API.

Importing the package does not touch CUDA; the compiled library is loaded on the first call and
its absence is an error, never a silent fallback.
"""

__version__ = "0.1.0"

from . import kernels, modules  # noqa: F401
from .kernels import Backend, Platform, kernel_registry
from .modules import page_attention, RaggedPageAttention, RaggedPageAttentionConfig, ragged_page_attention, ragged_page_attention_v3

__all__ = [
    "Backend",
    "Platform",
    "RaggedPageAttention",
    "RaggedPageAttentionConfig",
    "kernel_registry",
    "page_attention",
    "ragged_page_attention",
    "ragged_page_attention_v3",
]
