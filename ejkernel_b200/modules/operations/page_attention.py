"""Public ``page_attention`` operator (decode over separate paged K / V caches).

Mirrors the module-level function of ejkernel/modules/operations/page_attention.py:364-382: five
positional-only arrays and the same keywords.  One implementation (CUDA); any other ``platform`` raises.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

import torch

from ...kernels._registry import Backend, kernel_registry
from .configs import BaseOperationConfig
from .ragged_page_attention import _resolve_platform

Array = torch.Tensor


@dataclass
class PageAttentionConfig(BaseOperationConfig):
    """Fields of the reference's ``PageAttentionConfig``; the CUDA path chooses its KV split on the device."""

    num_splits: int = 0
    pages_per_compute_block: int | None = None
    num_warps: int = 4
    num_stages: int = 1


def page_attention(
    query: Array,
    key_cache: Array,
    value_cache: Array,
    context_lens: Array,
    block_tables: Array,
    /,
    *,
    attn_scale: float | None = None,
    max_context_len: int | None = None,
    num_splits: int = 0,
    mask_value: float = -2.381976426469702e38,
    attn_logits_soft_cap: float | None = None,
    pages_per_compute_block: int | None = None,
    megacore_mode: str | None = None,
    inline_seq_dim: bool = True,
    platform: Literal["triton", "pallas", "cuda", "xla", "auto"] | None = None,
    cfg: PageAttentionConfig | None = None,
) -> Array:
    del cfg
    impl = kernel_registry.get("page_attention", platform=_resolve_platform(platform), backend=Backend.GPU)
    return impl(
        query, key_cache, value_cache, context_lens, block_tables, attn_scale, max_context_len, num_splits,
        mask_value=mask_value, attn_logits_soft_cap=attn_logits_soft_cap,
        pages_per_compute_block=pages_per_compute_block, megacore_mode=megacore_mode, inline_seq_dim=inline_seq_dim,
    )
