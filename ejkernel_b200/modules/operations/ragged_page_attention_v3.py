"""Public ``ragged_page_attention_v3`` operator (KV-cache page write fused with attention).

Mirrors the module-level function of ejkernel/modules/operations/ragged_page_attention_v3.py:787-813:
eight positional-only arrays, the same keywords, returns ``(out, kv_cache)``.  There is one
implementation (CUDA); any other ``platform`` raises.  Sharding by KV heads works exactly as for
``ragged_page_attention``: every rank passes its local head shard of q/k/v and of the cache.
"""

from __future__ import annotations

from typing import Literal

import torch

from ...kernels._registry import Backend, kernel_registry
from ...sharding import Mesh1D, PartitionSpec, all_gather_heads
from .configs import RaggedPageAttentionConfig
from .ragged_page_attention import _resolve_platform

Array = torch.Tensor


class RaggedPageAttentionv3Config(RaggedPageAttentionConfig):
    """Same tile hints as the v1 config (reference: configs.py, ``RaggedPageAttentionv3Config``)."""


def ragged_page_attention_v3(
    queries: Array,
    keys: Array,
    values: Array,
    kv_cache: Array,
    kv_lens: Array,
    block_tables: Array,
    query_start_loc: Array,
    distribution: Array,
    /,
    *,
    softmax_scale: float = 1.0,
    sliding_window: int | None = None,
    logits_soft_cap: float | None = None,
    q_scale: float | None = None,
    k_scale: float | None = None,
    v_scale: float | None = None,
    vmem_limit_bytes: int | None = None,
    platform: Literal["triton", "pallas", "cuda", "xla", "auto"] | None = None,
    cfg: RaggedPageAttentionv3Config | None = None,
    mesh: Mesh1D | None = None,
    in_specs: tuple[PartitionSpec | None, ...] | None = None,
    out_specs: PartitionSpec | None = None,
) -> tuple[Array, Array]:
    impl = kernel_registry.get("ragged_page_attention_v3", platform=_resolve_platform(platform), backend=Backend.GPU)
    out, cache = impl(
        queries, keys, values, kv_cache, kv_lens, block_tables, query_start_loc, distribution,
        softmax_scale=softmax_scale, sliding_window=sliding_window, logits_soft_cap=logits_soft_cap,
        q_scale=q_scale, k_scale=k_scale, v_scale=v_scale, vmem_limit_bytes=vmem_limit_bytes,
        num_kv_pages_per_block=None if cfg is None else cfg.num_kv_pages_per_block,
        num_queries_per_block=None if cfg is None else cfg.num_queries_per_block,
    )
    if mesh is not None and in_specs is not None and out_specs is not None and mesh.size > 1:
        o_spec = out_specs[0] if isinstance(out_specs, (tuple, list)) and out_specs and isinstance(out_specs[0], tuple) else out_specs
        if PartitionSpec(*o_spec).sharded_dim(mesh.axis_name) is None:
            out = all_gather_heads(out, mesh)
    return out, cache
