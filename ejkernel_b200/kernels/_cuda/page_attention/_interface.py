"""CUDA (sm_100a) implementation of ``page_attention``: decode-only attention over separate paged
key and value caches.

Registered as ``("page_attention", Platform.CUDA, Backend.GPU)`` with the parameters of the reference's
XLA entry (ejkernel/kernels/_xla/page_attention/_interface.py:27-42).  Semantics
(ejkernel/kernels/_xla/page_attention/_xla_impl_fwd.py:22-97): ``query [num_seqs, Hq, D]`` holds one row
per sequence, token ``j`` of sequence ``s`` lives in block ``block_tables[s, j // block_size]`` of
``key_cache`` / ``value_cache [num_blocks, Hkv, block_size, D]``, keys ``j < context_lens[s]`` are
visible, logits are ``(q . k) * attn_scale`` (default ``D ** -0.5``), optionally soft-capped
(``attn_logits_soft_cap``, honoured here as in the reference's Triton kernel; the XLA path ignores
it).  ``max_context_len``, ``num_splits``, ``mask_value``, ``pages_per_compute_block``,
``megacore_mode`` and ``inline_seq_dim`` are accepted and ignored as the XLA entry ignores them: the
split of long contexts is chosen on the device.

It runs the same split-KV kernels as ``ragged_page_attention`` through a tensor map over the split
layout (``ejk_page_attention_launch``); a ``block_size`` that is not a multiple of 8 goes through
the cp.async gather instead (slower).  A sequence
with ``context_len == 0`` yields zeros (the reference's softmax over all-masked scores would average
stale blocks).  There is no CPU fallback.
"""

from __future__ import annotations

import ctypes
import math

import torch
from jaxtyping import Float, Int
from torch import Tensor as Array

from .... import _cabi
from .._typecheck import typechecked_once
from ..._registry import Backend, Platform, kernel_registry
from ..ragged_page_attention._interface import _DTYPE_CODE, cached_workspace


@kernel_registry.register("page_attention", Platform.CUDA, Backend.GPU)
@typechecked_once
def page_attention(
    query: Float[Array, "num_seqs num_heads head_dim"],
    key_cache: Float[Array, "num_blocks num_kv_heads block_size head_dim"],
    value_cache: Float[Array, "num_blocks num_kv_heads block_size head_dim"],
    context_lens: Int[Array, "num_seqs"],
    block_tables: Int[Array, "num_seqs max_blocks"],
    attn_scale: float | None = None,
    max_context_len: int | None = None,
    num_splits: int = 0,
    *,
    mask_value: float = -2.381976426469702e38,
    attn_logits_soft_cap: float | None = None,
    pages_per_compute_block: int | None = None,
    megacore_mode: str | None = None,
    inline_seq_dim: bool = True,
) -> Float[Array, "num_seqs num_heads head_dim"]:
    del max_context_len, num_splits, mask_value, pages_per_compute_block, megacore_mode, inline_seq_dim
    if not query.is_cuda:
        raise RuntimeError("page_attention[cuda]: tensors must live on a CUDA device (no CPU fallback)")
    if query.dtype not in _DTYPE_CODE or key_cache.dtype != query.dtype or value_cache.dtype != query.dtype:
        raise NotImplementedError("query, key_cache and value_cache must share one 16-bit float dtype (bf16/f16)")
    S, Hq, D = query.shape
    P, Hkv, block_size, _ = key_cache.shape
    if Hq % Hkv != 0:
        raise ValueError(f"num_heads={Hq} must be divisible by num_kv_heads={Hkv}")
    if D not in (64, 128, 256):
        raise NotImplementedError(f"head_dim={D} is not supported by the CUDA path (64, 128, 256)")
    if context_lens.dtype != torch.int32 or block_tables.dtype != torch.int32:
        raise ValueError("context_lens and block_tables must be int32")
    if attn_logits_soft_cap is not None and attn_logits_soft_cap == 0.0:
        raise ValueError("attn_logits_soft_cap must not be 0.0")
    for name, t in (("query", query), ("key_cache", key_cache), ("value_cache", value_cache),
                    ("context_lens", context_lens), ("block_tables", block_tables)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
        if t.device != query.device:
            raise ValueError(f"{name} is on {t.device}, query on {query.device}")
    scale = D**-0.5 if attn_scale is None else float(attn_scale)
    if not math.isfinite(scale):
        raise ValueError(f"{attn_scale=} must be finite")

    device = query.device
    shape = _cabi.Shape(S, S, block_tables.shape[1], P, block_size, Hq, Hkv, D, _DTYPE_CODE[query.dtype])
    ws = cached_workspace(shape, device)
    attrs = _cabi.Attrs(scale, 0.0 if attn_logits_soft_cap is None else float(attn_logits_soft_cap), 0, 0, 0, 0, 0)
    out = torch.empty_like(query)  # one row per sequence, every row is written
    with torch.cuda.device(device):
        rc = _cabi.load().ejk_page_attention_launch(
            query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), context_lens.data_ptr(),
            block_tables.data_ptr(), out.data_ptr(), ws.buffer.data_ptr(), ws.nbytes, ws.status.data_ptr(),
            ctypes.byref(shape), ctypes.byref(attrs), torch.cuda.current_stream(device).cuda_stream,
        )
    _cabi.check(rc, "ejk_page_attention_launch")
    return out
