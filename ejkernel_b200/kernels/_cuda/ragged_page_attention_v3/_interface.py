"""CUDA (sm_100a) implementation of ``ragged_page_attention_v3``: the step's new key/value rows are
written into the paged KV cache, then the batch attends against the updated cache.

Registered as ``("ragged_page_attention_v3", Platform.CUDA, Backend.GPU)`` with the parameters of the
reference's XLA entry (ejkernel/kernels/_xla/ragged_page_attention_v3/_interface.py:24-49) and the
semantics of its kernel (ejkernel/kernels/_xla/ragged_page_attention_v3/_kernel.py:143-318):

  * ``kv_cache`` is ``[num_pages, page_size, 2*Hkv/pack, pack, head_dim_padded]`` with ``pack = 32 /
    bitwidth`` (2 for bf16/f16); ``merge_kv`` (:45-57) puts ``K_h`` at combined head ``2h`` and ``V_h`` at
    ``2h+1``, so its bytes are those of the ``[num_pages, page_size, 2*Hkv, head_dim]`` cache of
    ``ragged_page_attention``;
  * query row ``r`` of sequence ``s`` and its new K/V row go to position ``kv_len - q_len + r`` (:227-229),
    i.e. ``kv_lens`` already counts the new tokens;
  * ``block_tables`` is flat ``[max_num_seqs * pages_per_seq]``; ``distribution[2]`` is the number of
    sequences (:211);
  * ``softmax_scale`` defaults to 1.0 (sic); ``k_scale`` multiplies the logits, ``v_scale`` the output, in
    float32 before the cast to the output dtype (:262-263, :283-291).  ``q_scale`` divides the queries, which are
    then clipped to the finite range of the cache dtype and cast to it, and multiplies the logits back (:249-265);
  * the cache may be float8 e4m3 (``torch.float8_e4m3fn``) with ``keys`` / ``values`` of the same dtype and 16-bit
    ``queries``: ``pack`` is then 4.  Without ``q_scale`` the keys are widened to f16 for Q.K^T; with it Q.K^T runs
    on e4m3 operands.  The probabilities go into P.V as e4m3, as in the reference (:281), but unnormalised
    (``exp(s - m)`` against a running reference ``m``, values in (0, 256]) where the reference rounds the
    normalised ones -- which flushes every probability below 2^-10 to zero, i.e. most of a long context.

The cache is updated IN PLACE and returned (the reference donates it, :141).  A ``head_dim`` that is not
a multiple of 128 lives in a cache padded to one (``align_to(D, 128)``, :45-57): the page write zero-fills
the padding of the rows it writes, the attention kernels step over it.  There is no CPU fallback.
"""

from __future__ import annotations

import ctypes

import torch
from jaxtyping import Float, Int32
from torch import Tensor as Array

from .... import _cabi
from .._typecheck import typechecked_once
from ..._registry import Backend, Platform, kernel_registry
from ..ragged_page_attention._interface import _DTYPE_CODE, FP8, cached_workspace


def _packing(dtype: torch.dtype) -> int:
    return 32 // (torch.finfo(dtype).bits)  # get_dtype_packing, _kernel.py:38-39


@kernel_registry.register("ragged_page_attention_v3", Platform.CUDA, Backend.GPU)
@typechecked_once
def ragged_page_attention_v3(
    queries: Float[Array, "total_tokens num_q_heads head_dim"],
    keys: Float[Array, "total_tokens num_kv_heads head_dim"],
    values: Float[Array, "total_tokens num_kv_heads head_dim"],
    kv_cache: Float[Array, "num_pages page_size num_kv_heads_x2_per_kv_packing kv_packing head_dim_padded"],
    kv_lens: Int32[Array, "max_num_seqs"],
    block_tables: Int32[Array, "max_num_seqs_times_pages_per_seq"],
    query_start_loc: Int32[Array, "max_num_seqs_plus_1"],
    distribution: Int32[Array, "3"],
    *,
    softmax_scale: float = 1.0,
    sliding_window: int | None = None,
    logits_soft_cap: float | None = None,
    q_scale: float | None = None,
    k_scale: float | None = None,
    v_scale: float | None = None,
    chunk_prefill_size: int | None = None,
    num_kv_pages_per_block: int | None = None,
    num_queries_per_block: int | None = None,
    vmem_limit_bytes: int | None = None,
) -> tuple[
    Float[Array, "total_tokens num_q_heads head_dim"],
    Float[Array, "num_pages page_size num_kv_heads_x2_per_kv_packing kv_packing head_dim_padded"],
]:
    """Returns ``(out, kv_cache)``; ``kv_cache`` is the same tensor, updated in place."""
    del chunk_prefill_size, num_kv_pages_per_block, num_queries_per_block, vmem_limit_bytes
    # static half of the reference's contract (_kernel.py:73-126)
    if not queries.is_cuda:
        raise RuntimeError("ragged_page_attention_v3[cuda]: tensors must live on a CUDA device (no CPU fallback)")
    T, Hq, D = queries.shape
    if keys.shape != values.shape or keys.shape[0] != T or keys.shape[2] != D:
        raise ValueError("shape mismatch among q,k,v")
    Hkv = keys.shape[1]
    if Hq % Hkv != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    P, page_size, hx2_per_pack, pack, d_align = kv_cache.shape
    if queries.dtype not in _DTYPE_CODE:
        raise NotImplementedError("queries must be bf16 or f16")
    if kv_cache.dtype not in (queries.dtype, FP8) or keys.dtype != kv_cache.dtype or values.dtype != kv_cache.dtype:
        raise NotImplementedError("keys, values and kv_cache must share one dtype: that of the queries, or float8_e4m3fn")
    fp8 = kv_cache.dtype == FP8
    if fp8 and (D not in (64, 128, 256) or page_size % 8):
        raise NotImplementedError("an e4m3 KV cache needs head_dim 64, 128 or 256 and a page size that is a multiple of 8")
    for name, sc in (("q_scale", q_scale), ("k_scale", k_scale), ("v_scale", v_scale)):
        if sc is not None and not (sc > 0.0 and sc < float("inf")):
            raise ValueError(f"{name} must be positive and finite")
    if pack != _packing(kv_cache.dtype):
        raise ValueError("packing mismatch")
    if d_align != -(-D // 128) * 128:
        raise ValueError("cache last dim must be align_to(D,128)")
    if hx2_per_pack * pack != -(-2 * Hkv // pack) * pack:
        raise ValueError("cache combined-head axis must be align_to(2*num_kv_heads, packing)")  # merge_kv, _kernel.py:45-57
    S_max = kv_lens.shape[0]
    if block_tables.numel() % S_max != 0:
        raise ValueError("block_tables size % num_seqs != 0")
    if query_start_loc.shape != (S_max + 1,):
        raise ValueError("query_start_loc bad shape")
    if page_size % pack != 0:
        raise ValueError("page_size must be divisible by packing")
    if sliding_window is not None and sliding_window <= 0:
        raise ValueError("sliding_window > 0")
    if logits_soft_cap is not None and logits_soft_cap == 0.0:
        raise ValueError("soft_cap != 0")
    for name, t in (("queries", queries), ("keys", keys), ("values", values), ("kv_cache", kv_cache),
                    ("kv_lens", kv_lens), ("block_tables", block_tables), ("query_start_loc", query_start_loc),
                    ("distribution", distribution)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
        if t.device != queries.device:
            raise ValueError(f"{name} is on {t.device}, queries on {queries.device}")

    pps = block_tables.numel() // S_max
    shape = _cabi.Shape(T, S_max, pps, P, page_size, Hq, Hkv, D, _DTYPE_CODE[queries.dtype], _cabi.E4M3 if fp8 else 0)
    device = queries.device
    ws = cached_workspace(shape, device)
    # the logits are (q / q_scale) . k * softmax_scale * k_scale * q_scale (:259-265): one factor for the kernel
    scale = float(softmax_scale) * (1.0 if k_scale is None else float(k_scale)) * (1.0 if q_scale is None else float(q_scale))
    attrs = _cabi.Attrs(scale, 0.0 if logits_soft_cap is None else float(logits_soft_cap),
                        0 if sliding_window is None else int(sliding_window), 0, 0, 0, 0,
                        0.0 if q_scale is None else float(q_scale),
                        0.0 if v_scale is None else float(v_scale))  # v_scale: in float32, before the output cast
    out = torch.empty_like(queries)
    with torch.cuda.device(device):
        rc = _cabi.load().ejk_rpa_v3_launch(
            queries.data_ptr(), keys.data_ptr(), values.data_ptr(), kv_cache.data_ptr(), kv_lens.data_ptr(),
            block_tables.data_ptr(), query_start_loc.data_ptr(), distribution.data_ptr(), out.data_ptr(),
            ws.buffer.data_ptr(), ws.nbytes, ws.status.data_ptr(), ctypes.byref(shape), ctypes.byref(attrs),
            torch.cuda.current_stream(device).cuda_stream,
        )
    _cabi.check(rc, "ejk_rpa_v3_launch")
    return out, kv_cache
