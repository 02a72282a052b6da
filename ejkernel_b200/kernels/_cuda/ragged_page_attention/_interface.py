"""CUDA (sm_100a) implementation of ``ragged_page_attention``.

Registered as ``("ragged_page_attention", Platform.CUDA, Backend.GPU)`` with the parameter
names, order, kinds and defaults of the reference's XLA entry
(ejkernel/kernels/_xla/ragged_page_attention/_interface.py:25-109) so that
``kernel_registry.validate_signatures`` finds no mismatch.  Arrays are ``torch.Tensor`` on a
CUDA device where the reference takes ``jax.Array`` (JAX is not available to this build); the
default ``compute_dtype`` is therefore ``torch.bfloat16`` instead of ``jnp.bfloat16``.

The work is done by hand-written kernels behind the C ABI of ``include/ejk_rpa.h``; there is
no other code path -- without the compiled library or without an sm_100 GPU the call raises.

Semantics (reference lines in brackets):
  * ``kv_pages[p, t, 2h] = K_h``, ``kv_pages[p, t, 2h+1] = V_h``             [_xla_impl_fwd.py:113-114]
  * token j of sequence s lives in page ``block_tables[s, j // page_size]``   [:105-114]
  * query head h uses kv head ``h // (Hq // Hkv)``                            [:46]
  * row r of a sequence sits at position ``kv_len - q_len + r``               [:95-97]
  * key j is visible iff ``j <= pos`` and ``j > pos - sliding_window``         [:128-135]
  * logits = (q.k) * softmax_scale, then ``cap * tanh(x / cap)``, then mask   [:119-138]
  * softmax in fp32 over the visible keys; sinks add to the denominator only  [:161-172]
  * output has the dtype of ``queries``; rows past the last sequence are 0    [:197-201]
``compute_dtype`` below fp32 is not honoured for the carried softmax state: accumulation is
always fp32 (the reference's bf16 carry only loses accuracy).  float32 operands are accepted and, as
in the reference, cast to ``compute_dtype`` (bf16 by default) for the contractions; the result comes
back as float32.
"""

from __future__ import annotations

import ctypes
import math
import os
from collections import OrderedDict

import torch
from jaxtyping import Float, Int
from torch import Tensor as Array

from .... import _cabi
from .._typecheck import typechecked_once
from ..._registry import Backend, Platform, kernel_registry

DTypeLike = torch.dtype | str | None

_DTYPE_CODE = {torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}
FP8 = torch.float8_e4m3fn  # the 8-bit cache dtype (e4m3, no infinities, maximum 448)


class RpaWorkspace:
    """Scratch + status word for one static shape on one device, reusable across calls.

    Its size depends on array shapes only (never on the lengths inside ``context_lens``), which is
    what lets a tracing runtime allocate it ahead of time.
    """

    def __init__(self, shape: _cabi.Shape, device: torch.device, nbytes: int | None = None):
        if nbytes is None:
            nbytes = workspace_bytes(shape, device)
        self.shape = shape
        self.nbytes = nbytes
        self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        assert self.buffer.data_ptr() % 256 == 0


_need_cache: dict[tuple, int] = {}


def workspace_bytes(shape: _cabi.Shape, device: torch.device) -> int:
    """``ejk_rpa_workspace_bytes`` for this static shape on this device; remembered per (device, shape, option
    "waves"), so that the call path of a serving loop does not cross into the library for it every step."""
    key = (device.index, _cabi.get_option_cached("waves"), *[getattr(shape, f) for f, _ in shape._fields_])
    nbytes = _need_cache.get(key)
    if nbytes is None:
        with torch.cuda.device(device):
            nbytes = int(_cabi.load().ejk_rpa_workspace_bytes(ctypes.byref(shape)))
        if nbytes == 0:
            raise ValueError("ejk_rpa_workspace_bytes rejected the shape")
        if len(_need_cache) > 4096:
            _need_cache.clear()
        _need_cache[key] = nbytes
    return nbytes


# Workspaces of the operator entry points that own their scratch (the public operators; the ``*_into`` forms
# take the caller's).  One per (device, CUDA stream): calls on one stream are ordered and may share scratch,
# calls on different streams may run at the same time and must not.  A workspace serves every shape whose
# need fits into it and is replaced by a larger one (next power of two) when a call needs more, so a serving
# loop whose token count changes every step settles on one buffer instead of allocating one per shape; the
# least recently used entries are dropped beyond ``_WORKSPACE_CACHE_MAX`` streams.
_WORKSPACE_CACHE_MAX = 16
_workspace_cache: "OrderedDict[tuple[int, int], RpaWorkspace]" = OrderedDict()


def cached_workspace(shape: _cabi.Shape, device: torch.device) -> RpaWorkspace:
    need = workspace_bytes(shape, device)
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspace_cache.get(key)
    if ws is None or ws.nbytes < need:
        cap = 1 << max(16, (need - 1).bit_length())
        status = None if ws is None else ws.status  # a pending status bit survives the growth
        ws = RpaWorkspace(shape, device, cap)
        if status is not None:
            ws.status = status
        _workspace_cache[key] = ws
    _workspace_cache.move_to_end(key)
    while len(_workspace_cache) > _WORKSPACE_CACHE_MAX:
        _workspace_cache.popitem(last=False)
    ws.shape = shape
    return ws


def _shape_of(queries, kv_pages, block_tables) -> _cabi.Shape:
    T, Hq, D = queries.shape
    P, page, C2, _ = kv_pages.shape
    S_max, pps = block_tables.shape
    return _cabi.Shape(T, S_max, pps, P, page, Hq, C2 // 2, D, _DTYPE_CODE[queries.dtype],
                       _cabi.E4M3 if kv_pages.dtype == FP8 else 0)


def _validate(queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, *, sliding_window,
              logits_soft_cap, softmax_aux, num_kv_pages_per_block, num_queries_per_block, vmem_limit_bytes):
    """The static half of the reference's input contract
    (ejkernel/kernels/_pallas/tpu/ragged_page_attention/_pallas_impl_fwd.py:168-230); the
    data-dependent half (lengths, page ids) is checked on the device and reported through the
    status word."""
    if not queries.is_cuda:
        raise RuntimeError("ragged_page_attention[cuda]: tensors must live on a CUDA device (no CPU fallback)")
    for name, t in (("kv_pages", kv_pages), ("context_lens", context_lens), ("block_tables", block_tables),
                    ("query_start_loc", query_start_loc)):
        if t.device != queries.device:
            raise ValueError(f"{name} is on {t.device}, queries on {queries.device}")
    if queries.dtype not in _DTYPE_CODE:
        raise NotImplementedError(f"queries dtype {queries.dtype} is not supported by the CUDA path (bf16/f16 only)")
    if kv_pages.dtype != queries.dtype and kv_pages.dtype != FP8:
        raise NotImplementedError(f"kv_pages dtype {kv_pages.dtype} must equal queries dtype {queries.dtype} or be {FP8}")
    _, num_q_heads, head_dim = queries.shape
    _, page_size, num_combined_kv_heads, head_dim_k = kv_pages.shape
    if kv_pages.dtype == FP8:
        if head_dim not in (128, 256) or page_size % 8:
            raise NotImplementedError("an e4m3 KV cache needs head_dim 128 or 256 and a page size that is a multiple of 8")
    if num_combined_kv_heads % 2 != 0:
        raise ValueError(f"{num_combined_kv_heads=} must be even (K and V heads interleaved)")
    num_kv_heads = num_combined_kv_heads // 2
    max_num_seqs, pages_per_seq = block_tables.shape
    if head_dim_k != head_dim:
        raise ValueError(f"Q head_dim {head_dim} must be the same as that of K/V {head_dim_k}.")
    if head_dim not in (64, 128, 256):
        raise NotImplementedError(f"head_dim={head_dim} is not supported by the CUDA path (64, 128, 256)")
    if context_lens.shape != (max_num_seqs,):
        raise ValueError(f"Expected {context_lens.shape=} to be ({max_num_seqs},) where `max_num_seqs` is `block_tables.shape[0]`.")
    if query_start_loc.shape != (max_num_seqs + 1,):
        raise ValueError(f"Expected {query_start_loc.shape=} to be ({max_num_seqs + 1},) where `max_num_seqs` is `block_tables.shape[0]`.")
    if context_lens.dtype != torch.int32 or block_tables.dtype != torch.int32 or query_start_loc.dtype != torch.int32:
        raise ValueError(
            "The dtype of `context_lens`, `block_tables`, and `query_start_loc` must be int32. "
            f"Got {context_lens.dtype=}, {block_tables.dtype=}, {query_start_loc.dtype=}."
        )
    if num_q_heads % num_kv_heads != 0:
        raise ValueError(f"{num_q_heads=} must be divisible by {num_kv_heads=}")
    if sliding_window is not None and sliding_window <= 0:
        raise ValueError(f"{sliding_window=} must be positive.")
    if logits_soft_cap is not None and logits_soft_cap == 0.0:
        raise ValueError(f"{logits_soft_cap=} must not be 0.0.")
    if num_kv_pages_per_block is not None and not 0 < num_kv_pages_per_block <= pages_per_seq:
        raise ValueError(f"{num_kv_pages_per_block=} must be in range (0, {pages_per_seq}].")
    if num_queries_per_block is not None and num_queries_per_block <= 0:
        raise ValueError(f"{num_queries_per_block=} must be positive.")
    if vmem_limit_bytes is not None and vmem_limit_bytes <= 0:
        raise ValueError(f"{vmem_limit_bytes=} must be positive.")
    if softmax_aux is not None:
        if softmax_aux.ndim == 2:
            if softmax_aux.shape[0] not in (num_q_heads, num_kv_heads):
                raise ValueError(
                    f"softmax_aux first dim must be num_q_heads ({num_q_heads}) "
                    f"or num_kv_heads ({num_kv_heads}), got {tuple(softmax_aux.shape)}"
                )
        elif softmax_aux.ndim != 1:
            raise ValueError(f"Unsupported softmax_aux shape: {tuple(softmax_aux.shape)}")
    for name, t in (("queries", queries), ("kv_pages", kv_pages), ("context_lens", context_lens),
                    ("block_tables", block_tables), ("query_start_loc", query_start_loc)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous (dense row-major)")


_num_seqs_consts: dict[tuple[int, int], torch.Tensor] = {}


def _num_seqs_tensor(num_seqs, device) -> torch.Tensor:
    if isinstance(num_seqs, torch.Tensor):
        t = num_seqs.reshape(-1)[:1]
        if t.dtype != torch.int32:
            t = t.to(torch.int32)
        return t.to(device).contiguous()
    # a Python int: one small device constant per (device, value), made once (no per-call host-to-device copy)
    key = (device.index, int(num_seqs))
    t = _num_seqs_consts.get(key)
    if t is None:
        if len(_num_seqs_consts) > 4096:
            _num_seqs_consts.clear()
        t = _num_seqs_consts[key] = torch.tensor([int(num_seqs)], dtype=torch.int32, device=device)
    return t


def ragged_page_attention_into(
    out: torch.Tensor,
    workspace: RpaWorkspace,
    queries: torch.Tensor,
    kv_pages: torch.Tensor,
    context_lens: torch.Tensor,
    block_tables: torch.Tensor,
    query_start_loc: torch.Tensor,
    num_seqs: torch.Tensor,
    *,
    softmax_scale: float,
    logits_soft_cap: float | None = None,
    sliding_window: int | None = None,
    softmax_aux: torch.Tensor | None = None,
    num_kv_pages_per_block: int | None = None,
    num_queries_per_block: int | None = None,
    stream: torch.cuda.Stream | None = None,
) -> None:
    """Enqueue one call through the C ABI into caller-owned ``out`` and ``workspace``.

    Allocates nothing and never synchronises: this is the form an XLA custom-call handler or a
    serving loop uses.  ``softmax_aux`` must already be float32 ``[rows, n]``; ``num_seqs`` a
    device int32 tensor of one element.

    ``queries`` and ``out`` may live in pinned (page-locked) host memory instead of device memory: such memory is
    mapped into the device's address space, the kernels read the query rows once per work item and write every output
    row once, so a step whose queries come from and whose result goes to the host needs no staging copies for them
    (2 + 2 MB per step at 256 decode tokens of 32 heads; measured 0.73 -> 0.67 ms per step including the copies of
    the other operands).  The KV pool, the index arrays and the workspace must be device memory.
    """
    lib = _cabi.load()
    attrs = _cabi.Attrs(
        float(softmax_scale),
        0.0 if logits_soft_cap is None else float(logits_soft_cap),
        0 if sliding_window is None else int(sliding_window),
        0 if softmax_aux is None else int(softmax_aux.shape[-1]),
        0 if softmax_aux is None else int(softmax_aux.shape[0]),
        int(num_kv_pages_per_block or 0),
        int(num_queries_per_block or 0),
    )
    device = kv_pages.device  # the pool is always device memory; queries / out may be pinned host memory (see below)
    st = stream if stream is not None else torch.cuda.current_stream(device)
    with torch.cuda.device(device):
        rc = lib.ejk_rpa_launch(
            queries.data_ptr(),
            kv_pages.data_ptr(),
            context_lens.data_ptr(),
            block_tables.data_ptr(),
            query_start_loc.data_ptr(),
            num_seqs.data_ptr(),
            None if softmax_aux is None else softmax_aux.data_ptr(),
            out.data_ptr(),
            workspace.buffer.data_ptr(),
            workspace.nbytes,
            workspace.status.data_ptr(),
            ctypes.byref(workspace.shape),
            ctypes.byref(attrs),
            st.cuda_stream,
        )
    _cabi.check(rc, "ejk_rpa_launch")


def ragged_page_attention_static_scratch_into(
    out: torch.Tensor,
    status: torch.Tensor,
    queries: torch.Tensor,
    kv_pages: torch.Tensor,
    context_lens: torch.Tensor,
    block_tables: torch.Tensor,
    query_start_loc: torch.Tensor,
    num_seqs: torch.Tensor,
    *,
    softmax_scale: float,
    logits_soft_cap: float | None = None,
    sliding_window: int | None = None,
    softmax_aux: torch.Tensor | None = None,
    stream: torch.cuda.Stream | None = None,
) -> None:
    """Enqueue one call through ``ejk_rpa_launch_static_scratch``: like
    ``ragged_page_attention_into`` but with no workspace argument.

    For callers that cannot allocate device memory where they call from (a custom-call handler
    that only receives operand/result buffers, a host that forbids ``cudaMalloc`` outside its own
    pool, a path that must not risk an allocation-induced sync).  The scratch is a fixed 32 MiB
    array inside the library's device image; shapes that need more raise ``RpaLibraryError``
    (code ``E_SCRATCH``) -- use the workspace form for those.  All calls on a GPU share that
    array, so calls must not overlap on the device (keep them on one stream).  ``out`` (same
    shape/dtype as ``queries``) and ``status`` (int32 ``[1]``) are caller-owned, as are all inputs.
    """
    lib = _cabi.load()
    shape = _shape_of(queries, kv_pages, block_tables)
    attrs = _cabi.Attrs(
        float(softmax_scale),
        0.0 if logits_soft_cap is None else float(logits_soft_cap),
        0 if sliding_window is None else int(sliding_window),
        0 if softmax_aux is None else int(softmax_aux.shape[-1]),
        0 if softmax_aux is None else int(softmax_aux.shape[0]),
        0,
        0,
    )
    st = stream if stream is not None else torch.cuda.current_stream(queries.device)
    with torch.cuda.device(queries.device):
        rc = lib.ejk_rpa_launch_static_scratch(
            queries.data_ptr(), kv_pages.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(),
            query_start_loc.data_ptr(), num_seqs.data_ptr(),
            None if softmax_aux is None else softmax_aux.data_ptr(),
            out.data_ptr(), status.data_ptr(), ctypes.byref(shape), ctypes.byref(attrs), st.cuda_stream,
        )
    _cabi.check(rc, "ejk_rpa_launch_static_scratch")


@kernel_registry.register("ragged_page_attention", Platform.CUDA, Backend.GPU)
@typechecked_once
def ragged_page_attention(
    queries: Float[Array, "total_tokens num_q_heads head_dim"],
    kv_pages: Float[Array, "num_pages page_size num_combined_kv_heads head_dim"],
    context_lens: Int[Array, "num_seqs"],
    block_tables: Int[Array, "num_seqs pages_per_seq"],
    query_start_loc: Int[Array, "num_seqs_plus_one"],
    num_seqs: Array | int,
    *,
    softmax_scale: float | None = None,
    logits_soft_cap: float | None = None,
    compute_dtype: DTypeLike = torch.bfloat16,
    optimized: bool = False,
    sliding_window: int | None = None,
    softmax_aux: Float[Array, "num_kv_heads num_sinks"] | Float[Array, "num_sinks"] | None = None,
    mask_value: float | None = None,
    num_kv_pages_per_block: int | None = None,
    num_queries_per_block: int | None = None,
    vmem_limit_bytes: int | None = None,
    num_warps: int | None = None,
    num_stages: int | None = None,
) -> Float[Array, "total_tokens num_q_heads head_dim"]:
    """Paged attention for a ragged batch of decode and chunked-prefill tokens on sm_100a.

    Same contract as the reference's XLA operator
    (ejkernel/kernels/_xla/ragged_page_attention/_interface.py:27-109); ``mask_value``,
    ``vmem_limit_bytes``, ``num_warps``, ``num_stages``, ``optimized`` and ``compute_dtype`` are
    accepted and ignored exactly as the XLA entry ignores them (:93).  Returns a tensor with the
    shape and dtype of ``queries``.
    """
    del mask_value, num_warps, num_stages, optimized
    if queries.dtype == torch.float32 and kv_pages.dtype == torch.float32 and queries.is_cuda:
        # The reference casts float32 operands to ``compute_dtype`` before both contractions
        # (_xla_impl_fwd.py:121-122,148) and returns the dtype of ``queries``; the same is done here.
        # The cast walks the whole pool on every call: keep the cache in bf16/f16 for speed.
        cd = torch.bfloat16 if compute_dtype in (None, "bfloat16") else compute_dtype
        if cd not in _DTYPE_CODE:
            raise NotImplementedError(f"compute_dtype={compute_dtype} is not supported by the CUDA path (bf16/f16 only)")
        out16 = ragged_page_attention(
            queries.to(cd), kv_pages.to(cd), context_lens, block_tables, query_start_loc, num_seqs,
            softmax_scale=softmax_scale, logits_soft_cap=logits_soft_cap, compute_dtype=cd,
            sliding_window=sliding_window, softmax_aux=softmax_aux, num_kv_pages_per_block=num_kv_pages_per_block,
            num_queries_per_block=num_queries_per_block, vmem_limit_bytes=vmem_limit_bytes,
        )
        return out16.to(torch.float32)
    del compute_dtype
    _validate(
        queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs,
        sliding_window=sliding_window, logits_soft_cap=logits_soft_cap, softmax_aux=softmax_aux,
        num_kv_pages_per_block=num_kv_pages_per_block, num_queries_per_block=num_queries_per_block,
        vmem_limit_bytes=vmem_limit_bytes,
    )
    if softmax_scale is None:
        softmax_scale = queries.shape[-1] ** -0.5  # _interface.py:94-95
    if not math.isfinite(softmax_scale):
        raise ValueError(f"{softmax_scale=} must be finite")
    device = queries.device
    shape = _shape_of(queries, kv_pages, block_tables)
    ws = cached_workspace(shape, device)
    aux = None
    if softmax_aux is not None:
        aux = softmax_aux.to(device=device, dtype=torch.float32)
        aux = aux.reshape(1, -1) if aux.ndim == 1 else aux
        aux = aux.contiguous()
    out = torch.empty_like(queries)  # every row is written: sequences by their tiles, the rest zero-filled
    ragged_page_attention_into(
        out, ws, queries, kv_pages, context_lens, block_tables, query_start_loc,
        _num_seqs_tensor(num_seqs, device),
        softmax_scale=float(softmax_scale), logits_soft_cap=logits_soft_cap, sliding_window=sliding_window,
        softmax_aux=aux, num_kv_pages_per_block=num_kv_pages_per_block,
        num_queries_per_block=num_queries_per_block,
    )
    _debug_check_status(ws, "ragged_page_attention")
    return out


def _debug_check_status(ws: RpaWorkspace, what: str) -> None:
    """Opt-in (``EJKERNEL_B200_CHECK_STATUS=1``): read the status word after the call -- this synchronises --
    and raise when it says the outputs are invalid (a wait ran out, or the planner ran out of workspace)."""
    if os.environ.get("EJKERNEL_B200_CHECK_STATUS", "0") not in ("", "0"):
        word = int(ws.status.item())
        if word & (_cabi.ST_TIMEOUT | _cabi.ST_INTERNAL):
            ws.status.zero_()
            raise _cabi.RpaLibraryError(f"{what}: status word {word:#x}: " + "; ".join(_cabi.decode_status(word)))


def read_status(queries: torch.Tensor, kv_pages: torch.Tensor | None = None, block_tables: torch.Tensor | None = None,
                clear: bool = True) -> int:
    """Status word of the operator's workspace for the device of ``queries`` and the current stream (forces a
    device sync).  Debug aid: the reference has no device-side error reporting at all."""
    device = queries.device
    ws = _workspace_cache.get((device.index, torch.cuda.current_stream(device).cuda_stream))
    if ws is None:
        return 0
    word = int(ws.status.item())
    if clear:
        ws.status.zero_()
    return word
