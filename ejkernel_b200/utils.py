"""Seeded synthetic inputs for ``ragged_page_attention``.

The reference builds its inputs with ``make_dummy_ragged_paged_attention_inputs``
(test/test_ragged_page_attn.py:27-115) and ``benchmarks/benchmark_ragged_page_attn.py:40-129``:
a paged KV pool ``[num_pages, page_size, 2*num_kv_heads, head_dim]`` with K_h at combined
index ``2h`` and V_h at ``2h+1``, a per-sequence page table, int32 lengths and a
cumulative query offset array.  This module produces inputs of the same layout for the
five benchmark workloads ("C1".."C5") and for arbitrary ragged batches.

Index arrays always come from ``numpy.random.Generator(PCG64(seed))`` so they are
identical on every machine.  The float payload (q, k, v ~ N(0,1), rounded to the
storage dtype) comes from a seeded torch generator on the device that will hold it,
because the full-size pools (4.8 - 21.5 GB) are impractical to draw on the host.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class RaggedBatch:
    """One call's worth of operands, named as the reference names them
    (ejkernel/kernels/_xla/ragged_page_attention/_interface.py:27-47)."""

    queries: torch.Tensor  # [T_buf, Hq, D]
    kv_pages: torch.Tensor  # [P, page, 2*Hkv, D]
    context_lens: torch.Tensor  # [S_max] int32
    block_tables: torch.Tensor  # [S_max, pages_per_seq] int32
    query_start_loc: torch.Tensor  # [S_max+1] int32
    num_seqs: torch.Tensor  # [1] int32
    softmax_scale: float
    sliding_window: int | None = None
    logits_soft_cap: float | None = None
    softmax_aux: torch.Tensor | None = None
    meta: dict = field(default_factory=dict)

    def to(self, device) -> "RaggedBatch":
        mv = lambda t: None if t is None else t.to(device, non_blocking=False)
        return RaggedBatch(
            mv(self.queries),
            mv(self.kv_pages),
            mv(self.context_lens),
            mv(self.block_tables),
            mv(self.query_start_loc),
            mv(self.num_seqs),
            self.softmax_scale,
            self.sliding_window,
            self.logits_soft_cap,
            mv(self.softmax_aux),
            dict(self.meta),
        )

    @property
    def total_tokens(self) -> int:
        return int(self.meta["total_tokens"])

    def kwargs(self) -> dict:
        """Keyword arguments of the operator call."""
        return dict(
            softmax_scale=self.softmax_scale,
            sliding_window=self.sliding_window,
            logits_soft_cap=self.logits_soft_cap,
            softmax_aux=self.softmax_aux,
        )

    def args(self) -> tuple:
        return (
            self.queries,
            self.kv_pages,
            self.context_lens,
            self.block_tables,
            self.query_start_loc,
            self.num_seqs,
        )


def visible_kv_tokens(q_lens, kv_lens, sliding_window=None) -> int:
    """Number of distinct KV tokens a call has to read: per sequence the union of the
    keys visible to any of its query rows (row r sits at position kv_len-q_len+r and
    sees keys (pos-W, pos])."""
    total = 0
    for ql, kl in zip(q_lens, kv_lens):
        ql, kl = int(ql), int(kl)
        if ql == 0:
            continue
        lo = 0
        if sliding_window is not None:
            lo = max(0, (kl - ql) - int(sliding_window) + 1)
        total += kl - lo
    return total


def algorithmic_kv_bytes(batch: RaggedBatch) -> int:
    """KV bytes a perfect kernel must move: visible tokens * 2 (K,V) * Hkv * D * itemsize."""
    m = batch.meta
    vis = visible_kv_tokens(m["q_lens"], m["kv_lens"], batch.sliding_window)
    return vis * 2 * m["num_kv_heads"] * m["head_dim"] * batch.kv_pages.element_size()


def make_ragged_batch(
    q_lens,
    kv_lens,
    *,
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    page_size: int,
    pages_per_seq: int | None = None,
    num_pages: int | None = None,
    max_num_seqs: int | None = None,
    pad_query_rows: int = 0,
    dtype=torch.bfloat16,
    device="cpu",
    seed: int = 0,
    softmax_scale: float | None = None,
    sliding_window: int | None = None,
    logits_soft_cap: float | None = None,
    kv_head_slice: tuple[int, int] | None = None,
    page_order: str = "permuted",
    kv_dtype=None,
) -> RaggedBatch:
    """Build one ragged batch.

    ``block_tables[s, :n_s]`` are consecutive slices of one global random permutation of
    the pool's pages (``page_order="permuted"``) or consecutive page ids (``"linear"``,
    as in the reference's own test builders); unused table entries are 0.  ``kv_dtype`` gives the pool another
    dtype than the queries (``torch.float8_e4m3fn``: the same N(0,1) draws rounded to e4m3).

    ``kv_head_slice=(h0, h1)`` materialises only KV heads ``[h0, h1)`` (and the query heads
    of their groups) while drawing the same index arrays, which is how one rank of a
    KV-head-sharded run builds its shard without ever holding the full pool.
    """
    q_lens = np.asarray(q_lens, dtype=np.int64)
    kv_lens = np.asarray(kv_lens, dtype=np.int64)
    assert q_lens.shape == kv_lens.shape and q_lens.ndim == 1
    assert np.all(q_lens <= kv_lens), "a sequence cannot have more query rows than KV tokens"
    assert num_q_heads % num_kv_heads == 0
    S = len(q_lens)
    S_max = max_num_seqs if max_num_seqs is not None else S
    assert S <= S_max
    n_pages_seq = [cdiv(int(k), page_size) for k in kv_lens]
    if pages_per_seq is None:
        pages_per_seq = max(1, max(n_pages_seq, default=1))
    assert max(n_pages_seq, default=0) <= pages_per_seq
    used = int(sum(n_pages_seq))
    if num_pages is None:
        num_pages = max(1, math.ceil(used * 1.1))
    assert used <= num_pages

    rng = np.random.Generator(np.random.PCG64(seed))
    if page_order == "permuted":
        perm = rng.permutation(num_pages).astype(np.int32)
    else:
        perm = np.arange(num_pages, dtype=np.int32)
    tables = np.zeros((S_max, pages_per_seq), dtype=np.int32)
    off = 0
    for s in range(S):
        n = n_pages_seq[s]
        tables[s, :n] = perm[off : off + n]
        off += n
    ctx = np.zeros((S_max,), dtype=np.int32)
    ctx[:S] = kv_lens
    cu = np.zeros((S_max + 1,), dtype=np.int32)
    cu[1 : S + 1] = np.cumsum(q_lens)
    cu[S + 1 :] = cu[S]
    T = int(cu[S])
    T_buf = T + pad_query_rows

    G = num_q_heads // num_kv_heads
    h0, h1 = (0, num_kv_heads) if kv_head_slice is None else kv_head_slice
    Hkv_loc = h1 - h0
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + 7919 * (h0 + 1))
    scale = softmax_scale if softmax_scale is not None else head_dim**-0.5
    q = torch.randn((max(T_buf, 1), Hkv_loc * G, head_dim), generator=gen, device=device, dtype=torch.float32).to(dtype)
    q = q[:T_buf] if T_buf > 0 else q[:0]
    # Draw the pool page-block by page-block so the fp32 staging buffer stays small.
    kv = torch.empty((num_pages, page_size, 2 * Hkv_loc, head_dim), device=device, dtype=kv_dtype or dtype)
    page_elems = page_size * 2 * Hkv_loc * head_dim
    step = max(1, (1 << 27) // page_elems)
    for p0 in range(0, num_pages, step):
        p1 = min(num_pages, p0 + step)
        blk = torch.randn((p1 - p0, page_size, 2 * Hkv_loc, head_dim), generator=gen, device=device, dtype=torch.float32)
        kv[p0:p1] = blk.to(kv_dtype or dtype)
        del blk

    meta = dict(
        total_tokens=T,
        q_lens=q_lens.tolist(),
        kv_lens=kv_lens.tolist(),
        num_q_heads=Hkv_loc * G,
        num_kv_heads=Hkv_loc,
        head_dim=head_dim,
        page_size=page_size,
        pages_per_seq=pages_per_seq,
        num_pages=num_pages,
        kv_head_slice=(h0, h1),
        seed=seed,
    )
    return RaggedBatch(
        queries=q,
        kv_pages=kv,
        context_lens=torch.from_numpy(ctx).to(device),
        block_tables=torch.from_numpy(tables).to(device),
        query_start_loc=torch.from_numpy(cu).to(device),
        num_seqs=torch.tensor([S], dtype=torch.int32, device=device),
        softmax_scale=float(scale),
        sliding_window=sliding_window,
        logits_soft_cap=logits_soft_cap,
        meta=meta,
    )


# ----------------------------------------------------------------------------------------
# The five benchmark workloads.  ``scale`` < 1 shrinks the number of sequences (and, for the
# long-context ones, the lengths) so the CPU checker finishes in seconds; 1.0 is full size.
# ----------------------------------------------------------------------------------------

WORKLOADS = ("c1", "c2", "c3", "c4", "c5")


def workload_lengths(name: str, *, num_seqs: int | None = None, len_scale: float = 1.0, seed: int | None = None):
    """Return (q_lens, kv_lens, shape kwargs) for a named workload, seeded 1000+id."""
    name = name.lower()
    idx = WORKLOADS.index(name) + 1
    rng = np.random.Generator(np.random.PCG64(1000 + idx if seed is None else seed))
    sc = lambda x: max(1, int(round(x * len_scale)))
    if name == "c1":
        S = num_seqs or 8
        kv = rng.integers(16, 512, size=S, endpoint=True)
        q = np.ones(S, dtype=np.int64)
        shape = dict(num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, pages_per_seq=32, num_pages=256)
        extra = {}
    elif name == "c2":
        S = num_seqs or 256
        kv = rng.integers(sc(128), sc(8192), size=S, endpoint=True)
        q = np.ones(S, dtype=np.int64)
        shape = dict(num_q_heads=32, num_kv_heads=8, head_dim=128, page_size=16, pages_per_seq=cdiv(sc(8192), 16))
        extra = {}
    elif name == "c3":
        n_dec = 64 if num_seqs is None else max(1, num_seqs - 4)
        n_pre = 4 if num_seqs is None else min(4, max(0, num_seqs - n_dec))
        q_pre = sc(512)
        kv_dec = rng.integers(sc(512), sc(16384), size=n_dec, endpoint=True)
        prior = rng.integers(0, sc(8192), size=n_pre, endpoint=True)
        kv = np.concatenate([kv_dec, prior + q_pre])
        q = np.concatenate([np.ones(n_dec, dtype=np.int64), np.full(n_pre, q_pre, dtype=np.int64)])
        shape = dict(num_q_heads=32, num_kv_heads=8, head_dim=128, page_size=16, pages_per_seq=cdiv(sc(16384), 16))
        extra = {}
    elif name == "c4":
        S = num_seqs or 128
        kv = rng.integers(sc(2048), sc(32768), size=S, endpoint=True)
        q = np.ones(S, dtype=np.int64)
        shape = dict(num_q_heads=16, num_kv_heads=8, head_dim=256, page_size=32, pages_per_seq=cdiv(sc(32768), 32))
        extra = dict(sliding_window=sc(4096), logits_soft_cap=50.0)
    elif name == "c5":
        S = num_seqs or 64
        kv = rng.integers(sc(32768), sc(131072), size=S, endpoint=True)
        q = np.ones(S, dtype=np.int64)
        shape = dict(num_q_heads=64, num_kv_heads=8, head_dim=128, page_size=32, pages_per_seq=cdiv(sc(131072), 32))
        extra = {}
    else:
        raise ValueError(name)
    return q, kv, shape, extra


def make_workload(
    name: str,
    *,
    device="cpu",
    num_seqs: int | None = None,
    len_scale: float = 1.0,
    dtype=torch.bfloat16,
    kv_head_slice: tuple[int, int] | None = None,
    pad_query_rows: int = 0,
    seed: int | None = None,
    kv_dtype=None,
) -> RaggedBatch:
    q, kv, shape, extra = workload_lengths(name, num_seqs=num_seqs, len_scale=len_scale, seed=seed)
    idx = WORKLOADS.index(name.lower()) + 1
    b = make_ragged_batch(
        q,
        kv,
        dtype=dtype,
        device=device,
        seed=(1000 + idx) if seed is None else seed,
        kv_head_slice=kv_head_slice,
        pad_query_rows=pad_query_rows,
        kv_dtype=kv_dtype,
        **shape,
        **extra,
    )
    b.meta["workload"] = name.lower()
    return b


def to_v3_inputs(batch: RaggedBatch, fill: float = float("nan"), pad_fill: float = 3.0):
    """Recast a ``ragged_page_attention`` batch as inputs of ``ragged_page_attention_v3``.

    The new key/value rows of the step are the last ``q_len`` tokens of every sequence, taken out of
    the batch's (complete) pool; in the returned cache those positions hold ``fill`` so that the
    operator's page write is observable.  Returns ``(keys, values, kv_cache_5d, block_tables_flat,
    distribution)``; after a correct v3 call the cache equals ``batch.kv_pages`` bit for bit.  When
    ``head_dim`` is not a multiple of 128 the cache's last dim is padded to one, as the reference pads it,
    and so is the combined-head axis when ``2 * num_kv_heads`` is not a multiple of the packing (an e4m3 cache with
    an odd number of kv heads); the padding starts as ``pad_fill`` (the operator must step over it when it reads
    and zero it in the rows it writes).
    Layout as in the reference's ``merge_kv`` / cache (ragged_page_attention_v3/_kernel.py:45-57).
    """
    m = batch.meta
    page, Hkv, D = m["page_size"], m["num_kv_heads"], m["head_dim"]
    pool_t = batch.kv_pages
    # an 8-bit pool is handled as bytes (indexed assignment is not defined for float8); NaN of e4m3 is 0x7f
    eight = pool_t.element_size() == 1
    pool = pool_t.view(torch.uint8) if eight else pool_t
    if eight:
        fill, pad_fill = 0x7F, 0x44
    dev = pool.device
    T = batch.queries.shape[0]
    keys = torch.zeros((T, Hkv, D), dtype=pool.dtype, device=dev)
    values = torch.zeros_like(keys)
    cache = pool.clone()
    cu = batch.query_start_loc.tolist()
    tab = batch.block_tables
    for s, (ql, kl) in enumerate(zip(m["q_lens"], m["kv_lens"])):
        if ql == 0:
            continue
        pos = torch.arange(kl - ql, kl, device=dev)
        pages = tab[s, (pos // page).long()].long()
        slots = (pos % page).long()
        rows = pool[pages, slots]  # [ql, 2Hkv, D]
        keys[cu[s] : cu[s] + ql] = rows[:, 0::2]
        values[cu[s] : cu[s] + ql] = rows[:, 1::2]
        cache[pages, slots] = fill
    pack = 32 // (pool.element_size() * 8)
    d_align = -(-D // 128) * 128
    if d_align != D:
        padded = torch.full((*cache.shape[:-1], d_align), pad_fill, dtype=cache.dtype, device=dev)
        padded[..., :D] = cache
        cache = padded
    c2 = -(-2 * Hkv // pack) * pack  # the combined heads are padded to a multiple of the packing as well (merge_kv)
    if c2 != 2 * Hkv:
        padded = torch.full((pool.shape[0], page, c2, d_align), pad_fill, dtype=cache.dtype, device=dev)
        padded[:, :, : 2 * Hkv] = cache
        cache = padded
    cache5 = cache.view(pool.shape[0], page, c2 // pack, pack, d_align)
    if eight:
        keys, values, cache5 = (t.view(pool_t.dtype) for t in (keys, values, cache5))
    S = len(m["q_lens"])
    distribution = torch.tensor([S, S, S], dtype=torch.int32, device=dev)
    return keys, values, cache5, batch.block_tables.reshape(-1).contiguous(), distribution
