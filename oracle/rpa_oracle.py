"""CPU restatement of the reference's ``ragged_page_attention`` -- TEST INFRASTRUCTURE ONLY.

Nothing in the product path may import this module: it is the checker used by ``tests/``,
by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py``.

PINNED to outputs of the reference's own kernel.  The reference's XLA implementation needs JAX, which is not
installed where this was written and cannot be installed (no network), and its repository holds no golden
vectors or known-answer files for this operator (the only numeric comparisons,
test/kernels/_pallas/tpu/test_ragged_page_attention.py:465-554, are TPU-gated XLA-vs-Pallas checks with freshly
drawn inputs).  Its Triton implementation of the same operator, ``_ragged_paged_attn_fwd``
(ejkernel/kernels/_triton/ragged_page_attention/_triton_impl_fwd.py:27-208), is a plain ``@triton.jit`` function:
tests/golden/make_reference_fixtures.py runs it from the reference checkout (Triton's interpreter on the CPU, and
compiled for a B200) and tests/test_reference_fixtures.py holds ``dense_reference`` and ``blocked_as_written``
against those outputs.  Not covered by that kernel, hence not pinned: attention sinks, and XLA's accumulation
order inside bf16 contractions.  Further anchors: the two restatements below follow two *independent* reference
sources and must agree with each other (tests/test_oracle.py), and a set of analytically known answers (uniform
softmax over encoded values, single visible key, planted keys).

Two modes:

``dense_reference``  -- the intended semantics.  Follows ``ref_ragged_page_attention``
    (ejkernel/kernels/_pallas/tpu/ragged_page_attention/_pallas_impl_fwd.py:62-121):
    per sequence gather the pages, cut to ``kv_len``, ``einsum`` in high precision, scale,
    optional ``cap*tanh(x/cap)``, causal + sliding-window mask, softmax, ``P @ V``.
    Attention sinks follow ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:60-77,161-172
    (extra logits that enter the denominator only).

``blocked_as_written`` -- the XLA implementation as written, loop for loop
    (ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:25-201): sequences ->
    8-row query blocks -> KV blocks of 64 pages, page gather, two contractions, online
    softmax with the carried state rounded to ``compute_dtype``.  Includes the start-index
    clamping of ``lax.dynamic_slice`` / ``dynamic_update_slice`` (so it shows the same
    artefacts as the reference when a block would overrun its array) and the ``-inf - -inf``
    NaN of a fully masked leading KV block under a sliding window.  Used for timing the CPU
    baseline and for demonstrating those artefacts; XLA's internal accumulation precision for
    bf16 contractions is not specified by the reference, so fp32 accumulation then rounding
    to ``compute_dtype`` is assumed.
"""

from __future__ import annotations

import numpy as np
import torch

# ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:22
DEFAULT_MASK_VALUE = -0.7 * float(np.finfo(np.dtype("float32")).max)


def _np(x, dtype=None):
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu()
        if x.dtype in (torch.bfloat16, torch.float16, torch.float8_e4m3fn):
            x = x.float()
        x = x.numpy()
    x = np.asarray(x)
    return x if dtype is None else x.astype(dtype, copy=False)


def _num_seqs(num_seqs) -> int:
    # _xla_impl_fwd.py:195 -- accepts a (1,) array or a scalar
    a = _np(num_seqs)
    return int(a.reshape(-1)[0])


def _sinks_per_q_head(softmax_aux, num_q_heads, num_kv_heads):
    """_xla_impl_fwd.py:60-77: [Hq,n] | [Hkv,n] (broadcast over the group) | [n] (all heads)."""
    if softmax_aux is None:
        return None
    aux = _np(softmax_aux, np.float64)
    G = num_q_heads // num_kv_heads
    if aux.ndim == 2:
        if aux.shape[0] == num_q_heads:
            return aux
        if aux.shape[0] == num_kv_heads:
            return np.repeat(aux, G, axis=0)
        raise ValueError(
            f"softmax_aux first dim must be num_q_heads ({num_q_heads}) or num_kv_heads ({num_kv_heads}), got {aux.shape}"
        )
    if aux.ndim == 1:
        return np.broadcast_to(aux[None, :], (num_q_heads, aux.shape[0]))
    raise ValueError(f"Unsupported softmax_aux shape: {aux.shape}")


def dense_reference(
    queries,
    kv_pages,
    context_lens,
    block_tables,
    query_start_loc,
    num_seqs,
    *,
    softmax_scale: float | None = None,
    sliding_window: int | None = None,
    logits_soft_cap: float | None = None,
    softmax_aux=None,
    precision: str = "fp64",
    seq_subset=None,
    p_dtype=None,
    return_weight_bound: bool = False,
):
    """Intended semantics; returns float64 ``[T, Hq, D]`` (rows past the last sequence are 0).

    ``precision="fp32"`` runs the two contractions in float32 (for the larger cases);
    the softmax statistics stay in float64 either way.

    ``p_dtype`` (a torch dtype) rounds the NORMALISED probabilities to that dtype before ``P @ V``, as the v3
    operator of the reference does with the dtype of the cache
    (ejkernel/kernels/_xla/ragged_page_attention_v3/_kernel.py:281).  ``return_weight_bound=True`` also returns
    ``P @ |V|`` of the unrounded probabilities: a rounding of the weights with relative error <= eps changes
    an output element by at most eps times that.
    """
    ft = np.float64 if precision == "fp64" else np.float32
    q = _np(queries, ft)
    kv = _np(kv_pages)
    ctx = _np(context_lens, np.int64)
    tab = _np(block_tables, np.int64)
    cu = _np(query_start_loc, np.int64)
    S = _num_seqs(num_seqs)
    T, Hq, D = q.shape
    P, page, C2, Dk = kv.shape
    assert C2 % 2 == 0 and Dk == D
    Hkv = C2 // 2
    assert Hq % Hkv == 0
    G = Hq // Hkv
    scale = D**-0.5 if softmax_scale is None else float(softmax_scale)
    sinks = _sinks_per_q_head(softmax_aux, Hq, Hkv)
    out = np.zeros((T, Hq, D), dtype=np.float64)
    wbound = np.zeros((T, Hq, D), dtype=np.float64) if return_weight_bound else None
    seqs = range(S) if seq_subset is None else seq_subset
    for s in seqs:
        q0, q1 = int(cu[s]), int(cu[s + 1])
        q_len = q1 - q0
        if q_len <= 0:
            continue
        kv_len = int(ctx[s])
        n_pages = -(-kv_len // page)
        ids = tab[s, :n_pages]
        # _pallas_impl_fwd.py:104-105: K at 0::2, V at 1::2 of the combined-head axis
        blk = kv[ids].reshape(n_pages * page, C2, D)[:kv_len]
        q_pos = (kv_len - q_len) + np.arange(q_len)[:, None]  # :110
        k_pos = np.arange(kv_len)[None, :]
        masked = q_pos < k_pos  # :112
        if sliding_window is not None:
            masked |= (q_pos - int(sliding_window)) >= k_pos  # :114
        for h in range(Hkv):
            k = blk[:, 2 * h, :].astype(ft, copy=False)
            v = blk[:, 2 * h + 1, :].astype(ft, copy=False)
            qh = q[q0:q1, h * G : (h + 1) * G, :]  # [q_len, G, D]; q head h*G+g <-> kv head h
            logits = np.einsum("qgd,kd->gqk", qh, k, optimize=True).astype(np.float64) * scale
            if logits_soft_cap is not None:
                logits = logits_soft_cap * np.tanh(logits / logits_soft_cap)  # :115-116
            logits = np.where(masked[None], -np.inf, logits)
            m = logits.max(axis=-1, keepdims=True)
            if sinks is not None:
                sk = sinks[h * G : (h + 1) * G]  # [G, n]
                m = np.maximum(m, sk.max(axis=-1)[:, None, None])
            m = np.where(np.isfinite(m), m, 0.0)
            p = np.exp(logits - m)
            den = p.sum(axis=-1, keepdims=True)
            if sinks is not None:
                den = den + np.exp(sk[:, None, :] - m).sum(axis=-1, keepdims=True)
            den = np.maximum(den, 1e-30)
            pn = p / den
            if return_weight_bound:
                wbound[q0:q1, h * G : (h + 1) * G, :] = np.einsum("gqk,kd->qgd", pn.astype(ft), np.abs(v), optimize=True)
            if p_dtype is not None:
                pn = torch.from_numpy(pn).to(p_dtype).to(torch.float64).numpy()
            o = np.einsum("gqk,kd->qgd", pn.astype(ft), v, optimize=True)
            out[q0:q1, h * G : (h + 1) * G, :] = o
    return (out, wbound) if return_weight_bound else out


# ----------------------------------------------------------------------------------------


def _dyn_start(start: int, size: int, dim: int) -> int:
    """lax.dynamic_slice / dynamic_update_slice clamp the start so the window fits."""
    return max(0, min(int(start), dim - size))


def blocked_as_written(
    queries: torch.Tensor,
    kv_pages: torch.Tensor,
    context_lens,
    block_tables,
    query_start_loc,
    num_seqs,
    *,
    softmax_scale: float | None = None,
    sliding_window: int | None = None,
    logits_soft_cap: float | None = None,
    softmax_aux=None,
    compute_dtype=torch.bfloat16,
    seq_subset=None,
) -> torch.Tensor:
    """The XLA implementation as written (_xla_impl_fwd.py:25-201), on torch CPU tensors.

    Every intermediate the reference keeps in ``compute_dtype`` is rounded to it here.
    Returns ``[T, Hq, D]`` in the dtype of ``queries``.
    """
    q_in = queries.detach().cpu()
    kvp = kv_pages.detach().cpu()
    ctx = _np(context_lens, np.int64)
    tab = torch.as_tensor(_np(block_tables, np.int64))
    cu = _np(query_start_loc, np.int64)
    S = _num_seqs(num_seqs)
    T, Hq, D = q_in.shape
    page = kvp.shape[1]
    Hkv = kvp.shape[2] // 2
    G = Hq // Hkv
    pages_per_seq = tab.shape[-1]
    cd = compute_dtype
    rd = lambda x: x.to(cd).float()  # "stored in compute_dtype"
    scale = D**-0.5 if softmax_scale is None else float(softmax_scale)

    qblocks = 8 if T >= 8 else max(1, T)  # :47
    kvblocks = 64 if pages_per_seq >= 64 else max(1, pages_per_seq)  # :48
    # :49 -- the product is formed in the dtype of ``queries``
    q = (q_in.float() * scale).to(q_in.dtype).reshape(T, Hkv, G, D)
    pad = (-T) % qblocks  # :51
    if pad:
        q = torch.cat([q, torch.zeros((pad, Hkv, G, D), dtype=q.dtype)], 0)
    Tp = q.shape[0]
    out = torch.zeros_like(q)
    sinks = None
    if softmax_aux is not None:
        sinks = torch.as_tensor(np.array(_sinks_per_q_head(softmax_aux, Hq, Hkv))).float().reshape(Hkv, G, -1)

    kv_tokens_per_block = page * kvblocks
    base_k = torch.arange(kv_tokens_per_block)
    seqs = range(S) if seq_subset is None else seq_subset
    for s in seqs:
        n_q = int(cu[s + 1] - cu[s])
        if n_q <= 0:  # :189-193
            continue
        kv_len = int(ctx[s])
        for qb in range(-(-n_q // qblocks)):
            q_off = qb * qblocks
            g0 = int(cu[s]) + q_off
            g0c = _dyn_start(g0, qblocks, Tp)  # :88-92 (clamped slice start)
            qblk = q[g0c : g0c + qblocks].to(cd).float()  # [8,Hkv,G,D]
            q_idx = torch.arange(qblocks) + (kv_len - n_q + q_off)  # :95-97 (not clamped)
            n_kvb = -(-kv_len // kv_tokens_per_block)
            o = torch.zeros((qblocks, Hkv, G, D))
            l = torch.zeros((qblocks, Hkv, G))
            m = torch.full((qblocks, Hkv, G), float("-inf"))
            for kb in range(n_kvb):
                p0 = _dyn_start(kb * kvblocks, kvblocks, pages_per_seq)  # :105-109
                ids = tab[s, p0 : p0 + kvblocks]
                blk = kvp[ids]  # [kvblocks, page, 2Hkv, D]
                kblk = blk[:, :, 0::2, :].reshape(kvblocks * page, Hkv, D).to(cd).float()  # :113
                vblk = blk[:, :, 1::2, :].reshape(kvblocks * page, Hkv, D).to(cd).float()  # :114
                k_idx = base_k + kb * kv_tokens_per_block
                sc = rd(torch.einsum("bihd,kid->bihk", qblk, kblk))  # :119-124
                if logits_soft_cap is not None:
                    sc = rd(rd(torch.tanh(rd(sc / logits_soft_cap))) * logits_soft_cap)  # :126
                keep = q_idx[:, None] >= k_idx[None, :]  # :128
                if sliding_window is not None:
                    keep &= k_idx[None, :] > (q_idx - int(sliding_window))[:, None]  # :131-134
                keep &= (k_idx < kv_len)[None, :]  # :135
                keep = keep[:, None, None, :]
                sc = torch.where(keep, sc, torch.tensor(float("-inf")))  # :138
                cur = sc.max(dim=3).values
                new_m = torch.maximum(m, cur)  # :141
                pr = rd(torch.exp(rd(sc - new_m[..., None])))  # :143 (NaN when both are -inf)
                pr = torch.where(keep, pr, torch.tensor(0.0))  # :144
                resc = rd(torch.exp(rd(m - new_m)))  # :146 (NaN when both are -inf)
                l = rd(rd(resc * l) + rd(pr.sum(dim=3)))  # :147
                upd = rd(torch.einsum("bihk,kid->bihd", pr, vblk))  # :148
                o = rd(rd(resc[..., None] * o) + upd)  # :149
                m = new_m
            if sinks is not None:  # :161-172
                sk = sinks[None].expand(qblocks, Hkv, G, sinks.shape[-1])
                m_tot = torch.maximum(m, sk.max(dim=3).values)
                den = torch.exp(m - m_tot) * l + torch.exp(sk - m_tot[..., None]).sum(dim=3)
                den = torch.clamp_min(den, 1e-6)
                norm = (torch.exp(m - m_tot)[..., None] * o) / den[..., None]
            else:  # :173-177
                norm = o / torch.clamp_min(l, 1e-6)[..., None]
            norm = norm.to(q.dtype)
            w0 = _dyn_start(g0, qblocks, Tp)  # :181-185 (clamped update start)
            out[w0 : w0 + qblocks] = norm
    return out[:T].reshape(T, Hq, D)


def v3_reference(
    queries,
    keys,
    values,
    kv_cache,
    kv_lens,
    block_tables,
    query_start_loc,
    distribution,
    *,
    softmax_scale: float = 1.0,
    sliding_window: int | None = None,
    logits_soft_cap: float | None = None,
    q_scale: float | None = None,
    k_scale: float | None = None,
    v_scale: float | None = None,
    precision: str = "fp64",
    round_p: bool = False,
    return_weight_bound: bool = False,
):
    """The v3 operator (ejkernel/kernels/_xla/ragged_page_attention_v3/_kernel.py:143-318): scatter the
    new key/value rows into the paged cache, then attend against the updated cache.

    ``kv_cache`` is ``[P, page, 2*Hkv/pack, pack, D]``; ``merge_kv`` (:45-57) interleaves K_h / V_h at
    combined heads 2h / 2h+1.  Row r of sequence s lands at position ``kv_len - q_len + r`` (:227-229).
    ``block_tables`` is flat, ``distribution[-1]`` the number of sequences (:211).  Returns
    ``(out float64 [T,Hq,D], updated cache as a torch tensor of the cache dtype)``; attention is
    ``dense_reference`` on the updated cache with scale ``softmax_scale * k_scale`` and the output
    times ``v_scale`` (:262-263, :290-291).

    Quantised path (:249-291; keys, values and cache may be ``torch.float8_e4m3fn``): with ``q_scale`` the
    queries are divided by it in their own dtype, clipped to the finite range of the cache dtype and cast to it,
    and the logits are multiplied by ``q_scale`` again; ``round_p=True`` casts the normalised probabilities to the
    cache dtype before ``P @ V`` as the reference does (:281) -- with an e4m3 cache that flushes every
    probability below 2^-10 to zero, so it is off by default and the tests use it on short contexts only.
    """
    cache = kv_cache.detach().cpu().clone()
    P, page, hx2p, pack, D = cache.shape
    C2 = hx2p * pack
    # an 8-bit cache is written as bytes (indexed assignment is not defined for float8 tensors)
    as_bytes = (lambda t: t.view(torch.uint8)) if cache.element_size() == 1 else (lambda t: t)
    flat = as_bytes(cache).view(P, page, C2, D)
    ctx = _np(kv_lens, np.int64)
    S_max = ctx.shape[0]
    tab = _np(block_tables, np.int64).reshape(S_max, -1)
    cu = _np(query_start_loc, np.int64)
    S = int(_np(distribution).reshape(-1)[-1])
    k = as_bytes(keys.detach().cpu())
    v = as_bytes(values.detach().cpu())
    Hkv = k.shape[1]
    fused = torch.stack([k, v], dim=2).reshape(k.shape[0], 2 * Hkv, k.shape[2])  # merge_kv
    for s in range(S):
        q0, q1 = int(cu[s]), int(cu[s + 1])
        kl = int(ctx[s])
        for r in range(q1 - q0):
            pos = kl - (q1 - q0) + r
            flat[int(tab[s, pos // page]), pos % page, : 2 * Hkv, : k.shape[2]] = fused[q0 + r]
            # merge_kv pads the row with zeros, lanes beyond head_dim and combined heads beyond 2*Hkv alike (:45-57)
            flat[int(tab[s, pos // page]), pos % page, : 2 * Hkv, k.shape[2] :] = 0
            flat[int(tab[s, pos // page]), pos % page, 2 * Hkv :, :] = 0
    scale = float(softmax_scale) * (1.0 if k_scale is None else float(k_scale))
    q_in = queries
    if q_scale is not None:
        qt = queries.detach().cpu()
        lim = float(torch.finfo(cache.dtype).max)
        q_in = (qt / float(q_scale)).clamp(-lim, lim).to(cache.dtype)  # :249-254 (the division rounds to q's dtype first)
        scale *= float(q_scale)  # :264-265
    # the cache's last dim is align_to(D, 128) and its combined-head axis align_to(2*Hkv, pack); attention reads the
    # first D lanes of the first 2*Hkv heads (:240-241)
    res = dense_reference(q_in, flat.view(cache.dtype)[:, :, : 2 * Hkv, : k.shape[2]], ctx, tab, cu, np.array([S]), softmax_scale=scale,
                          sliding_window=sliding_window, logits_soft_cap=logits_soft_cap, precision=precision,
                          p_dtype=cache.dtype if round_p else None, return_weight_bound=return_weight_bound)
    out, wb = res if return_weight_bound else (res, None)
    if v_scale is not None:
        out = out * float(v_scale)
        wb = None if wb is None else wb * float(v_scale)
    return (out, cache, wb) if return_weight_bound else (out, cache)


def page_attention_reference(query, key_cache, value_cache, context_lens, block_tables, *, attn_scale=None,
                             attn_logits_soft_cap=None) -> np.ndarray:
    """Decode attention over separate paged caches, float64
    (ejkernel/kernels/_xla/page_attention/_xla_impl_fwd.py:22-97): ``query [S,Hq,D]``, caches
    ``[num_blocks, Hkv, block_size, D]``, token j of sequence s in block ``block_tables[s, j // block_size]``,
    keys ``j < context_lens[s]`` visible, logits ``(q.k) * attn_scale`` (default ``D**-0.5``), optional soft
    cap (Triton version of the operator), softmax, weighted sum of V.  Sequences with no visible key give 0.
    """
    q = _np(query, np.float64)
    kc = _np(key_cache, np.float64)
    vc = _np(value_cache, np.float64)
    ctx = _np(context_lens, np.int64)
    tab = _np(block_tables, np.int64)
    S, Hq, D = q.shape
    _, Hkv, bs, _ = kc.shape
    G = Hq // Hkv
    scale = D**-0.5 if attn_scale is None else float(attn_scale)
    out = np.zeros_like(q)
    for s in range(S):
        n = int(ctx[s])
        if n <= 0:
            continue
        nb = -(-n // bs)
        k = kc[tab[s, :nb]].transpose(1, 0, 2, 3).reshape(Hkv, nb * bs, D)[:, :n]
        v = vc[tab[s, :nb]].transpose(1, 0, 2, 3).reshape(Hkv, nb * bs, D)[:, :n]
        for h in range(Hkv):
            logits = (q[s, h * G : (h + 1) * G] @ k[h].T) * scale
            if attn_logits_soft_cap is not None:
                logits = attn_logits_soft_cap * np.tanh(logits / attn_logits_soft_cap)
            logits -= logits.max(axis=-1, keepdims=True)
            p = np.exp(logits)
            out[s, h * G : (h + 1) * G] = (p / p.sum(axis=-1, keepdims=True)) @ v[h]
    return out


def compare(got, want, *, atol=2e-2, rtol=2e-2, rows: int | None = None, rms_tol=3e-2, rel_tol=1e-2) -> dict:
    """Error summary of ``got`` against ``want`` on rows ``[0, rows)``.

    ``allclose`` is the stated criterion ``|got-want| <= atol + rtol*|want|``.  On N(0,1) inputs with
    long contexts the outputs themselves are smaller than ``atol`` (an all-zero result would pass),
    so ``tight`` additionally demands ``|got-want| <= rms_tol*rms(want) + rel_tol*|want|``: an
    absolute floor that scales with the size of the expected output plus 1 % relative error, which is
    what bf16 rounding of the probabilities and of the output allows.
    """
    g = _np(got, np.float64)
    w = _np(want, np.float64)
    if rows is not None:
        g, w = g[:rows], w[:rows]
    err = np.abs(g - w)
    rms = float(np.sqrt(np.mean(w * w))) if w.size else 0.0
    return dict(
        max_abs=float(err.max()) if err.size else 0.0,
        tight=bool(np.all(err <= rms_tol * rms + rel_tol * np.abs(w))),
        rms_want=rms,
        max_rel_rms=float(err.max() / max(rms, 1e-30)) if err.size else 0.0,
        allclose=bool(np.all(err <= atol + rtol * np.abs(w))),
        finite=bool(np.all(np.isfinite(g))),
    )
