"""The float8 (e4m3) KV cache: ``ragged_page_attention`` on an e4m3 pool and ``ragged_page_attention_v3`` with an
e4m3 cache, ``q_scale`` / ``k_scale`` / ``v_scale`` (ejkernel/kernels/_xla/ragged_page_attention_v3/_kernel.py:45-57,
157-159,249-291).

Tolerance.  Keys and values are e4m3 on both sides, so they add no error.  The kernel feeds the probabilities to the
P.V tensor-core instruction as e4m3 (the reference casts them to the cache dtype as well, :281): each weight is off
by at most half an e4m3 ulp, 2^-4 relative, so an output element is off by at most ``2^-4 * (P @ |V|)``.  The oracle
returns that bound per element (``return_weight_bound``); on top of it the tests allow the bf16 rounding of the
output (2^-8 relative) and 1e-3.  The reference rounds the NORMALISED probabilities, the kernel's online softmax the
unnormalised ones, so the two roundings differ element by element; against the oracle with the reference's rounding
(``round_p=True``) twice the bound holds, on contexts short enough that the normalised probabilities stay e4m3 normals."""

import numpy as np
import pytest
import torch

from ejkernel_b200.utils import make_ragged_batch, make_workload, to_v3_inputs
from oracle.rpa_oracle import dense_reference, v3_reference

FP8 = torch.float8_e4m3fn
EPS = 2.0**-4


def _cases():
    mk = lambda ql, kl, **kw: make_ragged_batch(ql, kl, kv_dtype=FP8, **kw)
    yield "decode", mk([1, 1, 1, 1], [300, 17, 64, 2500], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=71)
    yield "mixed", mk([1, 40, 3, 130], [500, 40, 77, 900], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16,
                      seed=72, sliding_window=256, logits_soft_cap=30.0)
    yield "gqa16_wide_tiles", mk([1, 2, 1], [700, 130, 33], num_q_heads=32, num_kv_heads=2, head_dim=128, page_size=32, seed=73)
    yield "d256", mk([2, 70, 1], [100, 300, 1000], num_q_heads=4, num_kv_heads=2, head_dim=256, page_size=32, seed=74)
    yield "page8", mk([1, 9], [333, 100], num_q_heads=8, num_kv_heads=4, head_dim=128, page_size=8, seed=75)
    yield "page24", mk([1, 30, 1], [500, 130, 24], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=24, seed=83)
    yield "page128", mk([1, 5, 1], [1000, 129, 128], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=128, seed=76)
    yield "f16_queries", mk([1, 7], [260, 64], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=77,
                            dtype=torch.float16)
    yield "empty_seq", mk([1, 0, 5], [50, 20, 5], num_q_heads=4, num_kv_heads=4, head_dim=128, page_size=8, max_num_seqs=5,
                          pad_query_rows=3, seed=78)


CASES = list(_cases())
IDS = [n for n, _ in CASES]


def _within(got, want, bound, rows, factor=1.0):
    g = got[:rows].float().cpu().numpy().astype(np.float64)
    err = np.abs(g - want[:rows])
    lim = factor * EPS * 1.02 * bound[:rows] + 2.0**-8 * np.abs(want[:rows]) + 1e-3
    assert np.isfinite(g).all()
    assert (err <= lim).all(), (float((err / lim).max()), float(err.max()))
    # the errors of the weights are not aligned: the typical element is far inside the bound
    assert np.sqrt(np.mean(err**2)) <= 0.5 * EPS * np.sqrt(np.mean(bound[:rows] ** 2)) + 1e-3


@pytest.mark.parametrize("name,b", CASES, ids=IDS)
def test_oracle_v3_with_an_e4m3_cache(name, b):
    keys, values, cache, tab, dist = to_v3_inputs(b)
    assert cache.dtype == FP8 and cache.shape[3] == 4  # four combined heads per 32-bit word (:38-39)
    out, new_cache, wb = v3_reference(b.queries, keys, values, cache, b.context_lens, tab, b.query_start_loc, dist,
                                      softmax_scale=b.softmax_scale, sliding_window=b.sliding_window,
                                      logits_soft_cap=b.logits_soft_cap, return_weight_bound=True)
    assert torch.equal(new_cache.view(torch.uint8).reshape(b.kv_pages.shape), b.kv_pages.view(torch.uint8))
    np.testing.assert_allclose(out, dense_reference(*b.args(), **b.kwargs()), atol=1e-12)
    # the reference's own rounding of the normalised probabilities stays within the weight bound while they are normals
    if max(b.meta["kv_lens"]) <= 64:
        out_r, _ = v3_reference(b.queries, keys, values, cache, b.context_lens, tab, b.query_start_loc, dist,
                                softmax_scale=b.softmax_scale, round_p=True)
        assert (np.abs(out_r - out) <= EPS * 1.02 * wb + 1e-9).all()


def test_oracle_q_scale_rounds_the_queries_to_the_cache_dtype():
    b = CASES[0][1]
    keys, values, cache, tab, dist = to_v3_inputs(b)
    a, _ = v3_reference(b.queries, keys, values, cache, b.context_lens, tab, b.query_start_loc, dist, softmax_scale=0.1,
                        q_scale=0.03, k_scale=1.5, v_scale=2.0)
    q8 = (b.queries / 0.03).clamp(-448, 448).to(FP8).float()
    want = 2.0 * dense_reference(q8, *b.args()[1:], softmax_scale=0.1 * 1.5 * 0.03)
    np.testing.assert_allclose(a, want, atol=1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("name,b", CASES, ids=IDS)
def test_cuda_operator_on_an_e4m3_pool(rpa_lib, name, b):
    from tests.helpers import run_cuda, status_word

    bc = b.to("cuda")
    out = run_cuda(bc)
    assert status_word(bc) == 0
    want, wb = dense_reference(*b.args(), **b.kwargs(), return_weight_bound=True)
    _within(out, want, wb, b.total_tokens)
    assert torch.count_nonzero(out[b.total_tokens:]) == 0
    assert torch.equal(out, run_cuda(bc)), "two runs agree bit for bit"


@pytest.mark.gpu
@pytest.mark.parametrize("q_scale", [None, 0.04])
@pytest.mark.parametrize("name,b", CASES[:5], ids=IDS[:5])
def test_cuda_v3_with_an_e4m3_cache(rpa_lib, name, b, q_scale):
    import ejkernel_b200 as ej

    bc = b.to("cuda")
    keys, values, cache, tab, dist = to_v3_inputs(bc)
    kw = dict(softmax_scale=b.softmax_scale, sliding_window=b.sliding_window, logits_soft_cap=b.logits_soft_cap,
              q_scale=q_scale, k_scale=1.25, v_scale=0.5)
    out, new_cache = ej.ragged_page_attention_v3(bc.queries, keys, values, cache, bc.context_lens, tab, bc.query_start_loc,
                                                 dist, **kw)
    torch.cuda.synchronize()
    assert new_cache.data_ptr() == cache.data_ptr()
    assert torch.equal(new_cache.view(torch.uint8).reshape(b.kv_pages.shape), bc.kv_pages.view(torch.uint8)), "page write"
    ck, cv, cc, ctab, cdist = to_v3_inputs(b)
    want, _, wb = v3_reference(b.queries, ck, cv, cc, b.context_lens, ctab, b.query_start_loc, cdist, **kw,
                               return_weight_bound=True)
    _within(out, want, wb, b.total_tokens)


@pytest.mark.gpu
def test_cuda_against_the_reference_rounding_on_short_contexts(rpa_lib):
    import ejkernel_b200 as ej

    b = make_ragged_batch([1, 20, 1, 64], [40, 20, 64, 64], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16,
                          seed=79, kv_dtype=FP8)
    bc = b.to("cuda")
    keys, values, cache, tab, dist = to_v3_inputs(bc)
    out, _ = ej.ragged_page_attention_v3(bc.queries, keys, values, cache, bc.context_lens, tab, bc.query_start_loc, dist,
                                         softmax_scale=b.softmax_scale, q_scale=0.05)
    torch.cuda.synchronize()
    ck, cv, cc, ctab, cdist = to_v3_inputs(b)
    want, _, wb = v3_reference(b.queries, ck, cv, cc, b.context_lens, ctab, b.query_start_loc, cdist,
                               softmax_scale=b.softmax_scale, q_scale=0.05, round_p=True, return_weight_bound=True)
    g = out.float().cpu().numpy().astype(np.float64)
    assert (np.abs(g - want) <= 2 * EPS * 1.02 * wb + 2.0**-8 * np.abs(want) + 1e-3).all()


@pytest.mark.gpu
def test_e4m3_page_gather_is_bit_exact(rpa_lib):
    """q = 0 makes every weight exp2(0 - m) with m = -4: exactly 16 in e4m3; V carries integers 0..15 that encode
    (page, slot, head, lane).  The float32 mean of such integers over a power-of-two number of keys is exact, so any
    wrong byte, page or slot shows up as an unequal bit pattern."""
    from tests.helpers import run_cuda

    b = make_ragged_batch([1, 1, 4], [256, 64, 128], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=80,
                          kv_dtype=FP8)
    P, page, C2, D = b.kv_pages.shape
    code = (torch.arange(P)[:, None, None, None] * 7 + torch.arange(page)[None, :, None, None] * 3
            + torch.arange(C2)[None, None, :, None] * 5 + torch.arange(D)[None, None, None, :]) % 16
    b.kv_pages = code.float().to(FP8)
    b.queries.zero_()
    out = run_cuda(b.to("cuda")).float().cpu()
    want = torch.from_numpy(dense_reference(*b.args(), **b.kwargs())).to(torch.bfloat16).float()
    assert torch.equal(out[: b.total_tokens], want[: b.total_tokens])


@pytest.mark.gpu
def test_q_scale_with_a_16_bit_cache(rpa_lib):
    import ejkernel_b200 as ej

    b = make_ragged_batch([1, 40, 3], [500, 40, 77], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=81)
    bc = b.to("cuda")
    keys, values, cache, tab, dist = to_v3_inputs(bc)
    kw = dict(softmax_scale=b.softmax_scale, q_scale=3.0, k_scale=0.5, v_scale=2.0)
    out, _ = ej.ragged_page_attention_v3(bc.queries, keys, values, cache, bc.context_lens, tab, bc.query_start_loc, dist, **kw)
    torch.cuda.synchronize()
    ck, cv, cc, ctab, cdist = to_v3_inputs(b)
    want, _ = v3_reference(b.queries, ck, cv, cc, b.context_lens, ctab, b.query_start_loc, cdist, **kw)
    from tests.helpers import assert_parity
    assert_parity(out, want, b.total_tokens, what="q_scale, bf16 cache")


@pytest.mark.gpu
def test_e4m3_decode_batch_at_benchmark_shape(rpa_lib):
    """A slice of the Llama-3-8B-shaped decode batch on an e4m3 pool: sampled sequences against the oracle."""
    from tests.helpers import run_cuda, status_word

    b = make_workload("c2", num_seqs=48, device="cuda", kv_dtype=FP8)
    out = run_cuda(b)
    assert status_word(b) == 0
    bc = b.to("cpu")
    ids = [0, 7, 23, 47]
    want, wb = dense_reference(*bc.args(), **bc.kwargs(), seq_subset=ids, return_weight_bound=True, precision="fp32")
    rows = torch.tensor(ids)
    _within(out[rows], want[ids], wb[ids], len(ids))


@pytest.mark.gpu
def test_e4m3_pool_with_attention_sinks_and_refusals(rpa_lib):
    """Sinks enter the denominator in the shared epilogues, whatever the cache dtype; shapes the e4m3 kernels do not
    serve are refused by the host layer with a clear error (and by the C ABI with a negative code), never served wrongly."""
    import ctypes

    from ejkernel_b200 import _cabi
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import RpaWorkspace, _shape_of
    from tests.helpers import run_cuda, status_word

    b = make_ragged_batch([1, 6, 1], [400, 90, 33], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=82,
                          kv_dtype=FP8)
    b.softmax_aux = torch.tensor([[0.5, -1.0], [2.0, 0.0]])
    bc = b.to("cuda")
    out = run_cuda(bc)
    assert status_word(bc) == 0
    want, wb = dense_reference(*b.args(), **b.kwargs(), return_weight_bound=True)
    _within(out, want, wb, b.total_tokens)

    bad = make_ragged_batch([1], [40], num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=16, seed=1, kv_dtype=FP8).to("cuda")
    with pytest.raises(NotImplementedError):
        ragged_page_attention(*bad.args(), softmax_scale=0.1)  # head_dim 64
    odd = make_ragged_batch([1], [40], num_q_heads=4, num_kv_heads=2, head_dim=128, page_size=12, seed=1, kv_dtype=FP8).to("cuda")
    with pytest.raises(NotImplementedError):
        ragged_page_attention(*odd.args(), softmax_scale=0.1)  # page size not a multiple of 8
    # the same through the raw C ABI: negative codes, nothing launched
    shape = _shape_of(bc.queries, bc.kv_pages, bc.block_tables)
    ws = RpaWorkspace(shape, bc.queries.device)
    o = torch.full_like(bc.queries, 7.0)
    attrs = _cabi.Attrs(0.1, 0.0, 0, 0, 0, 0, 0)
    args = lambda sh: (bc.queries.data_ptr(), bc.kv_pages.data_ptr(), bc.context_lens.data_ptr(), bc.block_tables.data_ptr(),
                       bc.query_start_loc.data_ptr(), bc.num_seqs.data_ptr(), None, o.data_ptr(), ws.buffer.data_ptr(),
                       ws.nbytes, ws.status.data_ptr(), ctypes.byref(sh), ctypes.byref(attrs),
                       torch.cuda.current_stream().cuda_stream)
    for field, value, code in (("head_dim", 64, -3), ("page_size", 12, -2), ("kv_dtype", 7, -4)):
        sh = _cabi.Shape(*[getattr(shape, f) for f, _ in shape._fields_])
        setattr(sh, field, value)
        assert rpa_lib.ejk_rpa_launch(*args(sh)) == code, field
    torch.cuda.synchronize()
    assert bool((o == 7.0).all())


# ---- odd numbers of kv heads: MQA, or one rank's share of an 8-way head split of an 8-kv-head model.  The plain
# operator reads a dense [P, page, 2*Hkv, D] pool; the v3 cache pads the combined heads to four per 32-bit word
# (merge_kv, _kernel.py:45-57), two padding heads that the page write zeroes and the attention steps over. ----
def _odd_cases():
    mk = lambda ql, kl, **kw: make_ragged_batch(ql, kl, kv_dtype=FP8, **kw)
    yield "mqa", mk([1, 1, 9, 1], [600, 33, 140, 2100], num_q_heads=8, num_kv_heads=1, head_dim=128, page_size=16, seed=91)
    yield "three_heads", mk([1, 20, 2], [300, 90, 1000], num_q_heads=12, num_kv_heads=3, head_dim=128, page_size=32, seed=92,
                            sliding_window=400)
    yield "mqa_d256", mk([1, 3], [500, 64], num_q_heads=4, num_kv_heads=1, head_dim=256, page_size=16, seed=93)


ODD = list(_odd_cases())
ODD_IDS = [n for n, _ in ODD]


def _check_padded_cache(new_cache, before, b):
    """Rows the step wrote: the pool's bytes in the first 2*Hkv heads, zeros in the padding heads; every other row as
    it was (the padding heads keep their fill)."""
    Hkv, page = b.meta["num_kv_heads"], b.meta["page_size"]
    P = b.kv_pages.shape[0]
    got = new_cache.view(torch.uint8).reshape(P, page, -1, new_cache.shape[-1]).cpu()
    old = before.view(torch.uint8).reshape(got.shape).cpu()
    pool = b.kv_pages.view(torch.uint8).cpu()
    assert torch.equal(got[:, :, : 2 * Hkv], pool), "page write: live heads"
    written = torch.zeros(P, page, dtype=torch.bool)
    tab = b.block_tables.cpu()
    for s, (ql, kl) in enumerate(zip(b.meta["q_lens"], b.meta["kv_lens"])):
        for pos in range(kl - ql, kl):
            written[int(tab[s, pos // page]), pos % page] = True
    assert got.shape[2] == 2 * Hkv + 2
    assert torch.count_nonzero(got[:, :, 2 * Hkv :][written]) == 0, "padding heads of written rows are zeros"
    assert torch.equal(got[:, :, 2 * Hkv :][~written], old[:, :, 2 * Hkv :][~written]), "other rows untouched"


@pytest.mark.parametrize("name,b", ODD, ids=ODD_IDS)
def test_oracle_v3_with_padded_combined_heads(name, b):
    keys, values, cache, tab, dist = to_v3_inputs(b)
    assert cache.shape[2] * cache.shape[3] == 2 * b.meta["num_kv_heads"] + 2 and cache.shape[3] == 4
    out, new_cache = v3_reference(b.queries, keys, values, cache, b.context_lens, tab, b.query_start_loc, dist,
                                  softmax_scale=b.softmax_scale, sliding_window=b.sliding_window)
    np.testing.assert_allclose(out, dense_reference(*b.args(), **b.kwargs()), atol=1e-12)
    _check_padded_cache(new_cache, cache, b)


@pytest.mark.gpu
@pytest.mark.parametrize("name,b", ODD, ids=ODD_IDS)
def test_cuda_e4m3_with_an_odd_number_of_kv_heads(rpa_lib, name, b):
    import ejkernel_b200 as ej
    from tests.helpers import run_cuda, status_word

    bc = b.to("cuda")
    want, wb = dense_reference(*b.args(), **b.kwargs(), return_weight_bound=True)
    out = run_cuda(bc)  # the plain operator on the dense pool
    assert status_word(bc) == 0
    _within(out, want, wb, b.total_tokens)
    keys, values, cache, tab, dist = to_v3_inputs(bc)
    before = cache.clone()
    out3, new_cache = ej.ragged_page_attention_v3(bc.queries, keys, values, cache, bc.context_lens, tab, bc.query_start_loc,
                                                  dist, softmax_scale=b.softmax_scale, sliding_window=b.sliding_window)
    torch.cuda.synchronize()
    _within(out3, want, wb, b.total_tokens)
    _check_padded_cache(new_cache, before, b)


# ---- head_dim 64: the v3 cache pads a row to 128 bytes, and the operator attends it as head_dim 128 with the upper half
# of every query zero (the padding lanes of K meet zeros; those of V land in output columns that are not stored).  The
# plain operator's dense e4m3 pool has 64-byte rows, half a swizzle row: refused. ----
def _d64_cases():
    mk = lambda ql, kl, **kw: make_ragged_batch(ql, kl, kv_dtype=FP8, **kw)
    yield "d64", mk([1, 1, 12, 1], [700, 20, 130, 3000], num_q_heads=8, num_kv_heads=2, head_dim=64, page_size=16, seed=95)
    yield "d64_mqa_window", mk([1, 30], [900, 200], num_q_heads=8, num_kv_heads=1, head_dim=64, page_size=32, seed=96,
                               sliding_window=300, logits_soft_cap=20.0)


D64 = list(_d64_cases())


@pytest.mark.parametrize("name,b", D64, ids=[n for n, _ in D64])
def test_oracle_v3_e4m3_head_dim_64(name, b):
    keys, values, cache, tab, dist = to_v3_inputs(b)
    assert cache.shape[-1] == 128
    out, _ = v3_reference(b.queries, keys, values, cache, b.context_lens, tab, b.query_start_loc, dist,
                          softmax_scale=b.softmax_scale, sliding_window=b.sliding_window, logits_soft_cap=b.logits_soft_cap)
    np.testing.assert_allclose(out, dense_reference(*b.args(), **b.kwargs()), atol=1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("q_scale", [None, 0.05])
@pytest.mark.parametrize("name,b", D64, ids=[n for n, _ in D64])
def test_cuda_v3_e4m3_head_dim_64(rpa_lib, name, b, q_scale):
    import ejkernel_b200 as ej
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention

    bc = b.to("cuda")
    keys, values, cache, tab, dist = to_v3_inputs(bc)
    kw = dict(softmax_scale=b.softmax_scale, sliding_window=b.sliding_window, logits_soft_cap=b.logits_soft_cap,
              q_scale=q_scale, v_scale=0.75)
    out, new_cache = ej.ragged_page_attention_v3(bc.queries, keys, values, cache, bc.context_lens, tab, bc.query_start_loc,
                                                 dist, **kw)
    torch.cuda.synchronize()
    ck, cv, cc, ctab, cdist = to_v3_inputs(b)
    want, want_cache, wb = v3_reference(b.queries, ck, cv, cc, b.context_lens, ctab, b.query_start_loc, cdist, **kw,
                                        return_weight_bound=True)
    _within(out, want, wb, b.total_tokens)
    # rows the step wrote equal the oracle's (data, zeroed padding); the others keep their fill
    assert torch.equal(new_cache.view(torch.uint8).cpu(), want_cache.view(torch.uint8))
    with pytest.raises(NotImplementedError):
        ragged_page_attention(*bc.args(), softmax_scale=b.softmax_scale)  # dense pool with 64-byte rows
