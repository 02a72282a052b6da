"""``ragged_page_attention_v3``: the KV-cache page write fused with attention.  The CPU part pins the
oracle restatement; the GPU part checks the CUDA path through the C ABI: the cache must come back
bit-identical to the complete pool (the page write is pure data movement) and the output must match
the oracle within the bf16 tolerance."""

import numpy as np
import pytest
import torch

from ejkernel_b200.utils import make_ragged_batch, make_workload, to_v3_inputs
from oracle.rpa_oracle import dense_reference, v3_reference
from tests.helpers import assert_parity


def _cases():
    yield "decode", make_ragged_batch([1, 1, 1], [300, 17, 64], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=61)
    yield "mixed", make_ragged_batch([1, 40, 3, 130], [500, 40, 77, 900], num_q_heads=8, num_kv_heads=2, head_dim=128,
                                     page_size=16, seed=62, sliding_window=256, logits_soft_cap=30.0)
    yield "d256", make_ragged_batch([2, 70], [100, 300], num_q_heads=4, num_kv_heads=2, head_dim=256, page_size=32, seed=63)
    # head_dim 64: the cache's last dim is padded to 128 (align_to(D, 128), _kernel.py:45-57)
    yield "d64_padded", make_ragged_batch([1, 33, 2, 90], [700, 33, 130, 400], num_q_heads=8, num_kv_heads=2, head_dim=64,
                                          page_size=16, seed=65, sliding_window=300)
    # ... and with a page size that is no power of two (8-token TMA boxes) / no multiple of 8 (cp.async gather)
    yield "d64_padded_page24", make_ragged_batch([1, 20], [333, 100], num_q_heads=4, num_kv_heads=2, head_dim=64,
                                                 page_size=24, seed=66)
    yield "d64_padded_page12", make_ragged_batch([1, 20], [333, 100], num_q_heads=4, num_kv_heads=2, head_dim=64,
                                                 page_size=12, seed=67)
    yield "empty_seq", make_ragged_batch([1, 0, 5], [50, 20, 5], num_q_heads=4, num_kv_heads=4, head_dim=128, page_size=8,
                                         max_num_seqs=5, pad_query_rows=3, seed=64)


def _check_cache(new_cache, old_cache, b):
    """First head_dim lanes: the complete pool, bit for bit.  Padding lanes (head_dim not a multiple of 128):
    zero in the rows the call wrote (merge_kv pads with zeros), untouched elsewhere."""
    P, page, C2, D = b.kv_pages.shape
    flat = new_cache.reshape(P, page, C2, -1)
    assert torch.equal(flat[..., :D], b.kv_pages), "page write must be bit-exact"
    if flat.shape[-1] != D:
        pad_new, pad_old = flat[..., D:].float(), old_cache.reshape(P, page, C2, -1)[..., D:].float()
        written = torch.zeros(P, page, dtype=torch.bool, device=flat.device)
        m = b.meta
        for s_, (ql, kl) in enumerate(zip(m["q_lens"], m["kv_lens"])):
            if ql:
                pos = torch.arange(kl - ql, kl, device=flat.device)
                written[b.block_tables[s_, (pos // page).long()].long(), (pos % page).long()] = True
        assert torch.count_nonzero(pad_new[written]) == 0
        assert torch.equal(pad_new[~written], pad_old[~written])


@pytest.mark.parametrize("name,b", list(_cases()), ids=[n for n, _ in _cases()])
def test_oracle_v3_restores_the_pool_and_matches_v1(name, b):
    keys, values, cache, tab_flat, dist = to_v3_inputs(b)
    out, new_cache = v3_reference(b.queries, keys, values, cache, b.context_lens, tab_flat, b.query_start_loc, dist,
                                  softmax_scale=b.softmax_scale, sliding_window=b.sliding_window,
                                  logits_soft_cap=b.logits_soft_cap)
    _check_cache(new_cache, cache, b)
    want = dense_reference(*b.args(), **b.kwargs())
    np.testing.assert_allclose(out, want, atol=1e-12)
    # scales: k_scale multiplies the logits, v_scale the output (_kernel.py:262-263,290-291)
    out2, _ = v3_reference(b.queries, keys, values, cache, b.context_lens, tab_flat, b.query_start_loc, dist,
                           softmax_scale=b.softmax_scale / 2.0, k_scale=2.0, v_scale=3.0,
                           sliding_window=b.sliding_window, logits_soft_cap=b.logits_soft_cap)
    np.testing.assert_allclose(out2, 3.0 * want, atol=1e-12)


def test_v3_is_registered_with_the_reference_signature():
    import inspect

    import ejkernel_b200 as ej

    impl = ej.kernel_registry.get("ragged_page_attention_v3", platform="cuda", backend="gpu")
    names = list(inspect.signature(impl).parameters)
    assert names == ["queries", "keys", "values", "kv_cache", "kv_lens", "block_tables", "query_start_loc", "distribution",
                     "softmax_scale", "sliding_window", "logits_soft_cap", "q_scale", "k_scale", "v_scale",
                     "chunk_prefill_size", "num_kv_pages_per_block", "num_queries_per_block", "vmem_limit_bytes"]
    assert inspect.signature(impl).parameters["softmax_scale"].default == 1.0
    pub = list(inspect.signature(ej.ragged_page_attention_v3).parameters)
    assert pub[:8] == names[:8] and pub[-5:] == ["platform", "cfg", "mesh", "in_specs", "out_specs"]


@pytest.mark.gpu
@pytest.mark.parametrize("name,b", list(_cases()), ids=[n for n, _ in _cases()])
def test_cuda_v3_matches_oracle_and_restores_the_pool(rpa_lib, name, b):
    import ejkernel_b200 as ej

    bc = b.to("cuda")
    keys, values, cache, tab_flat, dist = to_v3_inputs(bc)
    assert torch.isnan(cache.float()).any()
    before = cache.clone()
    out, new_cache = ej.ragged_page_attention_v3(bc.queries, keys, values, cache, bc.context_lens, tab_flat,
                                                 bc.query_start_loc, dist, softmax_scale=b.softmax_scale,
                                                 sliding_window=b.sliding_window, logits_soft_cap=b.logits_soft_cap)
    torch.cuda.synchronize()
    assert new_cache.data_ptr() == cache.data_ptr(), "the cache is updated in place"
    _check_cache(new_cache, before, bc)
    assert_parity(out, dense_reference(*b.args(), **b.kwargs()), b.total_tokens, what=f"v3 {name}")
    assert torch.count_nonzero(out[b.total_tokens:]) == 0


@pytest.mark.gpu
def test_cuda_v3_scales_and_full_size_decode(rpa_lib):
    import ejkernel_b200 as ej

    b = make_workload("c2", num_seqs=64, device="cuda")
    keys, values, cache, tab_flat, dist = to_v3_inputs(b)
    ref = ej.ragged_page_attention(*b.args(), softmax_scale=b.softmax_scale, cfg=ej.RaggedPageAttention().heuristic_cfg())
    out, new_cache = ej.ragged_page_attention_v3(b.queries, keys, values, cache, b.context_lens, tab_flat,
                                                 b.query_start_loc, dist, softmax_scale=b.softmax_scale / 4.0,
                                                 k_scale=4.0, v_scale=2.0)
    torch.cuda.synchronize()
    assert torch.equal(new_cache.view(b.kv_pages.shape), b.kv_pages)
    # same kernels on the same bytes: v3 with folded scales reproduces v1 exactly (x2 is exact in bf16)
    assert torch.equal(out, ref * 2.0)


@pytest.mark.gpu
def test_a_refused_v3_call_leaves_the_cache_untouched_and_launches_nothing(rpa_lib):
    """Every host-side check of the launch comes before the page write: a call that returns a negative code
    has not modified the cache (a retry would otherwise apply the write twice) and has launched no kernel."""
    import ctypes

    from ejkernel_b200 import _cabi
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import RpaWorkspace

    b = make_ragged_batch([1, 5], [90, 33], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=71).to("cuda")
    keys, values, cache, tab_flat, dist = to_v3_inputs(b)
    T, Hq, D = b.queries.shape
    shape = _cabi.Shape(T, 2, b.block_tables.shape[1], cache.shape[0], 16, Hq, 2, D, _cabi.BF16)
    ws = RpaWorkspace(shape, b.queries.device)
    out = torch.full_like(b.queries, 7.0)
    attrs = _cabi.Attrs(b.softmax_scale, 0.0, 0, 0, 0, 0, 0)
    before = cache.clone()
    P = lambda t: None if t is None else t.data_ptr()

    def call(**kw):
        a = dict(queries=P(b.queries), keys=P(keys), values=P(values), cache=P(cache), kv_lens=P(b.context_lens),
                 tab=P(tab_flat), cu=P(b.query_start_loc), dist=P(dist), out=P(out), ws=P(ws.buffer), ws_bytes=ws.nbytes,
                 attrs=attrs)
        a.update(kw)
        return rpa_lib.ejk_rpa_v3_launch(a["queries"], a["keys"], a["values"], a["cache"], a["kv_lens"], a["tab"], a["cu"],
                                         a["dist"], a["out"], a["ws"], a["ws_bytes"], P(ws.status), ctypes.byref(shape),
                                         ctypes.byref(a["attrs"]), torch.cuda.current_stream().cuda_stream)

    nan_scale = _cabi.Attrs(float("nan"), 0.0, 0, 0, 0, 0, 0)
    for what, kw, code in (
        ("null kv_lens", dict(kv_lens=None), -1),
        ("null block_tables", dict(tab=None), -1),
        ("null query_start_loc", dict(cu=None), -1),
        ("null out", dict(out=None), -1),
        ("null workspace", dict(ws=None), -1),
        ("short workspace", dict(ws_bytes=1024), -5),
        ("misaligned workspace", dict(ws=P(ws.buffer) + 16), -5),
        ("cache not 16-byte aligned", dict(cache=P(cache) + 2), -8),
        ("queries not 16-byte aligned", dict(queries=P(b.queries) + 2), -8),
        ("NaN scale", dict(attrs=nan_scale), -6),
    ):
        rc = call(**kw)
        assert rc == code, (what, rc, _cabi.error_string(rc))
        assert rpa_lib.ejk_rpa_last_launch_count() == 0, what
        torch.cuda.synchronize()
        assert torch.equal(cache.view(torch.int16), before.view(torch.int16)), f"{what}: the cache was modified"
        assert bool((out == 7.0).all()), f"{what}: something was launched"
    assert call() == 0  # and the same arguments, unbroken, go through
    torch.cuda.synchronize()
    assert torch.equal(cache.view(b.kv_pages.shape), b.kv_pages)
