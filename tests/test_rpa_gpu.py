"""Parity of the sm_100a kernels (called through the C ABI via the registered operator) with the
CPU oracle on the same seeded inputs.  Tolerance: atol = rtol = 2e-2 for bf16 with fp32
accumulation, plus |err| <= 3e-2 * rms(expected) + 1e-2 * |expected| because on N(0,1) inputs with
long contexts the outputs themselves are smaller than atol.  Index work (page gather, masking) is checked
bit-exactly through integer-valued cases."""

import numpy as np
import pytest
import torch

from ejkernel_b200.utils import make_ragged_batch, make_workload
from tests.helpers import assert_parity, oracle, run_cuda, status_word

pytestmark = pytest.mark.gpu


def _check(batch, what, **kw):
    bc = batch.to("cuda")
    out = run_cuda(bc)
    assert out.shape == bc.queries.shape and out.dtype == bc.queries.dtype
    assert status_word(bc) == 0, "clean inputs must leave the status word at 0"
    return assert_parity(out, oracle(batch), batch.total_tokens, what=what, **kw)


def test_golden_fixtures(rpa_lib):
    from pathlib import Path
    from tests.golden.make_golden import cases
    golden = np.load(Path(__file__).parent / "golden" / "rpa_golden.npz")
    for name, b in cases():
        out = run_cuda(b)
        assert_parity(out, golden[f"{name}.out"].astype(np.float64), b.total_tokens, what=f"golden {name}")


def test_c1_decode_toy(rpa_lib):
    _check(make_workload("c1"), "c1")


@pytest.mark.parametrize("name,num_seqs,len_scale", [("c2", 24, 0.25), ("c4", 6, 0.25), ("c5", 3, 0.03)])
def test_decode_workloads_reduced(rpa_lib, name, num_seqs, len_scale):
    _check(make_workload(name, num_seqs=num_seqs, len_scale=len_scale), name)


def test_c3_mixed_reduced(rpa_lib):
    _check(make_workload("c3", num_seqs=12, len_scale=0.125), "c3")


def test_reference_tpu_test_shapes(rpa_lib):
    # shapes of test/kernels/_pallas/tpu/test_ragged_page_attention.py:465-554 of the reference
    b = make_ragged_batch([64, 64], [64, 96], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16,
                          pages_per_seq=8, num_pages=32, seed=11)
    _check(b, "prefill 2 seqs")
    b = make_ragged_batch([100, 50, 40, 10], [128, 64, 192, 96], num_q_heads=8, num_kv_heads=2, head_dim=128,
                          page_size=16, pages_per_seq=12, num_pages=64, seed=12)
    _check(b, "mixed 4 seqs")


@pytest.mark.parametrize("head_dim", [64, 128, 256])
@pytest.mark.parametrize("hq,hkv", [(8, 8), (8, 4), (16, 4), (8, 1), (32, 2), (6, 2)])
def test_head_configs(rpa_lib, head_dim, hq, hkv):
    b = make_ragged_batch([1, 3, 1, 17], [200, 64, 1, 90], num_q_heads=hq, num_kv_heads=hkv, head_dim=head_dim,
                          page_size=16, seed=hq * 100 + hkv + head_dim)
    _check(b, f"hq{hq} hkv{hkv} d{head_dim}")


@pytest.mark.parametrize("page_size", [1, 3, 4, 8, 12, 16, 24, 32, 40, 48, 64, 96, 128, 136])
def test_page_sizes(rpa_lib, page_size):
    """Multiples of 8 take the TMA gather (boxes of the largest power of two dividing the page, 8 to 64 tokens, so
    that no box straddles a page), every other size the cp.async gather; mixed batch, so the tensor-tile kernel's
    8-token boxes are covered too."""
    b = make_ragged_batch([1, 1, 5, 1, 70], [777, 129, 300, 64, 400], num_q_heads=8, num_kv_heads=2, head_dim=128,
                          page_size=page_size, seed=page_size)
    _check(b, f"page_size {page_size}")


@pytest.mark.parametrize("kv_len", list(range(1, 20)) + [63, 64, 65, 127, 128, 129, 255, 256, 257, 1023, 1025])
def test_every_kv_remainder(rpa_lib, kv_len):
    q_lens = [1, min(kv_len, 2), min(kv_len, 9)]
    b = make_ragged_batch(q_lens, [kv_len] * 3, num_q_heads=4, num_kv_heads=2, head_dim=128, page_size=16, seed=kv_len)
    _check(b, f"kv_len {kv_len}")


@pytest.mark.parametrize("q_len", [1, 2, 3, 7, 8, 9, 127, 128, 129])
def test_query_lengths(rpa_lib, q_len):
    b = make_ragged_batch([q_len, 1, q_len], [q_len + 300, 50, q_len], num_q_heads=8, num_kv_heads=2, head_dim=128,
                          page_size=16, seed=q_len)
    _check(b, f"q_len {q_len}")


@pytest.mark.parametrize("window", [1, 5, 64, 100, 1000])
@pytest.mark.parametrize("cap", [None, 30.0])
def test_window_and_soft_cap(rpa_lib, window, cap):
    b = make_ragged_batch([1, 4, 1, 33], [700, 350, 20, 400], num_q_heads=8, num_kv_heads=4, head_dim=128,
                          page_size=16, seed=window, sliding_window=window, logits_soft_cap=cap)
    _check(b, f"window {window} cap {cap}")


def test_window_invariants_of_reference_tests(rpa_lib):
    # test/kernels/_triton/test_ragged_page_attention.py:437-487: a window larger than every context
    # equals no window; a huge soft cap approximates none
    base = make_ragged_batch([1, 6], [200, 300], num_q_heads=8, num_kv_heads=4, head_dim=64, page_size=16, seed=5)
    o0 = run_cuda(base)
    o1 = run_cuda(base, sliding_window=1000)
    assert torch.equal(o0, o1)
    o2 = run_cuda(base, logits_soft_cap=1e6)
    assert (o0.float() - o2.float()).abs().max().item() < 0.1
    o3 = run_cuda(base, sliding_window=7)
    assert (o0.float() - o3.float()).abs().max().item() > 1e-6


def test_prefill_tiles_many_items_per_cta(rpa_lib):
    """More 128-row tiles than SMs, so every persistent CTA of the tcgen05 kernel walks several items
    (query-tile reload, O hand-over between items, ring reuse), with ragged last tiles."""
    b = make_ragged_batch([700, 1, 333, 2, 129], [1500, 40, 333, 900, 4000], num_q_heads=8, num_kv_heads=2,
                          head_dim=128, page_size=16, seed=51)
    _check(b, "many prefill tiles")
    b = make_ragged_batch([300, 260], [2100, 300], num_q_heads=16, num_kv_heads=2, head_dim=64, page_size=32,
                          seed=52, sliding_window=700, logits_soft_cap=40.0)
    _check(b, "prefill window+cap d64")
    b = make_ragged_batch([200], [1000], num_q_heads=4, num_kv_heads=2, head_dim=256, page_size=8, seed=53)
    b.softmax_aux = torch.tensor([[0.5, -1.0], [2.0, 0.0]])
    _check(b, "prefill d256 sinks")


def test_prefill_threshold_does_not_change_results_beyond_tolerance(rpa_lib):
    """The same batch through 8-row split-KV tiles only (prefill_rows=0), through 128-row tensor tiles
    for every multi-row sequence (prefill_rows=1) and with the default threshold."""
    from ejkernel_b200 import _cabi
    b = make_ragged_batch([1, 40, 3, 160, 1], [800, 640, 77, 1700, 9], num_q_heads=8, num_kv_heads=2, head_dim=128,
                          page_size=16, seed=54)
    want = oracle(b)
    old = _cabi.get_option("prefill_rows")
    try:
        for rows in (0, 1, 64, 4096):
            _cabi.set_option("prefill_rows", rows)
            out = run_cuda(b)
            assert_parity(out, want, b.total_tokens, what=f"prefill_rows={rows}")
    finally:
        _cabi.set_option("prefill_rows", old)


def test_prefill_tile_kernel_shapes(rpa_lib):
    """The tcgen05 tile kernel on ragged tiles, windows, caps, sinks, one-tile items, sequences whose length
    is not a multiple of the 64-token stage, every head_dim, and fp16."""
    b = make_ragged_batch([700, 1, 333, 2, 129], [1500, 40, 333, 900, 4000], num_q_heads=8, num_kv_heads=2,
                          head_dim=128, page_size=16, seed=71)
    _check(b, "many tiles")
    b = make_ragged_batch([300, 260, 17], [2100, 300, 97], num_q_heads=16, num_kv_heads=2, head_dim=64,
                          page_size=32, seed=72, sliding_window=700, logits_soft_cap=40.0)
    _check(b, "window+cap d64")
    b = make_ragged_batch([96, 33, 64], [96, 1000, 191], num_q_heads=4, num_kv_heads=4, head_dim=128, page_size=8,
                          seed=73)
    b.softmax_aux = torch.randn(4, 2, generator=torch.Generator().manual_seed(5))
    _check(b, "g1 sinks page8")
    b = make_ragged_batch([512, 512], [4096, 513], num_q_heads=32, num_kv_heads=8, head_dim=128, page_size=64,
                          seed=74, dtype=torch.float16)
    _check(b, "fp16 chunked prefill")
    b = make_ragged_batch([130, 400, 1], [1000, 450, 77], num_q_heads=8, num_kv_heads=4, head_dim=256, page_size=16,
                          seed=75, sliding_window=300)
    _check(b, "d256 one tile per CTA, window")


@pytest.mark.parametrize("which", ["split-KV kernel", "prefill kernel"])
def test_a_wait_that_runs_out_sets_the_timeout_bit_and_leaves_the_context_usable(rpa_lib, which):
    """Every in-kernel wait is bounded.  The test hook makes CTA 0 never announce its first KV stage
    (nothing faults, nothing hangs): the waits on it expire after ``wait_ms``, the CTA gives up, frees
    what it holds and returns, the status word carries EJK_RPA_ST_TIMEOUT, and the next call on the same
    context is correct again."""
    from ejkernel_b200 import _cabi
    if which == "prefill kernel":
        b = make_ragged_batch([200, 1], [900, 300], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=95)
    else:
        b = make_ragged_batch([1, 1, 2], [700, 64, 1500], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=96)
    want = oracle(b)
    bc = b.to("cuda")
    old = _cabi.get_option("wait_ms")
    try:
        _cabi.set_option("wait_ms", 50)
        _cabi.set_option("test_withhold", 2 if which == "prefill kernel" else 1)
        run_cuda(bc)
        torch.cuda.synchronize()
        word = status_word(bc)
        assert word & _cabi.ST_TIMEOUT, (which, word)
        assert "wait" in " ".join(_cabi.decode_status(word)).lower() or "time" in " ".join(_cabi.decode_status(word)).lower()
    finally:
        _cabi.set_option("test_withhold", 0)
        _cabi.set_option("wait_ms", old)
    out = run_cuda(bc)
    assert status_word(bc) == 0
    assert_parity(out, want, b.total_tokens, what=f"after a timed-out {which}")


def test_tile_hints_change_the_partition_not_the_result(rpa_lib, tmp_path):
    """``num_kv_pages_per_block`` (KV-chunk floor) and ``num_queries_per_block`` (threshold of the tensor
    tiles) of RaggedPageAttentionConfig reach the planner per call; every setting must match the oracle,
    and the autotuner must return one of its candidates and persist it."""
    from ejkernel_b200.modules.operations import RaggedPageAttention, RaggedPageAttentionConfig
    from ejkernel_b200.modules.operations.tuning import PersistentCache
    b = make_ragged_batch([1, 40, 3, 160, 1], [2800, 640, 77, 1700, 900], num_q_heads=8, num_kv_heads=2, head_dim=128,
                          page_size=16, seed=91)
    want = oracle(b)
    bc = b.to("cuda")
    kern = RaggedPageAttention(cache=PersistentCache("ragged_page_attention", str(tmp_path / "t.json"),
                                                     cfg_type=RaggedPageAttentionConfig))
    for kvp, nq in ((None, None), (4, None), (128, None), (None, 1), (None, 100), (8, 3)):
        cfg = RaggedPageAttentionConfig(num_kv_pages_per_block=kvp, num_queries_per_block=nq, platform="cuda", backend="gpu")
        out = kern.run(*bc.args(), **bc.kwargs(), cfg=cfg)
        assert_parity(out, want, b.total_tokens, what=f"hints kv_pages={kvp} queries={nq}")
    best = kern.autotune(*bc.args(), softmax_scale=bc.softmax_scale)
    assert best in kern.candidate_cfgs(page_size=16)
    assert kern.lookup_cfg(bc.queries, bc.kv_pages, bc.block_tables) == best
    assert_parity(kern.run(*bc.args(), **bc.kwargs(), cfg=best), want, b.total_tokens, what="tuned cfg")


def test_prefill_items_split_along_kv(rpa_lib):
    """With room in the workspace the tile kernel cuts the stage sequence of all (item, kv head) pairs
    into one quota per CTA; items that straddle a quota boundary are finished by several CTAs and
    combined by the part that arrives last, in part order.  Few long items (every one is split many
    ways), many short ones, one-tile items, windows, sinks: all must match the oracle, repeat bitwise,
    and agree with the unsplit schedule within the tolerance."""
    from ejkernel_b200 import _cabi
    cases = [
        dict(q=[256], kv=[6000], hq=4, hkv=1, d=128, page=16, kw={}),                       # 4 long items -> 148 CTAs
        dict(q=[512, 300], kv=[2048, 5000], hq=8, hkv=2, d=128, page=32, kw=dict(sliding_window=3000)),
        dict(q=[40] * 12 + [1, 1], kv=[700 + 37 * i for i in range(12)] + [900, 50], hq=16, hkv=2, d=64, page=16, kw={}),
        dict(q=[129, 500], kv=[129, 3100], hq=8, hkv=4, d=256, page=16, kw=dict(logits_soft_cap=30.0)),
    ]
    old = _cabi.get_option("prefill_split")
    try:
        for i, c in enumerate(cases):
            b = make_ragged_batch(c["q"], c["kv"], num_q_heads=c["hq"], num_kv_heads=c["hkv"], head_dim=c["d"],
                                  page_size=c["page"], seed=110 + i, **c["kw"])
            if i == 1:
                b.softmax_aux = torch.randn(c["hq"], 2, generator=torch.Generator().manual_seed(6))
            want = oracle(b)
            _cabi.set_option("prefill_split", 1)
            outs = [run_cuda(b) for _ in range(3)]
            assert status_word(b.to("cuda")) == 0
            _cabi.set_option("prefill_split", 0)
            whole = run_cuda(b)
            assert_parity(outs[0], want, b.total_tokens, what=f"split case {i}")
            assert_parity(whole, want, b.total_tokens, what=f"unsplit case {i}")
            for o in outs[1:]:
                assert torch.equal(o, outs[0]), i
    finally:
        _cabi.set_option("prefill_split", old)


def test_idle_tile_with_short_pieces_many_launches(rpa_lib):
    """Items with rows for one tile only leave the CTA's second tile idle; its softmax warps then skip
    whole items without waiting for anybody and can be several items ahead of the MMA role that checks
    on them -- whenever pieces are shorter than the stage ring: a quota that begins a stage or two
    before an item's end (KV split), or a queue of one-stage items (dynamic schedule).  How far ahead
    depends on timing, so every case is launched many times; each launch must leave the status word
    clean (no wait may run out) and repeat the first bitwise."""
    from ejkernel_b200 import _cabi
    cases = [
        # 32 (item, head) pairs of 79 stages, quota 18: CTAs 57 and 136 begin 1 stage before an item's end
        dict(q=[16] * 4, kv=[5000] * 4, hq=32, hkv=8, d=128, split=1),
        # 32 pairs of 313 stages, quota 68: CTA 23 begins 1 stage before an item's end
        dict(q=[16] * 4, kv=[20000] * 4, hq=32, hkv=8, d=128, split=1),
        # 1200 pairs of one stage each on the dynamic queue
        dict(q=[16] * 300, kv=[40 + (i % 24) for i in range(300)], hq=16, hkv=4, d=64, split=0),
    ]
    old = (_cabi.get_option("prefill_split"), _cabi.get_option("wait_ms"))
    try:
        _cabi.set_option("wait_ms", 200)
        for i, c in enumerate(cases):
            b = make_ragged_batch(c["q"], c["kv"], num_q_heads=c["hq"], num_kv_heads=c["hkv"], head_dim=c["d"],
                                  page_size=16, seed=140 + i)
            bc = b.to("cuda")
            _cabi.set_option("prefill_split", c["split"])
            first = run_cuda(bc)
            assert status_word(bc) == 0, i
            assert_parity(first, oracle(b), b.total_tokens, what=f"idle tile case {i}")
            for rep in range(40):
                again = run_cuda(bc)
                assert status_word(bc) == 0, (i, rep)
                assert torch.equal(again, first), (i, rep)
    finally:
        _cabi.set_option("prefill_split", old[0])
        _cabi.set_option("wait_ms", old[1])


def test_prefill_queue_order_does_not_depend_on_thread_timing(rpa_lib):
    """The KV split cuts the prefill items in queue order, so the order in which the planner queues
    items of one length bucket decides where partial sums are combined.  Many multi-token sequences
    with nearly equal lengths (one bucket, different stage counts), launched repeatedly: every
    launch must repeat the first bit for bit."""
    for i, (hq, hkv, d) in enumerate([(1, 1, 256), (8, 2, 128), (16, 4, 64)]):
        n = 39
        b = make_ragged_batch([33 + (j * 7) % 30 for j in range(n)], [900 + 37 * ((j * 11) % n) for j in range(n)],
                              num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=16, seed=150 + i)
        bc = b.to("cuda")
        first = run_cuda(bc)
        assert status_word(bc) == 0
        assert_parity(first, oracle(b), b.total_tokens, what=f"reproducible queue case {i}")
        for rep in range(12):
            assert torch.equal(run_cuda(bc), first), (i, rep)


def test_overlapped_launches_equal_stream_order_bitwise(rpa_lib):
    """With programmatic dependent launches the prefill kernel starts under the planner's tail and the
    split-KV kernel runs beside the prefill kernel's last CTAs; the kernels write different rows, so
    the output is bitwise the same as in plain stream order -- mixed, decode-only and prefill-only batches."""
    from ejkernel_b200 import _cabi
    batches = [
        make_ragged_batch([300, 1, 1, 200, 1, 3], [2000, 900, 3000, 260, 17, 640], num_q_heads=16, num_kv_heads=4,
                          head_dim=128, page_size=16, seed=81),
        make_ragged_batch([1] * 40, [int(x) for x in np.random.default_rng(5).integers(1, 3000, 40)], num_q_heads=8,
                          num_kv_heads=2, head_dim=128, page_size=32, seed=82),
        make_ragged_batch([512], [1536], num_q_heads=8, num_kv_heads=8, head_dim=64, page_size=64, seed=83),
    ]
    old = _cabi.get_option("overlap")
    try:
        for i, b in enumerate(batches):
            want = oracle(b)
            _cabi.set_option("overlap", 1)
            outs = [run_cuda(b) for _ in range(3)]
            _cabi.set_option("overlap", 0)
            plain = run_cuda(b)
            assert_parity(outs[0], want, b.total_tokens, what=f"overlap batch {i}")
            for o in outs:
                assert torch.equal(o, plain), i
    finally:
        _cabi.set_option("overlap", old)


def test_more_sequences_than_the_planner_caches(rpa_lib):
    """The planner keeps the lengths of the first 2048 sequences in shared memory between its passes
    and re-reads the others from global memory; 2500 short sequences (a few of them multi-token, some
    slots unused) go through both routes."""
    rng = np.random.default_rng(77)
    n = 2500
    kv = [int(x) for x in rng.integers(1, 200, n)]
    ql = [1] * n
    for i in (3, 700, 2047, 2048, 2499):
        ql[i] = min(kv[i], 5)
    b = make_ragged_batch(ql, kv, num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=16, seed=98, max_num_seqs=n + 7)
    _check(b, "2500 sequences")


def test_queue_order_does_not_change_results(rpa_lib):
    """The planner queues split-KV work items longest first (option ``sort_items``); inside a length
    bucket the order depends on atomics.  Every item writes its own rows or its own partial slot and
    partials are combined in chunk order, so the output is bitwise the same as in sequence order, run
    after run."""
    from ejkernel_b200 import _cabi
    b = make_ragged_batch([1, 2, 1, 5, 1, 1, 3], [5000, 37, 2900, 9000, 700, 64, 1300], num_q_heads=16, num_kv_heads=4,
                          head_dim=128, page_size=16, seed=97, sliding_window=6000)
    want = oracle(b)
    old = _cabi.get_option("sort_items")
    try:
        _cabi.set_option("sort_items", 0)
        plain = run_cuda(b)
        _cabi.set_option("sort_items", 1)
        outs = [run_cuda(b) for _ in range(4)]
    finally:
        _cabi.set_option("sort_items", old)
    assert_parity(plain, want, b.total_tokens, what="sequence order")
    for o in outs:
        assert torch.equal(o, plain)


def test_fused_merge_agrees_with_merge_kernel(rpa_lib):
    """The split-KV kernel's last-arriver merge combines the chunks of a tile in chunk order whichever chunk arrives
    last: bitwise the same run after run.  The separate merge kernel is as reproducible; with few rows and many
    chunks it lets several warps sum every K-th chunk of a row, i.e. it adds the same float32 terms in another order,
    so the two agree to the last float32 bits -- after the rounding to bf16 that is at most one output ulp, and
    nearly everywhere none."""
    from ejkernel_b200 import _cabi
    b = make_ragged_batch([1, 1, 4, 1, 2], [6000, 37, 2900, 9000, 700], num_q_heads=16, num_kv_heads=2,
                          head_dim=128, page_size=16, seed=61, max_num_seqs=7)
    b.softmax_aux = torch.randn(16, 2, generator=torch.Generator().manual_seed(4))
    want = oracle(b)
    old = _cabi.get_option("fused_merge"), _cabi.get_option("waves")
    try:
        _cabi.set_option("waves", 64)  # many chunks per tile
        _cabi.set_option("fused_merge", 2)  # force it (by default such a batch gets the separate kernel)
        fused = [run_cuda(b) for _ in range(3)]
        _cabi.set_option("fused_merge", 0)
        split = [run_cuda(b) for _ in range(3)]
    finally:
        _cabi.set_option("fused_merge", old[0])
        _cabi.set_option("waves", old[1])
    assert_parity(fused[0], want, b.total_tokens, what="fused merge")
    assert_parity(split[0], want, b.total_tokens, what="merge kernel")
    for o in fused[1:]:
        assert torch.equal(o, fused[0])
    for o in split[1:]:
        assert torch.equal(o, split[0])
    # one bf16 ulp is at most 2^-7 of the value
    fa, sa = fused[0].float(), split[0].float()
    assert bool(((fa - sa).abs() <= 2.0**-7 * torch.maximum(fa.abs(), sa.abs()) + 1e-30).all())
    assert float((fa != sa).float().mean()) < 1e-2


@pytest.mark.parametrize("seed", range(24))
def test_random_ragged_batches(rpa_lib, seed):
    """Seeded random batches over the whole argument space: head layout, head_dim, page size (powers
    of two and odd ones), decode / speculative / prefill query lengths, windows, caps, sinks, spare
    sequence slots and padded query rows."""
    rng = np.random.default_rng(9000 + seed)
    hkv = int(rng.choice([1, 2, 4, 8]))
    g = int(rng.choice([1, 2, 3, 4, 8, 16]))
    d = int(rng.choice([64, 128, 256]))
    page = int(rng.choice([1, 4, 8, 16, 16, 32, 64, 24]))
    n = int(rng.integers(1, 9))
    kinds = rng.choice(["decode", "spec", "prefill", "full"], size=n, p=[0.5, 0.2, 0.2, 0.1])
    q_lens, kv_lens = [], []
    for k in kinds:
        kv = int(rng.integers(1, 2500))
        ql = {"decode": 1, "spec": int(rng.integers(2, 6)), "prefill": int(rng.integers(17, 400)), "full": kv}[k]
        ql = min(ql, kv)
        q_lens.append(ql)
        kv_lens.append(kv)
    window = int(rng.integers(1, 1500)) if rng.random() < 0.3 else None
    cap = float(rng.uniform(5, 60)) if rng.random() < 0.3 else None
    b = make_ragged_batch(q_lens, kv_lens, num_q_heads=hkv * g, num_kv_heads=hkv, head_dim=d, page_size=page,
                          max_num_seqs=n + int(rng.integers(0, 3)), pad_query_rows=int(rng.integers(0, 4)),
                          seed=seed, sliding_window=window, logits_soft_cap=cap)
    if rng.random() < 0.25:
        gen = torch.Generator().manual_seed(seed)
        b.softmax_aux = torch.randn(int(rng.choice([hkv, hkv * g])), 3, generator=gen)
    _check(b, f"random seed {seed}: hkv{hkv} g{g} d{d} page{page} q{q_lens} kv{kv_lens} w{window} cap{cap}")


def test_sinks(rpa_lib):
    for rows in ("q", "kv", "flat"):
        b = make_ragged_batch([1, 5, 1], [300, 70, 2000], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=21)
        g = torch.Generator().manual_seed(3)
        if rows == "q":
            b.softmax_aux = torch.randn(8, 4, generator=g)
        elif rows == "kv":
            b.softmax_aux = torch.randn(2, 4, generator=g)
        else:
            b.softmax_aux = torch.randn(3, generator=g)
        _check(b, f"sinks {rows}")


def test_float32_operands_like_the_reference_dtype_test(rpa_lib):
    # test/kernels/_triton/test_ragged_page_attention.py:88-103: output dtype follows the queries' dtype
    b = make_ragged_batch([1, 2, 40], [500, 77, 300], num_q_heads=8, num_kv_heads=2, head_dim=64, page_size=16, seed=4)
    bc = b.to("cuda")
    out = run_cuda(bc)
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention
    out32 = ragged_page_attention(bc.queries.float(), bc.kv_pages.float(), bc.context_lens, bc.block_tables,
                                  bc.query_start_loc, bc.num_seqs, softmax_scale=bc.softmax_scale)
    assert out32.dtype == torch.float32 and torch.equal(out32, out.float())


def test_fp16(rpa_lib):
    b = make_ragged_batch([1, 2, 40], [500, 77, 300], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16,
                          seed=2, dtype=torch.float16)
    _check(b, "fp16")


def test_num_seqs_smaller_than_capacity_and_empty_sequences(rpa_lib):
    b = make_ragged_batch([1, 0, 3, 0, 1], [100, 50, 64, 0, 9], num_q_heads=8, num_kv_heads=2, head_dim=128,
                          page_size=16, max_num_seqs=9, pad_query_rows=5, seed=8)
    bc = b.to("cuda")
    out = run_cuda(bc)
    assert_parity(out, oracle(b), b.total_tokens, what="ragged/empty")
    assert torch.count_nonzero(out[b.total_tokens:]) == 0, "rows past the last sequence stay zero"
    # an int num_seqs is accepted like a (1,) array (_xla_impl_fwd.py:195)
    out2 = run_cuda(bc, )
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention
    out3 = ragged_page_attention(bc.queries, bc.kv_pages, bc.context_lens, bc.block_tables, bc.query_start_loc, 5,
                                 softmax_scale=bc.softmax_scale)
    assert torch.equal(out2, out3)


def test_zero_sequences(rpa_lib):
    b = make_ragged_batch([1, 1], [10, 10], num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=8, seed=1)
    bc = b.to("cuda")
    bc.num_seqs = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = run_cuda(bc)
    assert torch.count_nonzero(out) == 0


def test_page_gather_is_bit_exact(rpa_lib):
    """q = 0 makes the softmax uniform, V carries small integers that identify (page, slot, head,
    lane): the fp32 mean of integers below 2^11 over a power-of-two count is exact, so any wrong
    page, slot, head or mask boundary changes the result."""
    page, Hkv, G, D = 16, 2, 4, 128
    kv_lens = [64, 256, 1024, 16]
    b = make_ragged_batch([1] * 4, kv_lens, num_q_heads=Hkv * G, num_kv_heads=Hkv, head_dim=D, page_size=page, seed=77)
    b.queries.zero_()
    P = b.kv_pages.shape[0]
    g = torch.Generator().manual_seed(5)
    v = torch.randint(0, 256, (P, page, Hkv, D), generator=g).float()
    k = torch.randn(P, page, Hkv, D, generator=g)
    b.kv_pages = torch.stack([k, v], dim=3).reshape(P, page, 2 * Hkv, D).to(torch.bfloat16)
    out = run_cuda(b).float().cpu()
    want = oracle(b)
    want_bf16 = torch.from_numpy(want).to(torch.bfloat16).float()
    assert torch.equal(out, want_bf16)


def test_planted_keys_give_order_one_outputs(rpa_lib):
    """A few keys per sequence get a large score so the output is O(1) and dominated by specific
    (page, slot) entries; catches gather errors that N(0,1) averaging would hide."""
    b = make_ragged_batch([1, 1, 4], [4000, 900, 2500], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=31)
    q = b.queries.float()
    kv = b.kv_pages.float()
    tab = b.block_tables
    rng = np.random.default_rng(0)
    cu = b.query_start_loc.tolist()
    for s, kl in enumerate(b.meta["kv_lens"]):
        for j in rng.choice(kl - 4, size=3, replace=False):
            pg, sl = int(tab[s, j // 16]), int(j % 16)
            for h in range(2):
                kv[pg, sl, 2 * h] = q[cu[s], h * 4]
    b.kv_pages = kv.to(torch.bfloat16)
    r = _check(b, "planted")
    assert r["rms_want"] > 0.15


def test_deterministic_and_unaffected_by_poisoned_scratch(rpa_lib):
    """Two runs agree bitwise (the split-KV merge has no order dependence), and NaN in pool pages no
    sequence owns, in the tail slots of last pages and in the workspace does not leak into the output."""
    b = make_workload("c2", num_seqs=16, len_scale=0.5)
    bc = b.to("cuda")
    o1 = run_cuda(bc)
    used = torch.zeros(bc.kv_pages.shape[0], dtype=torch.bool, device="cuda")
    page = b.meta["page_size"]
    for s, kl in enumerate(b.meta["kv_lens"]):
        n = -(-kl // page)
        used[bc.block_tables[s, :n].long()] = True
        if kl % page:
            bc.kv_pages[bc.block_tables[s, n - 1].long(), kl % page:] = float("nan")
    bc.kv_pages[~used] = float("nan")
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import _workspace_cache
    for ws in _workspace_cache.values():
        ws.buffer.view(torch.float32)[: ws.nbytes // 4].fill_(float("nan"))
    o2 = run_cuda(bc)
    assert torch.equal(o1, o2)
    assert torch.isfinite(o2.float()).all()


def test_contract_violations_set_status_bits_and_never_fault(rpa_lib):
    from ejkernel_b200 import _cabi
    b = make_ragged_batch([1, 1, 1], [100, 50, 64], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=9)
    bc = b.to("cuda")
    bad = bc.to("cuda")
    bad.block_tables = bc.block_tables.clone()
    bad.block_tables[0, 1] = 10_000_000
    bad.block_tables[1, 0] = -3
    out = run_cuda(bad)
    assert status_word(bad) & _cabi.ST_PAGE_ID
    assert torch.isfinite(out.float()).all()
    bad = bc.to("cuda")
    bad.num_seqs = torch.tensor([50], dtype=torch.int32, device="cuda")
    run_cuda(bad)
    assert status_word(bad) & _cabi.ST_NUM_SEQS
    bad = bc.to("cuda")
    bad.context_lens = bc.context_lens.clone()
    bad.context_lens[2] = 1 << 20
    run_cuda(bad)
    assert status_word(bad) & _cabi.ST_KVLEN
    bad = bc.to("cuda")
    bad.query_start_loc = torch.tensor([0, 5, 2, 3], dtype=torch.int32, device="cuda")
    run_cuda(bad)
    assert status_word(bad) & _cabi.ST_QLEN
    # q_len > kv_len: rows at negative positions see nothing and come out as zeros
    b2 = make_ragged_batch([4], [4], num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=8, seed=1)
    b2c = b2.to("cuda")
    b2c.context_lens = torch.tensor([2], dtype=torch.int32, device="cuda")
    out = run_cuda(b2c)
    assert status_word(b2c) & _cabi.ST_QLEN
    assert torch.count_nonzero(out[:2]) == 0 and torch.isfinite(out.float()).all()


def test_host_errors(rpa_lib):
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention
    b = make_ragged_batch([1], [10], num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=8, seed=1).to("cuda")
    with pytest.raises(ValueError):
        ragged_page_attention(*b.args(), sliding_window=0)
    with pytest.raises(ValueError):
        ragged_page_attention(*b.args(), logits_soft_cap=0.0)
    with pytest.raises(ValueError):
        ragged_page_attention(b.queries, b.kv_pages, b.context_lens.long(), b.block_tables, b.query_start_loc, b.num_seqs)
    with pytest.raises(NotImplementedError):
        ragged_page_attention(b.queries.float(), b.kv_pages.float(), b.context_lens, b.block_tables, b.query_start_loc,
                              b.num_seqs, compute_dtype=torch.float32)
    with pytest.raises(NotImplementedError):
        ragged_page_attention(b.queries, b.kv_pages.float(), b.context_lens, b.block_tables, b.query_start_loc, b.num_seqs)
    with pytest.raises(Exception):  # rank mismatch is a type-check error, as in the reference
        ragged_page_attention(b.queries[0], b.kv_pages, b.context_lens, b.block_tables, b.query_start_loc, b.num_seqs)
    # shapes whose row or sequence counts do not fit the 32-bit work lists are refused on the host
    import ctypes

    from ejkernel_b200 import _cabi

    lib = _cabi.load()
    for shape in (_cabi.Shape(1 << 28, 4, 4, 16, 8, 8, 2, 64, _cabi.BF16, 0),   # 2^31 query rows
                  _cabi.Shape(8, 1 << 24, 4, 16, 8, 4, 2, 64, _cabi.BF16, 0)):  # 2^24 sequences
        assert lib.ejk_rpa_workspace_bytes(ctypes.byref(shape)) == 0
        rc = lib.ejk_rpa_launch(b.queries.data_ptr(), b.kv_pages.data_ptr(), b.context_lens.data_ptr(),
                                b.block_tables.data_ptr(), b.query_start_loc.data_ptr(), b.num_seqs.data_ptr(), None,
                                b.queries.data_ptr(), b.queries.data_ptr(), 1 << 20, None, ctypes.byref(shape),
                                ctypes.byref(_cabi.Attrs(1.0, 0.0, 0, 0, 0, 0, 0)), None)
        assert rc == -2 and lib.ejk_rpa_last_launch_count() == 0  # EJK_RPA_E_SHAPE, nothing enqueued


def test_enqueue_only_call_can_be_captured_in_a_cuda_graph(rpa_lib):
    """The C-ABI launch allocates nothing, never synchronises and never reads device memory from the
    host, so after one warm-up call (which sets per-device kernel attributes) the whole operator --
    planner, tensor-tile kernel, split-KV kernel, merge -- records into a CUDA graph.  Replaying the
    graph after changing the lengths in place must follow the new lengths: the work list is rebuilt on
    the device every time."""
    from ejkernel_b200.kernels._cuda.ragged_page_attention import RpaWorkspace, ragged_page_attention_into
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import _shape_of

    b = make_ragged_batch([1, 70, 1, 3], [900, 300, 64, 2000], num_q_heads=8, num_kv_heads=2, head_dim=128,
                          page_size=16, seed=81).to("cuda")
    ws = RpaWorkspace(_shape_of(b.queries, b.kv_pages, b.block_tables), b.queries.device)
    out = torch.zeros_like(b.queries)
    call = lambda: ragged_page_attention_into(out, ws, *b.args(), softmax_scale=b.softmax_scale)
    call()
    torch.cuda.synchronize()
    eager = out.clone()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            ragged_page_attention_into(out, ws, *b.args(), softmax_scale=b.softmax_scale, stream=side)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    # shorten every context in place and replay: the device planner must pick the new lengths up
    new_lens = [500, 200, 10, 1200]
    b.context_lens.copy_(torch.tensor(new_lens, dtype=torch.int32))
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    b.meta["kv_lens"] = new_lens
    assert_parity(out, oracle(b), b.total_tokens, what="graph replay with new lengths")
    assert int(ws.status.item()) == 0


def test_public_module_entry(rpa_lib):
    import ejkernel_b200 as ej
    b = make_workload("c1")
    bc = b.to("cuda")
    out = ej.ragged_page_attention(bc.queries, bc.kv_pages, bc.context_lens, bc.block_tables, bc.query_start_loc,
                                   bc.num_seqs, softmax_scale=bc.softmax_scale, platform="cuda")
    torch.cuda.synchronize()
    assert_parity(out, oracle(b), b.total_tokens, what="modules entry")
    with pytest.raises(ValueError):
        ej.ragged_page_attention(bc.queries, bc.kv_pages, bc.context_lens, bc.block_tables, bc.query_start_loc,
                                 bc.num_seqs, platform="xla")


def test_a_reader_enqueued_right_after_a_mixed_call_sees_the_prefill_rows(rpa_lib):
    """In a mixed batch the split-KV kernel is a programmatic dependent of the prefill-tile kernel and does
    not wait for it while it works; before it completes, one thread per CTA waits for the prefill grid, so a
    kernel enqueued behind the call with no host synchronisation in between (here a copy of ``out``) is
    ordered after BOTH kernels.  One long prefill sequence beside a one-token decode is the shape in which
    the split-KV kernel would otherwise finish long before the prefill kernel."""
    from ejkernel_b200.kernels._cuda.ragged_page_attention import RpaWorkspace, ragged_page_attention_into
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import _shape_of

    b = make_ragged_batch([1, 1024], [40, 6000], num_q_heads=16, num_kv_heads=4, head_dim=128, page_size=16, seed=91)
    want = oracle(b)
    bc = b.to("cuda")
    ws = RpaWorkspace(_shape_of(bc.queries, bc.kv_pages, bc.block_tables), bc.queries.device)
    out = torch.empty_like(bc.queries)
    copies = []
    for rep in range(20):
        out.fill_(float("nan"))
        ragged_page_attention_into(out, ws, *bc.args(), softmax_scale=bc.softmax_scale)
        copies.append(out.clone())  # enqueued on the same stream, no host sync since the launch
    torch.cuda.synchronize()
    assert int(ws.status.item()) == 0
    # per sequence: the tight criterion scales with the rms of the expected rows, and a 40-key row is ten times
    # larger than rows that average 6000 keys
    assert_parity(out[:1], want[:1], 1, what="mixed batch, decode row")
    assert_parity(out[1:], want[1:], b.total_tokens - 1, what="mixed batch, prefill rows")
    for c in copies:
        assert torch.equal(c, out), "a copy enqueued right behind the call missed rows of the prefill kernel"


def test_operator_workspace_is_bounded_and_per_stream(rpa_lib):
    """The public operator owns its scratch: one buffer per (device, stream) that grows to the largest need, so
    a serving loop with a different token count every step does not allocate one workspace per shape, and two
    streams running calls of the same shape at the same time do not share scratch."""
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention
    from ejkernel_b200.kernels._cuda.ragged_page_attention import _interface as itf

    torch.cuda.synchronize()
    itf._workspace_cache.clear()
    rng = np.random.default_rng(3)
    outs = {}
    for T in range(1, 201):  # 200 distinct shapes
        kv = [int(x) for x in rng.integers(1, 400, 2)]
        b = make_ragged_batch([1, T - 1] if T > 1 else [1, 0], [kv[0], kv[1] + T], num_q_heads=8, num_kv_heads=2,
                              head_dim=64, page_size=16, pages_per_seq=40, num_pages=90, max_num_seqs=2, seed=T).to("cuda")
        o = ragged_page_attention(*b.args(), softmax_scale=b.softmax_scale)
        if T in (1, 57, 200):
            outs[T] = (b, o)
    torch.cuda.synchronize()
    assert len(itf._workspace_cache) == 1
    (ws,) = itf._workspace_cache.values()
    b200 = outs[200][0]
    assert ws.nbytes < 4 * itf.workspace_bytes(itf._shape_of(b200.queries, b200.kv_pages, b200.block_tables), b200.queries.device)
    for T, (b, o) in outs.items():
        assert_parity(o, oracle(b), b.total_tokens, what=f"T={T}")

    # two streams, same shape, overlapping in time: each result equals the single-stream result bit for bit
    ba = make_workload("c2", num_seqs=48, len_scale=0.5, device="cuda")
    bb = make_workload("c2", num_seqs=48, len_scale=0.5, device="cuda", seed=77)
    ra = ragged_page_attention(*ba.args(), softmax_scale=ba.softmax_scale)
    rb = ragged_page_attention(*bb.args(), softmax_scale=bb.softmax_scale)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    got = []
    for _ in range(10):
        with torch.cuda.stream(s1):
            oa = ragged_page_attention(*ba.args(), softmax_scale=ba.softmax_scale)
        with torch.cuda.stream(s2):
            ob = ragged_page_attention(*bb.args(), softmax_scale=bb.softmax_scale)
        got.append((oa, ob))
    torch.cuda.synchronize()
    assert len(itf._workspace_cache) == 3
    for oa, ob in got:
        assert torch.equal(oa, ra) and torch.equal(ob, rb)


def test_rows_past_the_last_sequence_are_zero_filled_by_the_launch(rpa_lib):
    """``out`` needs no initialisation: like the reference, whose result starts as zeros, the launch writes
    zeros to every row past the last sequence (a padded token axis is the normal case under a tracing runtime)."""
    from ejkernel_b200.kernels._cuda.ragged_page_attention import RpaWorkspace, ragged_page_attention_into
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import _shape_of

    for q_lens, kv_lens, pad in (([1, 1, 1], [70, 9, 300], 61), ([40, 1], [100, 5], 300), ([1], [10], 0)):
        b = make_ragged_batch(q_lens, kv_lens, num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16,
                              pad_query_rows=pad, max_num_seqs=5, seed=pad).to("cuda")
        ws = RpaWorkspace(_shape_of(b.queries, b.kv_pages, b.block_tables), b.queries.device)
        for path in (0, 1):  # TMA gather and cp.async gather
            from ejkernel_b200 import _cabi
            _cabi.set_option("path", path)
            try:
                out = torch.full_like(b.queries, float("nan"))
                ragged_page_attention_into(out, ws, *b.args(), softmax_scale=b.softmax_scale)
                torch.cuda.synchronize()
            finally:
                _cabi.set_option("path", 0)
            T = b.total_tokens
            assert torch.isfinite(out.float()).all()
            assert torch.count_nonzero(out[T:]) == 0
            assert_parity(out, oracle(b), T, what="padded batch")
    # no sequence at all: everything is zero
    b.num_seqs = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full_like(b.queries, float("nan"))
    ragged_page_attention_into(out, ws, *b.args(), softmax_scale=b.softmax_scale)
    torch.cuda.synchronize()
    assert torch.count_nonzero(out) == 0


def test_tile_kernel_hands_sms_to_the_split_kv_kernel_in_mixed_batches(rpa_lib):
    """In a mixed batch the tensor-tile kernel keeps only as many CTAs as its estimate of the two kernels' times
    asks for (option ``prefill_share``, a percentage on that estimate) and the rest exit at once; whatever the
    share -- none, far too few CTAs, the default, far too many -- every item is still served exactly once."""
    from ejkernel_b200 import _cabi
    b = make_workload("c3", num_seqs=20, len_scale=0.25)  # 16 decode sequences + 4 prefill chunks
    want = oracle(b)
    bc = b.to("cuda")
    old = _cabi.get_option("prefill_share"), _cabi.get_option("prefill_split")
    try:
        for split in (1, 0):
            _cabi.set_option("prefill_split", split)
            outs = []
            for share in (0, 10, 120, 1000):
                _cabi.set_option("prefill_share", share)
                out = run_cuda(bc)
                assert status_word(bc) == 0
                assert_parity(out, want, b.total_tokens, what=f"prefill_share {share}, split {split}")
                outs.append(out)
            if split == 0:  # whole items: which CTA serves an item does not change its arithmetic
                assert all(torch.equal(o, outs[0]) for o in outs)
    finally:
        _cabi.set_option("prefill_share", old[0])
        _cabi.set_option("prefill_split", old[1])


def test_opt_in_status_check_raises_when_outputs_are_invalid(rpa_lib, monkeypatch):
    """``EJKERNEL_B200_CHECK_STATUS=1`` makes the operator read its status word after every call and raise when it says
    the outputs are invalid.  A wait is made to run out with the test hook (nothing faults or hangs); the call after it,
    with the hook off, is clean again."""
    from ejkernel_b200 import _cabi
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention
    b = make_ragged_batch([1, 1, 2], [700, 64, 1500], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=97).to("cuda")
    monkeypatch.setenv("EJKERNEL_B200_CHECK_STATUS", "1")
    old = _cabi.get_option("wait_ms")
    try:
        _cabi.set_option("wait_ms", 50)
        _cabi.set_option("test_withhold", 1)
        with pytest.raises(_cabi.RpaLibraryError, match="wait inside a kernel ran out"):
            ragged_page_attention(*b.args(), softmax_scale=b.softmax_scale)
    finally:
        _cabi.set_option("test_withhold", 0)
        _cabi.set_option("wait_ms", old)
    out = ragged_page_attention(*b.args(), softmax_scale=b.softmax_scale)  # raises nothing
    assert_parity(out, oracle(b), b.total_tokens, what="after a timed-out call")


def test_queries_and_output_in_pinned_host_memory(rpa_lib):
    """Page-locked host memory is mapped into the device's address space: the kernels can read the query rows from it
    and write the output rows to it, bit for bit what they do with device buffers (mixed batch: split-KV tiles, tensor
    tiles and the zero-filled padding rows all store to the host buffer)."""
    from ejkernel_b200.kernels._cuda.ragged_page_attention import RpaWorkspace, ragged_page_attention_into
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import _shape_of

    b = make_ragged_batch([1, 1, 200, 3, 1], [5000, 64, 900, 77, 2500], num_q_heads=16, num_kv_heads=4, head_dim=128,
                          page_size=16, seed=97, pad_query_rows=5)
    bc = b.to("cuda")
    ws = RpaWorkspace(_shape_of(bc.queries, bc.kv_pages, bc.block_tables), bc.queries.device)
    dev_out = torch.full_like(bc.queries, float("nan"))
    ragged_page_attention_into(dev_out, ws, *bc.args(), softmax_scale=b.softmax_scale)
    host_q = b.queries.clone().pin_memory()
    host_out = torch.full(b.queries.shape, float("nan"), dtype=b.queries.dtype).pin_memory()
    ragged_page_attention_into(host_out, ws, host_q, *bc.args()[1:], softmax_scale=b.softmax_scale)
    torch.cuda.synchronize()
    assert int(ws.status.item()) == 0
    assert torch.equal(host_out, dev_out.cpu())
    assert_parity(host_out, oracle(b), b.total_tokens, what="pinned host queries and output")
    assert torch.count_nonzero(host_out[b.total_tokens:]) == 0
