"""Pins the CPU oracle without a GPU: its two restatements (which follow two independent
reference sources) agree, analytically known answers come out, the committed golden fixtures are
reproduced, and the as-written mode shows the reference's documented artefacts."""

from pathlib import Path

import numpy as np
import pytest
import torch

from ejkernel_b200.utils import algorithmic_kv_bytes, make_ragged_batch, make_workload, visible_kv_tokens
from oracle.rpa_oracle import blocked_as_written, compare, dense_reference
from tests.golden.make_golden import cases, input_checksum

GOLDEN = np.load(Path(__file__).parent / "golden" / "rpa_golden.npz")


@pytest.mark.parametrize("name,batch", list(cases()), ids=[n for n, _ in cases()])
def test_golden_fixtures(name, batch):
    np.testing.assert_allclose(input_checksum(batch), GOLDEN[f"{name}.chk"], rtol=1e-12, err_msg="input generator drifted")
    got = dense_reference(*batch.args(), **batch.kwargs())
    np.testing.assert_allclose(got, GOLDEN[f"{name}.out"], rtol=0, atol=1e-6)


@pytest.mark.parametrize(
    "q_lens,kv_lens,kw",
    [
        ([1] * 8, [16, 100, 512, 33, 64, 65, 300, 17], {}),
        ([100, 50, 40, 10], [128, 64, 192, 96], {}),
        ([1, 4, 1], [700, 350, 20], dict(logits_soft_cap=30.0)),
        ([1, 3, 1], [300, 64, 200], dict(sliding_window=50, logits_soft_cap=30.0)),
    ],
)
def test_two_restatements_agree(q_lens, kv_lens, kw):
    # 16 pad rows keep the as-written 8-row blocks inside the query array (see the artefact test)
    b = make_ragged_batch(q_lens, kv_lens, num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16,
                          pad_query_rows=16, seed=len(q_lens), **kw)
    d = dense_reference(*b.args(), **b.kwargs())
    w = blocked_as_written(*b.args(), **b.kwargs())
    r = compare(w, d, rows=b.total_tokens)
    assert r["finite"] and r["allclose"] and r["max_rel_rms"] < 0.1, r


def test_sinks_agree_between_restatements():
    b = make_ragged_batch([1, 5], [300, 70], num_q_heads=8, num_kv_heads=2, head_dim=64, page_size=16,
                          pad_query_rows=16, seed=5)
    for aux in (torch.tensor([[0.3, -2.0], [1.0, 0.2]]), torch.linspace(-1, 1, 8).reshape(8, 1), torch.tensor([0.7])):
        b.softmax_aux = aux
        d = dense_reference(*b.args(), **b.kwargs())
        w = blocked_as_written(*b.args(), **b.kwargs(), compute_dtype=torch.float32)
        assert compare(w, d, rows=b.total_tokens)["max_abs"] < 2e-2


def test_uniform_softmax_known_answer():
    """q = 0 -> every visible key has weight 1/n, so the output is the plain mean of the visible V rows."""
    b = make_ragged_batch([1, 3], [40, 21], num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=8, seed=2,
                          sliding_window=10)
    b.queries.zero_()
    out = dense_reference(*b.args(), **b.kwargs())
    kv = b.kv_pages.float().numpy()
    for s, (ql, kl) in enumerate(zip([1, 3], [40, 21])):
        for r in range(ql):
            pos = kl - ql + r
            keys = [j for j in range(kl) if j <= pos and j > pos - 10]
            rows = np.stack([kv[int(b.block_tables[s, j // 8]), j % 8] for j in keys])  # [n, 2Hkv, D]
            for hq in range(4):
                want = rows[:, 2 * (hq // 2) + 1, :].astype(np.float64).mean(0)
                np.testing.assert_allclose(out[int(b.query_start_loc[s]) + r, hq], want, atol=1e-12)


def test_single_visible_key_returns_its_value():
    b = make_ragged_batch([1], [50], num_q_heads=2, num_kv_heads=1, head_dim=64, page_size=16, seed=3, sliding_window=1)
    out = dense_reference(*b.args(), **b.kwargs())
    v_last = b.kv_pages[int(b.block_tables[0, 49 // 16]), 49 % 16, 1].double().numpy()
    np.testing.assert_allclose(out[0, 0], v_last, atol=1e-12)
    np.testing.assert_allclose(out[0, 1], v_last, atol=1e-12)


def test_as_written_artefacts_of_the_reference():
    """The XLA implementation as written misplaces rows when the last 8-row query block would run
    past the padded token count (dynamic_slice clamps its start, _xla_impl_fwd.py:88-92,181-185), and
    returns NaN when a whole leading 64-page KV block lies outside the sliding window
    (exp(-inf - -inf), :140-147).  The restatement reproduces both; the dense mode is unaffected."""
    b = make_workload("c1")  # T = 8 with no padding rows
    d = dense_reference(*b.args(), **b.kwargs())
    w = blocked_as_written(*b.args(), **b.kwargs())
    assert not compare(w, d)["allclose"]
    bp = make_workload("c1", pad_query_rows=16)
    assert compare(blocked_as_written(*bp.args(), **bp.kwargs()), dense_reference(*bp.args(), **bp.kwargs()), rows=8)["allclose"]
    bw = make_ragged_batch([1], [64 * 16 * 2 + 5], num_q_heads=2, num_kv_heads=1, head_dim=64, page_size=16,
                           pages_per_seq=192, pad_query_rows=16, seed=4, sliding_window=64)
    w = blocked_as_written(*bw.args(), **bw.kwargs())
    assert torch.isnan(w[0].float()).all()
    assert np.isfinite(dense_reference(*bw.args(), **bw.kwargs())).all()


def test_algorithmic_bytes():
    assert visible_kv_tokens([1, 1], [100, 5000], None) == 5100
    assert visible_kv_tokens([1, 1], [100, 5000], 4096) == 100 + 4096
    assert visible_kv_tokens([4], [10], 3) == 6  # rows at 6..9 see keys 4..9
    b = make_workload("c1")
    assert algorithmic_kv_bytes(b) == sum(b.meta["kv_lens"]) * 2 * 2 * 128 * 2


def test_workload_generators_are_seeded_and_shaped():
    a, b = make_workload("c1"), make_workload("c1")
    assert torch.equal(a.kv_pages, b.kv_pages) and torch.equal(a.block_tables, b.block_tables)
    assert a.kv_pages.shape == (256, 16, 4, 128) and a.block_tables.shape == (8, 32)
    used = torch.cat([a.block_tables[s, : -(-k // 16)] for s, k in enumerate(a.meta["kv_lens"])])
    assert used.unique().numel() == used.numel(), "pages are not shared between sequences"
    c4 = make_workload("c4", num_seqs=3, len_scale=0.05)
    assert c4.sliding_window is not None and c4.logits_soft_cap == 50.0 and c4.kv_pages.shape[1:] == (32, 16, 256)
