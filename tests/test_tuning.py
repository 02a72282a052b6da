"""Tuning persistence of the ops layer (host logic; no GPU needed)."""

import json

import pytest
import torch

from ejkernel_b200.modules.operations import RaggedPageAttention, RaggedPageAttentionConfig
import importlib

rpa_module = importlib.import_module("ejkernel_b200.modules.operations.ragged_page_attention")
from ejkernel_b200.modules.operations.tuning import PersistentCache, call_key, device_fingerprint, pick_best


def _operands(T=6, S=3, pages_per_seq=4, P=16, page=16, hq=8, hkv=2, d=128):
    q = torch.zeros(T, hq, d, dtype=torch.bfloat16)
    kv = torch.zeros(P, page, 2 * hkv, d, dtype=torch.bfloat16)
    lens = torch.ones(S, dtype=torch.int32)
    tab = torch.zeros(S, pages_per_seq, dtype=torch.int32)
    qsl = torch.arange(S + 1, dtype=torch.int32)
    return q, kv, lens, tab, qsl, torch.tensor([S], dtype=torch.int32)


def test_persistent_cache_round_trip_and_key_format(tmp_path):
    path = tmp_path / "sub" / "rpa.json"
    cache = PersistentCache("ragged_page_attention", str(path), cfg_type=RaggedPageAttentionConfig)
    assert cache.get("cuda|X|sm100|148", "ragged_page_attention@v0", "abc") is None
    cfg = RaggedPageAttentionConfig(num_kv_pages_per_block=32, num_queries_per_block=None, platform="cuda", backend="gpu")
    cache.put("cuda|X|sm100|148", "ragged_page_attention@v0", "abc", cfg)
    stored = json.loads(path.read_text())
    assert list(stored) == ["cuda|X|sm100|148|ragged_page_attention@v0|abc"]  # device|op@v|call_key
    assert stored["cuda|X|sm100|148|ragged_page_attention@v0|abc"]["num_kv_pages_per_block"] == 32
    again = PersistentCache("ragged_page_attention", str(path), cfg_type=RaggedPageAttentionConfig)
    assert again.get("cuda|X|sm100|148", "ragged_page_attention@v0", "abc") == cfg
    assert again.get("cuda|Y|sm100|148", "ragged_page_attention@v0", "abc") is None
    # a second entry keeps the first; no temporary files are left behind
    again.put("cuda|X|sm100|148", "ragged_page_attention@v0", "def", cfg)
    assert len(PersistentCache("ragged_page_attention", str(path))) == 2
    assert [f.name for f in path.parent.iterdir()] == ["rpa.json"]


def test_call_key_depends_on_static_facts_only():
    q, kv, lens, tab, _, _ = _operands()
    k0 = call_key(q, kv, tab)
    assert k0 == call_key(q.clone(), kv.clone(), tab + 3)  # values do not matter
    assert k0 != call_key(q[:5], kv, tab)
    assert k0 != call_key(q, kv, tab, sliding_window=128)
    assert k0 != call_key(q, kv, tab, logits_soft_cap=30.0)
    assert k0 != call_key(q.half(), kv.half(), tab)
    assert device_fingerprint("cpu").startswith("cpu|")


def test_pick_best_takes_the_fastest_and_skips_failing_candidates():
    times = {"a": 3.0, "b": 1.0, "c": 1.0, "bad": 0.1}

    def run_with(c):
        if c == "bad":
            raise ValueError("shape not admitted")
        return lambda: c

    best, ts = pick_best(["a", "bad", "b", "c"], run_with, timer=lambda fn: times[fn()])
    assert best == "b" and ts == [3.0, float("inf"), 1.0, 1.0]
    with pytest.raises(RuntimeError):
        pick_best(["bad"], run_with, timer=lambda fn: 0.0)


def test_autotune_persists_and_the_operator_picks_it_up(tmp_path, monkeypatch):
    q, kv, lens, tab, qsl, n = _operands()
    cache = PersistentCache("ragged_page_attention", str(tmp_path / "c.json"), cfg_type=RaggedPageAttentionConfig)
    kern = RaggedPageAttention(cache=cache)
    seen = []

    def fake_run(self, *args, cfg, **kw):
        seen.append(cfg)
        return cfg

    monkeypatch.setattr(RaggedPageAttention, "run", fake_run)
    # candidates whose KV-chunk floor exceeds the 4 pages a sequence can have are dropped before measuring
    cands = kern.candidate_cfgs(page_size=16)
    assert cands[0] == kern.heuristic_cfg() and len(cands) == 7
    cost = lambda cfg: 5.0 if cfg.num_queries_per_block == 4 else 9.0  # noqa: E731
    best = kern.autotune(q, kv, lens, tab, qsl, n, timer=lambda fn: cost(fn()))
    assert best.num_queries_per_block == 4
    assert all(c.num_kv_pages_per_block is None or c.num_kv_pages_per_block <= 4 for c in seen)
    # a fresh kernel object with the same file finds it for this signature and falls back otherwise
    kern2 = RaggedPageAttention(cache=PersistentCache("ragged_page_attention", str(tmp_path / "c.json"),
                                                      cfg_type=RaggedPageAttentionConfig))
    assert kern2.lookup_cfg(q, kv, tab) == best
    assert kern2.lookup_cfg(q, kv, tab, sliding_window=7) == kern2.heuristic_cfg()
    # the module-level operator consults its kernel object's cache when no cfg is given
    monkeypatch.setattr(rpa_module, "_kernel", kern2)
    seen.clear()
    rpa_module.ragged_page_attention(q, kv, lens, tab, qsl, n)
    assert seen == [best]
    explicit = RaggedPageAttentionConfig(num_kv_pages_per_block=2, platform="cuda", backend="gpu")
    rpa_module.ragged_page_attention(q, kv, lens, tab, qsl, n, cfg=explicit)
    assert seen[-1] == explicit
