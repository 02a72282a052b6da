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
    assert k0 == call_key(q[:5], kv, tab)  # 6 and 5 query tokens round up to the same power of two: one signature ...
    assert k0 != call_key(q[:4], kv, tab) and k0 != call_key(q, kv[:8], tab)  # ... 4 tokens, or half the pool, do not
    assert k0 != call_key(q[:, :4], kv, tab)  # every other dimension counts exactly
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


def test_selection_chain_order_and_events(tmp_path):
    """override > overlay > memory cache > persistent cache > autotune > heuristic, as in the reference's
    ConfigSelectorChain.choose (ejkernel/ops/config/selection.py:384-566), with its events."""
    from ejkernel_b200.modules.operations.tuning import AutotunePolicy, ConfigSelectorChain, overlay_cache

    events = []
    pers = PersistentCache("op", str(tmp_path / "p.json"))
    chain = ConfigSelectorChain(persistent=pers, on_event=lambda ev, **d: events.append((ev, d.get("level"))))
    key = ("dev", "op@v0", "k1")
    tuned = {"n": 0}

    def autotune():
        tuned["n"] += 1
        return "tuned"

    assert chain.choose(*key, autotune=autotune, heuristic=lambda: "heur") == "tuned"  # nothing cached: measure once
    assert chain.choose(*key, autotune=autotune, heuristic=lambda: "heur") == "tuned" and tuned["n"] == 1  # memory tier
    assert pers.get(*key) == "tuned"  # and persisted
    with overlay_cache({key: "overlaid"}):
        assert chain.choose(*key, autotune=autotune, heuristic=lambda: "heur") == "overlaid"
        assert chain.choose(*key, override="explicit") == "explicit"  # an explicit cfg beats the overlay ...
    assert chain.choose(*key, autotune=autotune) == "explicit"  # ... and is remembered, as in the reference
    fresh = ConfigSelectorChain(persistent=PersistentCache("op", str(tmp_path / "p.json")),
                                on_event=lambda ev, **d: events.append((ev, d.get("level"))))
    assert fresh.choose(*key, autotune=autotune) == "explicit" and tuned["n"] == 1  # persistent tier of a new process
    assert [e for e, _ in events] == ["autotune_start", "autotune_finish", "cache_hit", "overlay_hit", "override", "cache_hit",
                                      "cache_hit"]
    assert events[2][1] == "memory" and events[-1][1] == "persistent"
    # policy "heuristics": no measuring; a call that may not measure right now takes the heuristic without caching it
    h = ConfigSelectorChain(policy=AutotunePolicy(allow_autotune=False, cache_miss_fallback="heuristics"))
    assert h.choose("d", "o", "k", autotune=autotune, heuristic=lambda: "heur") == "heur" and tuned["n"] == 1
    a = ConfigSelectorChain()
    assert a.choose("d", "o", "k", autotune=autotune, heuristic=lambda: "heur", may_autotune=False) == "heur"
    assert a.choose("d", "o", "k", autotune=autotune, heuristic=lambda: "heur") == "tuned" and tuned["n"] == 2
    with pytest.raises(RuntimeError):
        ConfigSelectorChain(policy=AutotunePolicy(allow_autotune=False, allow_heuristics=False,
                                                  cache_miss_fallback="heuristics")).choose("d", "o", "k")


def test_policy_from_env_and_stamp_label(monkeypatch):
    from ejkernel_b200.modules.operations.tuning import AutotunePolicy

    monkeypatch.setenv("EJKERNEL_AUTOTUNE_POLICY", "heuristics")
    p = AutotunePolicy.from_env()
    assert not p.allow_autotune and p.cache_miss_fallback == "heuristics"
    monkeypatch.setenv("EJKERNEL_AUTOTUNE_POLICY", "nonsense")
    with pytest.raises(ValueError):
        AutotunePolicy.from_env()
    monkeypatch.delenv("EJKERNEL_AUTOTUNE_POLICY")
    assert AutotunePolicy.from_env().cache_miss_fallback == "autotune"  # the reference's default
    q, kv, lens, tab, qsl, n = _operands()
    label = rpa_module.stamp_label(q, kv, tab, None, RaggedPageAttention().heuristic_cfg())
    assert label == f"ejkernel_ops#ragged_page_attention@v0:{call_key(q, kv, tab)}"
    js = rpa_module.stamp_label(q, kv, tab, None, RaggedPageAttention().heuristic_cfg(), mode="json")
    assert js.startswith("ejkernel_ops:{") and json.loads(js.split(":", 1)[1])["op_id"] == "ragged_page_attention@v0"


def test_operator_resolves_a_signature_once(monkeypatch):
    """The first call of a static signature walks the chain (here: a fake measurement), later calls take the
    dictionary look-up; a pick that does not beat the heuristic by 2 % keeps the heuristic."""
    q, kv, lens, tab, qsl, n = _operands()
    kern = RaggedPageAttention()
    monkeypatch.setattr(RaggedPageAttention, "run", lambda self, *a, cfg, **kw: cfg)
    calls = {"n": 0}

    def fake_autotune(*a, **kw):
        calls["n"] += 1
        return RaggedPageAttentionConfig(num_kv_pages_per_block=2, platform="cuda", backend="gpu")

    monkeypatch.setattr(kern, "autotune", fake_autotune)
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    monkeypatch.setattr(rpa_module, "device_fingerprint", lambda d=None: "cuda|fake|sm100|148")
    c1, k1 = kern.select_cfg(q, kv, lens, tab, qsl, n)
    c2, k2 = kern.select_cfg(q, kv, lens, tab, qsl, n)
    assert c1.num_kv_pages_per_block == 2 and c2 is c1 and calls["n"] == 1 and k1 is not None and k2 is None
    monkeypatch.undo()
    slow = {"heur": 1.0, "other": 0.99}
    best, _ = pick_best(["heur", "other"], lambda c: (lambda: c), timer=lambda fn: slow[fn()], margin=0.02)
    assert best == "heur"
