"""Tuning persistence for the CUDA operators: the two tile hints the kernels honour, measured per
(device, operator version, call signature) and kept in a JSON file across runs.

Mirrors the part of the reference's ops layer that EasyDeL-style callers rely on -- the
``PersistentCache`` of ejkernel/ops/config/persistent.py:58-200 with its ``device|op@v|call_key``
keys (:114-125) and atomic file replacement (:190-200), the measure-candidates-keep-the-best
step of ``Tuner`` (ejkernel/ops/config/selection.py:226-245), and the selection order of
``ConfigSelectorChain.choose`` (:384-566): explicit override, overlay, in-memory cache, persistent
cache, autotune on the first call of a signature, heuristic.  There is one implementation here and two
knobs, so the chain selects a configuration, never a backend.

What is tuned: ``RaggedPageAttentionConfig.num_kv_pages_per_block`` (smallest KV chunk a row tile is
split into, in pages) and ``num_queries_per_block`` (query tokens from which on a sequence is served
by 128-row tensor tiles).  ``None`` leaves the library's defaults in force.
"""

from __future__ import annotations

import hashlib
import json
import os
import pathlib
import tempfile
import contextlib
from collections.abc import Callable, Sequence
from dataclasses import asdict, dataclass, is_dataclass
from typing import Any

import torch


class PersistentCache:
    """JSON file of ``{"device|op@v|call_key": cfg}``; every ``put`` rewrites it atomically."""

    def __init__(self, opname: str, path: str | None = None, loader: Callable[[Any], Any] | None = None,
                 dumper: Callable[[Any], Any] | None = None, cfg_type: type | None = None):
        if path is None:
            path = str(pathlib.Path.home() / "ejkernel-b200-persistent-cache" / f"{opname}.json")
        pathlib.Path(os.path.dirname(os.path.abspath(path)) or ".").mkdir(parents=True, exist_ok=True)
        self.path = path
        self.loader = loader
        self.dumper = dumper
        self.cfg_type = cfg_type
        try:
            with open(path) as f:
                self._data = json.load(f)
        except FileNotFoundError:
            self._data = {}

    @staticmethod
    def _key(device: str, op_id: str, call_key: str) -> str:
        return "|".join((device, op_id, call_key))

    def get(self, device: str, op_id: str, call_key: str):
        raw = self._data.get(self._key(device, op_id, call_key))
        if raw is None:
            return None
        if self.loader is not None:
            return self.loader(raw)
        if isinstance(raw, dict) and self.cfg_type is not None:
            return self.cfg_type(**raw)
        return raw

    def put(self, device: str, op_id: str, call_key: str, cfg) -> None:
        if self.dumper is not None:
            val = self.dumper(cfg)
        elif is_dataclass(cfg):
            val = asdict(cfg)
        else:
            val = cfg
        self._data[self._key(device, op_id, call_key)] = val
        directory = os.path.dirname(os.path.abspath(self.path)) or "."
        with tempfile.NamedTemporaryFile("w", dir=directory, delete=False) as tmp:
            json.dump(self._data, tmp)
            tmp_path = tmp.name
        os.replace(tmp_path, self.path)

    def __len__(self) -> int:
        return len(self._data)


def device_fingerprint(device: torch.device | str | None = None) -> str:
    """``cuda|<name>|sm<cc>|<SMs>``: what a tuned split size depends on."""
    dev = torch.device(device) if device is not None else torch.device("cuda")
    if dev.type != "cuda" or not torch.cuda.is_available():
        return f"{dev.type}|unknown"
    props = torch.cuda.get_device_properties(dev)
    return f"cuda|{props.name}|sm{props.major}{props.minor}|{props.multi_processor_count}"


def call_key(queries: torch.Tensor, kv_pages: torch.Tensor, block_tables: torch.Tensor, *,
             sliding_window: int | None = None, logits_soft_cap: float | None = None,
             softmax_aux: torch.Tensor | None = None) -> str:
    """Hash of everything static about a call: operand shapes and dtypes and the static keywords.
    The lengths are data and are not part of it (the device planner adapts to them)."""
    # The token count and the pool size change from step to step in a serving loop, and the two tuned hints depend on
    # them only weakly: both enter rounded up to a power of two, so that a loop with ragged batches resolves (and, under
    # the autotune policy, measures) a handful of signatures instead of one per step.
    up = lambda n: 1 << max(0, int(n) - 1).bit_length()
    q_shape = (up(queries.shape[0]), *queries.shape[1:])
    kv_shape = (up(kv_pages.shape[0]), *kv_pages.shape[1:])
    sig = {
        "queries": (tuple(q_shape), str(queries.dtype)),
        "kv_pages": (tuple(kv_shape), str(kv_pages.dtype)),
        "block_tables": tuple(block_tables.shape),
        "sliding_window": None if sliding_window is None else int(sliding_window),
        "logits_soft_cap": None if logits_soft_cap is None else float(logits_soft_cap),
        "softmax_aux": None if softmax_aux is None else tuple(softmax_aux.shape),
    }
    return hashlib.sha1(json.dumps(sig, sort_keys=True).encode()).hexdigest()[:16]


def cuda_event_timer(fn: Callable[[], Any], warmup: int = 3, iters: int = 10) -> float:
    """Mean device milliseconds of ``fn`` on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def pick_best(candidates: Sequence[Any], run_with: Callable[[Any], Callable[[], Any]],
              timer: Callable[[Callable[[], Any]], float] = cuda_event_timer, margin: float = 0.0) -> tuple[Any, list[float]]:
    """Time ``run_with(cfg)`` for every candidate; the first of the fastest wins.  A candidate that
    raises is skipped (its time is ``inf``).  With ``margin`` > 0 the first candidate (the heuristic) is kept
    unless another one is faster by more than that fraction: timing noise must not replace the default."""
    times: list[float] = []
    for cfg in candidates:
        try:
            times.append(float(timer(run_with(cfg))))
        except Exception:  # a candidate the shapes do not admit
            times.append(float("inf"))
    if not times or min(times) == float("inf"):
        raise RuntimeError("no candidate configuration could be run")
    best = times.index(min(times))
    if margin > 0.0 and times[0] != float("inf") and times[best] >= times[0] * (1.0 - margin):
        best = 0
    return candidates[best], times


# ----------------------------------------------------------------------------------------------------------
# Selection chain (reference: ejkernel/ops/config/selection.py:82-578, cache.py:44-175)
# ----------------------------------------------------------------------------------------------------------
class ConfigCache:
    """In-memory ``(device, op@v, call_key) -> cfg`` (reference: ejkernel/ops/config/cache.py:44-110)."""

    def __init__(self):
        self._data: dict[tuple[str, str, str], Any] = {}

    def get(self, device: str, op_id: str, call_key: str):
        return self._data.get((device, op_id, call_key))

    def put(self, device: str, op_id: str, call_key: str, cfg) -> None:
        self._data[(device, op_id, call_key)] = cfg

    def clear(self) -> None:
        self._data.clear()

    def __len__(self) -> int:
        return len(self._data)


_overlays: list[dict[tuple[str, str, str], Any]] = []


@contextlib.contextmanager
def overlay_cache(mapping: dict[tuple[str, str, str], Any]):
    """Temporary ``(device, op@v, call_key) -> cfg`` overrides that win over both caches while the context is
    active; nested overlays are searched innermost first (reference: cache.py:113-175)."""
    _overlays.append(dict(mapping))
    try:
        yield
    finally:
        _overlays.pop()


@dataclass
class AutotunePolicy:
    """What a cache miss may do (reference: selection.py:82-110)."""

    allow_autotune: bool = True
    allow_heuristics: bool = True
    cache_miss_fallback: str = "autotune"  # "autotune" | "heuristics"

    @staticmethod
    def from_env(default: str = "autotune") -> "AutotunePolicy":
        """``EJKERNEL_AUTOTUNE_POLICY=autotune|heuristics``, the reference's switch
        (ejkernel/modules/operations/ragged_page_attention.py:531)."""
        mode = os.environ.get("EJKERNEL_AUTOTUNE_POLICY", default).lower()
        if mode not in ("autotune", "heuristics"):
            raise ValueError(f"EJKERNEL_AUTOTUNE_POLICY={mode!r}: expected 'autotune' or 'heuristics'")
        return AutotunePolicy(allow_autotune=mode == "autotune", cache_miss_fallback=mode)


class ConfigSelectorChain:
    """override -> overlay -> memory cache -> persistent cache -> autotune -> heuristic, with the reference's
    events (``override``, ``overlay_hit``, ``cache_hit``, ``autotune_start``, ``autotune_finish``, ``heuristics``,
    ``error``) reported to ``on_event`` (selection.py:384-578)."""

    def __init__(self, cache: ConfigCache | None = None, policy: AutotunePolicy | None = None,
                 persistent: PersistentCache | None = None, on_event: Callable[..., None] | None = None,
                 persist_autotune: bool = True, forbid_reautotune: bool = True):
        self.cache = cache if cache is not None else ConfigCache()
        self.policy = policy if policy is not None else AutotunePolicy()
        self.persistent = persistent
        self.on_event = on_event
        self.persist_autotune = persist_autotune
        self.forbid_reautotune = forbid_reautotune
        self._autotuned_keys: set[tuple[str, str, str]] = set()

    def _emit(self, event: str, **data) -> None:
        if self.on_event:
            self.on_event(event, **data)

    def choose(self, device: str, op_id: str, call_key: str, *, override=None,
               autotune: Callable[[], Any] | None = None, heuristic: Callable[[], Any] | None = None,
               may_autotune: bool = True):
        """``autotune()`` measures the candidates and returns the best; ``heuristic()`` returns the default.
        ``may_autotune=False`` (the stream is being captured into a graph, say) skips the measuring tier for this
        call without remembering the heuristic, so that a later call can still tune."""
        key = (device, op_id, call_key)
        if override is not None:
            self._emit("override", device=device, op_id=op_id, call_key=call_key, cfg=override)
            self.cache.put(*key, override)
            if self.persistent is not None:
                self.persistent.put(*key, override)
            return override
        for ov in reversed(_overlays):
            if (cfg := ov.get(key)) is not None:
                self._emit("overlay_hit", device=device, op_id=op_id, call_key=call_key, cfg=cfg)
                return cfg
        if (cfg := self.cache.get(*key)) is not None:
            self._emit("cache_hit", level="memory", device=device, op_id=op_id, call_key=call_key, cfg=cfg)
            return cfg
        if self.persistent is not None and (cfg := self.persistent.get(*key)) is not None:
            self._emit("cache_hit", level="persistent", device=device, op_id=op_id, call_key=call_key, cfg=cfg)
            self.cache.put(*key, cfg)
            return cfg
        if self.policy.cache_miss_fallback == "autotune" and self.policy.allow_autotune and autotune is not None:
            if not may_autotune:
                if heuristic is None:
                    raise RuntimeError("autotune is not possible here and there is no heuristic")
                return heuristic()
            if self.forbid_reautotune and key in self._autotuned_keys:
                raise RuntimeError(f"Re-autotune requested for {key}")
            self._emit("autotune_start", device=device, op_id=op_id, call_key=call_key)
            best = autotune()
            self._autotuned_keys.add(key)
            self.cache.put(*key, best)
            if self.persistent is not None and self.persist_autotune:
                self.persistent.put(*key, best)
            self._emit("autotune_finish", device=device, op_id=op_id, call_key=call_key, cfg=best)
            return best
        if self.policy.allow_heuristics and heuristic is not None:
            cfg = heuristic()
            self._emit("heuristics", device=device, op_id=op_id, call_key=call_key, cfg=cfg)
            self.cache.put(*key, cfg)
            if self.persistent is not None and self.persist_autotune:
                self.persistent.put(*key, cfg)
            return cfg
        self._emit("error", device=device, op_id=op_id, call_key=call_key, reason="no_config")
        raise RuntimeError("No config found: override/overlay/cache/persistent/autotune/heuristics all unavailable.")
