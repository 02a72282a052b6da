"""Tuning persistence for the CUDA operators: the two tile hints the kernels honour, measured per
(device, operator version, call signature) and kept in a JSON file across runs.

Mirrors the part of the reference's ops layer that EasyDeL-style callers rely on -- the
``PersistentCache`` of ejkernel/ops/config/persistent.py:58-200 with its ``device|op@v|call_key``
keys (:114-125) and atomic file replacement (:190-200), and the measure-candidates-keep-the-best
step of ``Tuner`` (ejkernel/ops/config/selection.py:226-245) -- without the seven-tier selector
chain around it: there is one implementation here and two knobs.

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
from collections.abc import Callable, Sequence
from dataclasses import asdict, is_dataclass
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
    sig = {
        "queries": (tuple(queries.shape), str(queries.dtype)),
        "kv_pages": (tuple(kv_pages.shape), str(kv_pages.dtype)),
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
              timer: Callable[[Callable[[], Any]], float] = cuda_event_timer) -> tuple[Any, list[float]]:
    """Time ``run_with(cfg)`` for every candidate; the first of the fastest wins.  A candidate that
    raises is skipped (its time is ``inf``)."""
    times: list[float] = []
    for cfg in candidates:
        try:
            times.append(float(timer(run_with(cfg))))
        except Exception:  # a candidate the shapes do not admit
            times.append(float("inf"))
    if not times or min(times) == float("inf"):
        raise RuntimeError("no candidate configuration could be run")
    return candidates[times.index(min(times))], times
