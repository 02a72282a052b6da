"""Algorithm registry with the same surface as the reference's
(ejkernel/kernels/_registry.py:86-377): ``kernel_registry.register(algorithm, platform, backend,
priority)`` as a decorator, ``.get(algorithm, platform, backend)`` returning the best match,
``.list_algorithms()``, ``.list_implementations()`` and ``.validate_signatures()``.

Only the CUDA platform is populated by this package; the enums keep the reference's members so
that a spec written for one registry is valid for the other.
"""

from __future__ import annotations

import inspect
import warnings
from dataclasses import dataclass
from enum import Enum
from typing import Callable


class Platform(str, Enum):
    TRITON = "triton"
    PALLAS = "pallas"
    CUDA = "cuda"
    XLA = "xla"


class Backend(str, Enum):
    GPU = "gpu"
    TPU = "tpu"
    CPU = "cpu"
    ANY = "any"


@dataclass(frozen=True)
class KernelSpec:
    platform: Platform
    backend: Backend
    algorithm: str
    implementation: Callable
    priority: int = 0


def _annotation_text(a) -> str:
    if a is inspect.Parameter.empty:
        return ""
    txt = a if isinstance(a, str) else getattr(a, "__name__", None) or repr(a)
    return "".join(str(txt).split()).replace("typing.", "")


class KernelRegistry:
    """algorithm name -> implementations, highest priority first."""

    def __init__(self) -> None:
        self._by_algorithm: dict[str, list[KernelSpec]] = {}

    def register(self, algorithm: str, platform, backend, priority: int = 0):
        plat, back = Platform(platform), Backend(backend)

        def deco(fn):
            specs = self._by_algorithm.setdefault(algorithm.lower(), [])
            specs.append(KernelSpec(plat, back, algorithm, fn, priority))
            specs.sort(key=lambda s: -s.priority)  # stable: equal priorities keep insertion order
            return fn

        return deco

    def get(self, algorithm: str, platform=None, backend=None) -> Callable:
        specs = self._by_algorithm.get(algorithm.lower())
        if not specs:
            raise ValueError(f"No implementation found for algorithm: {algorithm}")
        plat = None if platform is None else Platform(platform)
        back = None if backend is None else Backend(backend)
        for spec in specs:
            if plat is not None and spec.platform is not plat:
                continue
            # an implementation registered for ANY backend serves every query, and a query for ANY
            # backend is served by whatever this process can run (the reference resolves it through
            # jax.default_backend(), _registry.py:239-243; here the only device kind is a GPU).
            if back is not None and back is not Backend.ANY and spec.backend not in (back, Backend.ANY):
                continue
            return spec.implementation
        raise ValueError(f"No implementation found for algorithm={algorithm}, platform={platform}, backend={backend}")

    def list_algorithms(self) -> list[str]:
        return sorted(self._by_algorithm)

    def list_implementations(self, algorithm: str) -> list[KernelSpec]:
        return list(self._by_algorithm.get(algorithm.lower(), ()))

    def validate_signatures(self, algorithm: str | None = None, verbose: bool = False) -> bool:
        """Warn (never raise) when implementations of one algorithm disagree on parameter names,
        order, kinds, defaults or annotations; the first spec is the yardstick."""
        if algorithm is None:
            return all([self.validate_signatures(a, verbose) for a in self.list_algorithms()])
        specs = self._by_algorithm.get(algorithm.lower())
        if specs is None:
            raise ValueError(f"No implementation found for algorithm: {algorithm}")
        ref = specs[0]
        ref_params = list(inspect.signature(ref.implementation).parameters.values())
        ok = True
        for spec in specs[1:]:
            params = list(inspect.signature(spec.implementation).parameters.values())
            if verbose:
                print(f"{algorithm}: {spec.platform.value}/{spec.backend.value}: {[p.name for p in params]}")
            problems = []
            if len(params) != len(ref_params):
                problems.append(f"{len(params)} parameters instead of {len(ref_params)}")
            for a, b in zip(ref_params, params):
                if a.name != b.name:
                    problems.append(f"parameter '{b.name}' where '{a.name}' is expected")
                    continue
                if a.kind != b.kind:
                    problems.append(f"'{a.name}' is {b.kind.name}, expected {a.kind.name}")
                if a.default != b.default:
                    problems.append(f"'{a.name}' defaults to {b.default!r}, expected {a.default!r}")
                if _annotation_text(a.annotation) != _annotation_text(b.annotation):
                    problems.append(f"'{a.name}' annotated {b.annotation!r}, expected {a.annotation!r}")
            if problems:
                ok = False
                warnings.warn(
                    f"Signature mismatch for algorithm '{algorithm}' between "
                    f"{ref.platform.value}/{ref.backend.value} and {spec.platform.value}/{spec.backend.value}: "
                    + "; ".join(problems),
                    UserWarning,
                    stacklevel=2,
                )
        return ok


kernel_registry = KernelRegistry()
