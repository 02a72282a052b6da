"""Kernel implementations, grouped by platform as in the reference (ejkernel/kernels/__init__.py:51-54).
Only ``_cuda`` exists here; importing it registers its operators."""

from . import _cuda  # noqa: F401  (registers the CUDA implementations)
from ._registry import Backend, KernelRegistry, KernelSpec, Platform, kernel_registry

__all__ = ["Backend", "KernelRegistry", "KernelSpec", "Platform", "kernel_registry"]
