"""Operation configs with the fields of the reference's
(ejkernel/modules/operations/configs.py:29-34,242-258)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal


@dataclass
class BaseOperationConfig:
    platform: Literal["triton", "pallas", "cuda", "xla", "auto"] = "auto"
    backend: str = "any"


@dataclass
class RaggedPageAttentionConfig(BaseOperationConfig):
    """``num_kv_pages_per_block`` / ``num_queries_per_block`` are tile hints (None = auto);
    ``num_warps`` / ``num_stages`` exist for signature parity and are ignored by the CUDA path,
    as they are by the reference's XLA path."""

    num_kv_pages_per_block: int | None = None
    num_queries_per_block: int | None = None
    num_warps: int = 4
    num_stages: int = 1
