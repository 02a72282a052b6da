from ._interface import (
    RpaWorkspace,
    ragged_page_attention,
    ragged_page_attention_into,
    ragged_page_attention_static_scratch_into,
)

__all__ = [
    "RpaWorkspace",
    "ragged_page_attention",
    "ragged_page_attention_into",
    "ragged_page_attention_static_scratch_into",
]
