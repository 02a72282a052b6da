from ._interface import RpaWorkspace, ragged_page_attention, ragged_page_attention_into

__all__ = ["RpaWorkspace", "ragged_page_attention", "ragged_page_attention_into"]
