"""The CUDA entries check operand shapes and dtypes with jaxtyping + beartype like the reference's
interfaces do (ejkernel/kernels/_xla/ragged_page_attention/_interface.py:26), but only on the first
call with a given combination of shapes, dtypes, devices and keyword types."""

import inspect

import pytest
import torch
from jaxtyping import Float, Int
from torch import Tensor as Array

from ejkernel_b200.kernels._cuda._typecheck import typechecked_once


def _make():
    calls = []

    @typechecked_once
    def op(x: Float[Array, "rows cols"], idx: Int[Array, "rows"], *, scale: float | None = None) -> Float[Array, "rows cols"]:
        calls.append((tuple(x.shape), scale))
        return x * (1.0 if scale is None else scale)

    return op, calls


def test_a_signature_is_checked_once_and_a_bad_one_every_time():
    op, calls = _make()
    x, idx = torch.zeros(4, 3), torch.zeros(4, dtype=torch.int32)
    op(x, idx, scale=2.0)
    op(x, idx, scale=3.0)           # same signature (values are not part of it): body only
    assert len(calls) == 2
    for _ in range(2):              # a mismatch is never remembered
        with pytest.raises(Exception) as e:
            op(x, torch.zeros(5, dtype=torch.int32))
        assert "TypeCheck" in type(e.value).__name__ or "beartype" in type(e.value).__module__
    with pytest.raises(Exception):
        op(x, idx.float())          # float index array
    with pytest.raises(Exception):
        op(x, idx, scale="2")       # keyword of the wrong type
    assert len(calls) == 2
    op(torch.zeros(6, 3), torch.zeros(6, dtype=torch.int64))  # a new shape is checked and passes
    assert len(calls) == 3


def test_wrapper_keeps_the_signature_the_registry_compares():
    op, _ = _make()
    params = inspect.signature(op).parameters
    assert list(params) == ["x", "idx", "scale"]
    assert params["scale"].kind is inspect.Parameter.KEYWORD_ONLY and params["scale"].default is None


def test_registered_entries_use_it_and_still_validate():
    from ejkernel_b200.kernels import kernel_registry
    from ejkernel_b200.kernels._cuda import page_attention, ragged_page_attention, ragged_page_attention_v3
    for fn in (page_attention, ragged_page_attention, ragged_page_attention_v3):
        assert hasattr(fn, "typechecked"), fn
    assert kernel_registry.validate_signatures()
    # rank mismatch on CPU tensors: rejected by the type check before anything touches a device
    q = torch.zeros(4, 8, dtype=torch.bfloat16)
    with pytest.raises(Exception) as e:
        ragged_page_attention(q, torch.zeros(2, 16, 4, 128, dtype=torch.bfloat16), torch.zeros(2, dtype=torch.int32),
                              torch.zeros(2, 4, dtype=torch.int32), torch.zeros(3, dtype=torch.int32), 2)
    assert "TypeCheck" in type(e.value).__name__ or "beartype" in type(e.value).__module__
