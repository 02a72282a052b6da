"""Shape/dtype checking of the CUDA entries: jaxtyping + beartype, once per call signature.

The reference decorates its kernel interfaces with ``@jaxtyping.jaxtyped(typechecker=beartype)``
(ejkernel/kernels/_xla/ragged_page_attention/_interface.py:26) and runs them under ``jax.jit``, so
the check costs nothing after the first trace of a shape.  Here the operators run eagerly and
the same decorator costs ~80 us of host time per call -- several times the device time of a small
decode batch.  ``typechecked_once`` keeps the reference's behaviour (the first call with a given
combination of operand shapes, dtypes, devices and keyword types is checked in full and raises
the same ``TypeCheckError``) and lets later calls with an identical combination go straight to
the body, which still validates everything that depends on values.
"""

from __future__ import annotations

import functools

import jaxtyping
import torch
from beartype import beartype


def _describe(value):
    if isinstance(value, torch.Tensor):
        return (tuple(value.shape), value.dtype, value.device.type)
    return type(value)


def typechecked_once(fn):
    checked = jaxtyping.jaxtyped(typechecker=beartype)(fn)
    seen: set = set()

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        key = (tuple(_describe(a) for a in args), tuple((k, _describe(v)) for k, v in sorted(kwargs.items())))
        if key in seen:
            return fn(*args, **kwargs)
        out = checked(*args, **kwargs)
        seen.add(key)  # only signatures that passed the check are remembered
        return out

    wrapper.typechecked = checked  # the always-checking form, for tests
    return wrapper
