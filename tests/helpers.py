"""Shared helpers of the test-suite: run the CUDA operator and the CPU oracle on one batch."""

from __future__ import annotations

import numpy as np
import torch

from ejkernel_b200.utils import RaggedBatch
from oracle.rpa_oracle import compare, dense_reference

ATOL = RTOL = 2e-2  # bf16 tolerance of the operator's parity criterion
REL_RMS = 1.0  # loose sanity bound on max error / RMS of the expected output; the sharp check is compare()["tight"]


def run_cuda(batch: RaggedBatch, **override) -> torch.Tensor:
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import read_status

    b = batch if batch.queries.is_cuda else batch.to("cuda")
    read_status(b.queries)  # the operator's status word is per stream, not per shape: drop what earlier calls left
    kw = b.kwargs()
    kw.update(override)
    out = ragged_page_attention(*b.args(), **kw)
    torch.cuda.synchronize()
    return out


def status_word(batch_cuda: RaggedBatch) -> int:
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import read_status

    return read_status(batch_cuda.queries, batch_cuda.kv_pages, batch_cuda.block_tables)


def oracle(batch: RaggedBatch, precision="fp64") -> np.ndarray:
    b = batch if not batch.queries.is_cuda else batch.to("cpu")
    return dense_reference(*b.args(), **b.kwargs(), precision=precision)


def assert_parity(got: torch.Tensor, want: np.ndarray, rows: int, *, rel_rms=REL_RMS, what=""):
    r = compare(got, want, atol=ATOL, rtol=RTOL, rows=rows)
    assert r["finite"], f"{what}: non-finite output {r}"
    assert r["allclose"], f"{what}: outside atol=rtol={ATOL}: {r}"
    assert r["tight"], f"{what}: outside 3e-2*rms(expected) + 1e-2*|expected|: {r}"
    assert r["max_rel_rms"] <= rel_rms, f"{what}: max|err| / rms(expected) = {r['max_rel_rms']:.4g} > {rel_rms}: {r}"
    return r
