"""Pins the oracle, and the CUDA path, to outputs the reference's own code produced.

``tests/golden/rpa_reference_triton.npz`` holds inputs and outputs of the reference's Triton kernel
``_ragged_paged_attn_fwd`` (ejkernel/kernels/_triton/ragged_page_attention/_triton_impl_fwd.py:27-208), executed
by Triton's interpreter from the reference checkout (``tests/golden/make_reference_fixtures.py``).  The CPU
test checks the oracle against them; the GPU test checks the CUDA operator against the same vectors."""

from pathlib import Path

import numpy as np
import pytest
import torch

from ejkernel_b200.utils import RaggedBatch
from oracle.rpa_oracle import blocked_as_written, compare, dense_reference

FIX = np.load(Path(__file__).parent / "golden" / "rpa_reference_triton.npz")
CASES = sorted({k.split(".")[0] for k in FIX.files if k.endswith(".out")})


def _bf16(a) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def load_case(name) -> tuple[RaggedBatch, np.ndarray, np.ndarray]:
    """The stored operands with the keywords of the XLA semantics, the reference's bf16 output (as float)
    and the same kernel's unrounded float32 output."""
    g = lambda k: FIX[f"{name}.{k}"]
    win, cap = int(g("sliding_window")), float(g("logits_soft_cap"))
    q = _bf16(g("queries"))
    b = RaggedBatch(q, _bf16(g("kv_pages")), torch.from_numpy(g("context_lens")), torch.from_numpy(g("block_tables")),
                    torch.from_numpy(g("query_start_loc")), torch.from_numpy(g("num_seqs")), float(g("softmax_scale")),
                    win or None, cap or None, None, dict(total_tokens=q.shape[0]))
    return b, _bf16(g("out")).float().numpy(), g("out_f32")


def test_fixture_file_is_the_reference_kernels_output():
    assert "interpreter" in str(FIX["how"]) and {"tpu_a", "tpu_b", "c1", "window", "softcap"} <= set(CASES)
    # the q-block kernel cannot run under this Triton; the file says so instead of holding outputs for it
    assert "qblock_error" in FIX.files and not any(k.endswith("out_qblock") for k in FIX.files)


@pytest.mark.parametrize("name", CASES)
def test_dense_oracle_matches_the_reference_kernel(name):
    b, ref16, ref32 = load_case(name)
    got = dense_reference(*b.args(), **b.kwargs())
    # the kernel computes in float32 (renormalising its accumulator after every page), the oracle in float64
    np.testing.assert_allclose(got, ref32, rtol=0, atol=2e-5)
    # the reference's launcher stores in the dtype of the queries; Triton's interpreter narrows float32 to bf16
    # by dropping the low 16 bits, so that output is within one bf16 ulp (2^-7 relative) of the same numbers
    np.testing.assert_allclose(got, ref16, rtol=2.0**-7 * 1.01, atol=1e-6)


@pytest.mark.parametrize("name", ["tpu_a", "c1", "softcap"])
def test_as_written_oracle_matches_the_reference_kernel(name):
    """The loop-for-loop restatement of the XLA implementation (bf16 carried state) against the same vectors;
    query rows are padded so that its 8-row blocks stay inside the array."""
    b, _, ref32 = load_case(name)
    T = b.queries.shape[0]
    b.queries = torch.cat([b.queries, torch.zeros((16, *b.queries.shape[1:]), dtype=b.queries.dtype)])
    r = compare(blocked_as_written(*b.args(), **b.kwargs()), ref32, rows=T)
    # bf16 logits and carried state: the stated tolerance holds, the tighter rms criterion is not expected to
    assert r["finite"] and r["allclose"] and r["max_rel_rms"] < 0.1, r


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_cuda_operator_matches_the_reference_kernel(name):
    from tests.helpers import assert_parity, run_cuda, status_word

    b, _, ref32 = load_case(name)
    bc = b.to("cuda")
    out = run_cuda(bc)
    assert status_word(bc) == 0
    assert_parity(out, ref32, rows=b.queries.shape[0], what=f"reference Triton fixture {name}")


# ---- the same reference kernel COMPILED by Triton for a B200 (tl.dot of float32 operands runs as TF32) ----
FIX_CUDA = np.load(Path(__file__).parent / "golden" / "rpa_reference_triton_cuda.npz")
CASES_CUDA = sorted({k.split(".")[0] for k in FIX_CUDA.files if k.endswith(".out_f32")})


def test_compiled_fixture_file():
    assert "compiled for NVIDIA B200" in str(FIX_CUDA["how"]) and {"tpu_a", "fresh_prefill", "small_window"} <= set(CASES_CUDA)
    # what did not compile says why: the q-block kernel, and the soft-cap branch of the default kernel
    assert "qblock_error" in FIX_CUDA.files and "LOG2_CONST" in str(FIX_CUDA["small_softcap.error"])


@pytest.mark.parametrize("name", CASES_CUDA)
def test_dense_oracle_matches_the_compiled_reference_kernel(name):
    b, _, interp32 = load_case(name)
    ref32 = FIX_CUDA[f"{name}.out_f32"]
    got = dense_reference(*b.args(), **b.kwargs())
    # TF32 contractions: 10 mantissa bits on q, k, p and v
    r = compare(ref32, got, atol=2e-3, rtol=2e-3)
    assert r["finite"] and r["allclose"] and r["max_rel_rms"] < 1e-2, r
    # and the interpreter's run of the same kernel on the same inputs agrees with the compiled one
    assert compare(ref32, interp32, atol=2e-3, rtol=2e-3)["allclose"]


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES_CUDA)
def test_cuda_operator_matches_the_compiled_reference_kernel(name):
    from tests.helpers import assert_parity, run_cuda

    b, _, _ = load_case(name)
    assert_parity(run_cuda(b.to("cuda")), FIX_CUDA[f"{name}.out_f32"], rows=b.queries.shape[0],
                  what=f"reference Triton kernel compiled for B200, {name}")
