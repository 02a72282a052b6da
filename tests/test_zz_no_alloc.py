"""The workspace-free entry point ``ejk_rpa_launch_static_scratch``.

Some callers cannot hand the library a scratch buffer because they cannot allocate device memory
where they call from: an XLA-style custom-call handler gets only its operand and result buffers, a
plugin inside another framework's memory pool must not call cudaMalloc itself, and a latency
critical serving loop must not risk the implicit synchronisation of an allocation.  For them the
library carries a fixed 32 MiB scratch array in its own device image.

This test drives that entry point directly through the C ABI (ctypes, raw device pointers) and
checks its output against the ordinary ``ejk_rpa_launch`` on the same inputs, twice in a row:
the second call runs on top of whatever the first left in the shared array and must not be
affected by it.  It also checks that a shape needing more than the built-in array is refused
with the dedicated error code and launches nothing.

The file name makes pytest collect it last, so a run that stops at the first failure has
already exercised everything else.
"""

import ctypes

import pytest
import torch

from ejkernel_b200 import _cabi
from ejkernel_b200.kernels._cuda.ragged_page_attention import RpaWorkspace, ragged_page_attention_into
from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import _shape_of
from ejkernel_b200.utils import make_ragged_batch, make_workload
from oracle.rpa_oracle import compare, dense_reference
from tests.helpers import ATOL, REL_RMS, RTOL

pytestmark = pytest.mark.gpu


def _launch_static(lib, b, out, status):
    """Raw C-ABI call: pointers and plain structs only."""
    shape = _shape_of(b.queries, b.kv_pages, b.block_tables)
    attrs = _cabi.Attrs(b.softmax_scale, b.logits_soft_cap or 0.0, b.sliding_window or 0, 0, 0, 0, 0)
    return lib.ejk_rpa_launch_static_scratch(
        b.queries.data_ptr(), b.kv_pages.data_ptr(), b.context_lens.data_ptr(), b.block_tables.data_ptr(),
        b.query_start_loc.data_ptr(), b.num_seqs.data_ptr(), None, out.data_ptr(), status.data_ptr(),
        ctypes.byref(shape), ctypes.byref(attrs), torch.cuda.current_stream().cuda_stream)


def _reference_run(b):
    ws = RpaWorkspace(_shape_of(b.queries, b.kv_pages, b.block_tables), b.queries.device)
    out = torch.zeros_like(b.queries)
    ragged_page_attention_into(out, ws, *b.args(), softmax_scale=b.softmax_scale, sliding_window=b.sliding_window,
                               logits_soft_cap=b.logits_soft_cap)
    torch.cuda.synchronize()
    assert int(ws.status.item()) == 0
    return out


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(rpa_lib):
    # first a long-context decode batch that splits every sequence into many KV chunks (so the
    # shared array really carries work lists and partials), then a different, mixed batch with a
    # window and a soft cap on top of the leftovers of the first
    first = make_workload("c2", num_seqs=40, len_scale=0.5, device="cuda")
    second = make_ragged_batch([1, 9, 1, 30, 1], [3000, 700, 64, 1500, 5], num_q_heads=8, num_kv_heads=2, head_dim=128,
                               page_size=16, seed=41, sliding_window=512, logits_soft_cap=30.0).to("cuda")
    for b in (first, second):
        assert _cabi.load().ejk_rpa_workspace_bytes_min(ctypes.byref(_shape_of(b.queries, b.kv_pages, b.block_tables))) \
            <= _cabi.STATIC_SCRATCH_BYTES
        want = _reference_run(b)
        out = torch.zeros_like(b.queries)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        rc = _launch_static(rpa_lib, b, out, status)
        assert rc == 0, _cabi.error_string(rc)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        T = b.total_tokens
        r = compare(out[:T], want[:T].float().cpu().numpy(), atol=ATOL, rtol=RTOL)
        assert r["finite"] and r["allclose"] and r["tight"] and r["max_rel_rms"] <= REL_RMS, r
        assert torch.count_nonzero(out[T:]) == 0
    # the second batch once more, directly against the CPU oracle, with the device's free memory read before and
    # after: the call must not have allocated anything (the look-up of the array's address happened on the first call)
    bcpu = second.to("cpu")
    oracle_out = dense_reference(*bcpu.args(), **bcpu.kwargs())
    out.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    rc = _launch_static(rpa_lib, second, out, status)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert rc == 0 and int(status.item()) == 0
    assert free_after == free_before, "the workspace-free entry point allocated device memory"
    r = compare(out, oracle_out, atol=ATOL, rtol=RTOL, rows=second.total_tokens)
    assert r["finite"] and r["allclose"] and r["tight"], r


def test_static_scratch_refuses_shapes_beyond_its_maximum(rpa_lib):
    # thousands of query rows need far more partial slots than 32 MiB holds
    b = make_ragged_batch([3000], [3000], num_q_heads=32, num_kv_heads=8, head_dim=128, page_size=16, seed=1).to("cuda")
    need = rpa_lib.ejk_rpa_workspace_bytes_min(ctypes.byref(_shape_of(b.queries, b.kv_pages, b.block_tables)))
    assert need > _cabi.STATIC_SCRATCH_BYTES
    out = torch.full_like(b.queries, 7.0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _launch_static(rpa_lib, b, out, status)
    assert rc == _cabi.E_SCRATCH
    assert "static buffer" in _cabi.error_string(rc)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()), "a refused call must not launch anything"
    # invalid arguments are refused with the library's own codes before the array's address is looked up
    small = make_ragged_batch([1], [20], num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=8, seed=2).to("cuda")
    shape = _shape_of(small.queries, small.kv_pages, small.block_tables)
    attrs = _cabi.Attrs(small.softmax_scale, 0.0, 0, 0, 0, 0, 0)
    o = torch.zeros_like(small.queries)
    rc = rpa_lib.ejk_rpa_launch_static_scratch(
        small.queries.data_ptr(), None, small.context_lens.data_ptr(), small.block_tables.data_ptr(),
        small.query_start_loc.data_ptr(), small.num_seqs.data_ptr(), None, o.data_ptr(), status.data_ptr(),
        ctypes.byref(shape), ctypes.byref(attrs), torch.cuda.current_stream().cuda_stream)
    assert rc == -1  # EJK_RPA_E_NULL
