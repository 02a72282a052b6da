"""ctypes binding of ``libejk_rpa.so`` (the C ABI declared in ``include/ejk_rpa.h``).

This is the host-side stub a reference maintainer would add for the CUDA platform: it plays
the role ``jaxlib``'s ``gpu_triton`` custom call plays for the Triton kernels
(ejkernel/callib/_triton_call.py:36,737-757).  There is no CPU fallback: if the library is
missing or cannot be loaded the import of the CUDA operator fails loudly.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libejk_rpa.so"

BF16, F16, E4M3 = 0, 1, 2
STATIC_SCRATCH_BYTES = 32 << 20
E_SCRATCH = -9

ST_NUM_SEQS, ST_QLEN, ST_KVLEN, ST_PAGE_ID, ST_INTERNAL, ST_TIMEOUT = 1, 2, 4, 8, 16, 32
STATUS_TEXT = {
    ST_NUM_SEQS: "num_seqs exceeds block_tables.shape[0]",
    ST_QLEN: "a sequence has q_len < 0, q_len > kv_len or query rows past total_tokens",
    ST_KVLEN: "a context length is negative or exceeds pages_per_seq * page_size",
    ST_PAGE_ID: "a page id outside [0, num_pages) was read from block_tables",
    ST_INTERNAL: "the device planner ran out of workspace",
    ST_TIMEOUT: "a bounded wait inside a kernel ran out; outputs are invalid",
}

EXPORTS = (
    "ejk_rpa_version",
    "ejk_rpa_error_string",
    "ejk_rpa_workspace_bytes",
    "ejk_rpa_workspace_bytes_min",
    "ejk_rpa_launch",
    "ejk_rpa_set_option",
    "ejk_rpa_get_option",
    "ejk_rpa_last_launch_count",
    "ejk_rpa_profile_read",
    "ejk_rpa_profile_read_kernels",
    "ejk_rpa_launch_static_scratch",
    "ejk_rpa_v3_launch",
    "ejk_page_attention_launch",
    "ejk_rpa_stream_probe",
)


class Shape(Structure):
    _fields_ = [
        ("total_tokens", c_int32),
        ("max_num_seqs", c_int32),
        ("pages_per_seq", c_int32),
        ("num_pages", c_int32),
        ("page_size", c_int32),
        ("num_q_heads", c_int32),
        ("num_kv_heads", c_int32),
        ("head_dim", c_int32),
        ("dtype", c_int32),
        ("kv_dtype", c_int32),
    ]


class Attrs(Structure):
    _fields_ = [
        ("softmax_scale", c_float),
        ("logits_soft_cap", c_float),
        ("sliding_window", c_int32),
        ("num_sinks", c_int32),
        ("sink_rows", c_int32),
        ("num_kv_pages_per_block", c_int32),
        ("num_queries_per_block", c_int32),
        ("q_scale", c_float),
        ("out_scale", c_float),
    ]


class RpaLibraryError(RuntimeError):
    pass


_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RpaLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m ejkernel_b200._build` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.ejk_rpa_version.restype = c_int
    lib.ejk_rpa_version.argtypes = []
    lib.ejk_rpa_error_string.restype = c_char_p
    lib.ejk_rpa_error_string.argtypes = [c_int]
    lib.ejk_rpa_workspace_bytes.restype = c_size_t
    lib.ejk_rpa_workspace_bytes.argtypes = [POINTER(Shape)]
    lib.ejk_rpa_workspace_bytes_min.restype = c_size_t
    lib.ejk_rpa_workspace_bytes_min.argtypes = [POINTER(Shape)]
    lib.ejk_rpa_launch.restype = c_int
    lib.ejk_rpa_launch.argtypes = [
        c_void_p,  # queries
        c_void_p,  # kv_pages
        c_void_p,  # context_lens
        c_void_p,  # block_tables
        c_void_p,  # query_start_loc
        c_void_p,  # num_seqs
        c_void_p,  # softmax_aux
        c_void_p,  # out
        c_void_p,  # workspace
        c_size_t,
        c_void_p,  # status
        POINTER(Shape),
        POINTER(Attrs),
        c_void_p,  # stream
    ]
    lib.ejk_rpa_set_option.restype = c_int
    lib.ejk_rpa_set_option.argtypes = [c_char_p, c_int]
    lib.ejk_rpa_get_option.restype = c_int
    lib.ejk_rpa_get_option.argtypes = [c_char_p, POINTER(c_int)]
    lib.ejk_rpa_last_launch_count.restype = c_int
    lib.ejk_rpa_last_launch_count.argtypes = []
    lib.ejk_rpa_launch_static_scratch.restype = c_int
    lib.ejk_rpa_launch_static_scratch.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # queries .. num_seqs
        c_void_p,  # softmax_aux
        c_void_p,  # out
        c_void_p,  # status
        POINTER(Shape),
        POINTER(Attrs),
        c_void_p,  # stream
    ]
    lib.ejk_rpa_v3_launch.restype = c_int
    lib.ejk_rpa_v3_launch.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p,  # queries, keys, values, kv_cache
        c_void_p, c_void_p, c_void_p, c_void_p,  # kv_lens, block_tables, query_start_loc, distribution
        c_void_p,  # out
        c_void_p,  # workspace
        c_size_t,
        c_void_p,  # status
        POINTER(Shape),
        POINTER(Attrs),
        c_void_p,  # stream
    ]
    lib.ejk_page_attention_launch.restype = c_int
    lib.ejk_page_attention_launch.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # query, key_cache, value_cache, context_lens, block_tables
        c_void_p,  # out
        c_void_p,  # workspace
        c_size_t,
        c_void_p,  # status
        POINTER(Shape),
        POINTER(Attrs),
        c_void_p,  # stream
    ]
    lib.ejk_rpa_profile_read.restype = c_int
    lib.ejk_rpa_profile_read.argtypes = [POINTER(c_float), POINTER(c_float), POINTER(c_float)]
    lib.ejk_rpa_profile_read_kernels.restype = c_int
    lib.ejk_rpa_profile_read_kernels.argtypes = [POINTER(c_float)] * 4
    lib.ejk_rpa_stream_probe.restype = c_int
    lib.ejk_rpa_stream_probe.argtypes = [c_void_p, c_size_t, c_void_p, c_void_p]
    _lib = lib
    return lib


def error_string(code: int) -> str:
    return load().ejk_rpa_error_string(int(code)).decode()


def check(code: int, what: str = "ejk_rpa") -> None:
    if code != 0:
        raise RpaLibraryError(f"{what} failed with code {code}: {error_string(code)}")


_option_mirror: dict[str, int] = {}  # values set or read through this module (options are process-wide and host-side)


def set_option(name: str, value: int) -> None:
    check(load().ejk_rpa_set_option(name.encode(), int(value)), f"set_option({name})")
    _option_mirror[name] = int(value)


def get_option_cached(name: str) -> int:
    """``get_option`` without the library call once the value is known; valid as long as options are only changed
    through ``set_option`` of this module."""
    v = _option_mirror.get(name)
    if v is None:
        v = _option_mirror[name] = get_option(name)
    return v


def get_option(name: str) -> int:
    v = c_int(0)
    check(load().ejk_rpa_get_option(name.encode(), ctypes.byref(v)), f"get_option({name})")
    return v.value


def profile_read() -> tuple[float, float, float]:
    """(planner, attention, merge) device milliseconds of this thread's last profiled launch."""
    a, b, c = c_float(0), c_float(0), c_float(0)
    check(load().ejk_rpa_profile_read(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)), "profile_read")
    return a.value, b.value, c.value


def profile_read_kernels() -> tuple[float, float, float, float]:
    """(planner, prefill-tile kernel, split-KV kernel, merge) device milliseconds of this thread's last profiled launch."""
    v = [c_float(0) for _ in range(4)]
    check(load().ejk_rpa_profile_read_kernels(*[ctypes.byref(x) for x in v]), "profile_read_kernels")
    return tuple(x.value for x in v)


# (KB per copy, slots per CTA, CTAs per SM) the probe is tried with.  Measured on a B200 over a 4 GiB buffer, GB/s:
# 64/1/2 7360-7420, 32/1/4 7380, 32/2/3 7280, 64/3/1 7265, 32/3/2 (the split-KV kernel's own shape) 7235-7255,
# 16/3/4 7200, 16/4/3 7050, 32/6/1 6810, 16/6/2 6770, 8/6/4 6780, 16/12/1 and 8/12/2 6280, 4/12/4 6165: few large
# copies in flight beat many small ones.
PROBE_SHAPES = ((64, 1, 2), (32, 1, 4), (32, 3, 2))


def stream_probe_gbs(tensor, passes: int = 5) -> float:
    """Read-only streaming rate of the tensor's device in GB/s: the best of ``PROBE_SHAPES``, each timed over ``passes``
    passes of ``ejk_rpa_stream_probe`` over the tensor's bytes (use one far larger than the L2) after one untimed
    pass.  The practical ceiling of the split-KV kernel on that device."""
    import torch

    if not tensor.is_cuda or not tensor.is_contiguous():
        raise ValueError("stream_probe_gbs needs a contiguous CUDA tensor")
    nbytes = tensor.numel() * tensor.element_size() // 65536 * 65536
    sink = torch.zeros(2, dtype=torch.int32, device=tensor.device)
    lib = load()
    with torch.cuda.device(tensor.device):
        st = torch.cuda.current_stream(tensor.device)
        run = lambda: check(lib.ejk_rpa_stream_probe(tensor.data_ptr(), nbytes, sink.data_ptr(), st.cuda_stream), "stream_probe")
        old = [get_option(k) for k in ("probe_chunk_kb", "probe_slots", "probe_ctas")]
        best = 0.0
        try:
            for shape in PROBE_SHAPES:
                for k, v in zip(("probe_chunk_kb", "probe_slots", "probe_ctas"), shape):
                    set_option(k, v)
                run()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(st)
                for _ in range(passes):
                    run()
                e1.record(st)
                e1.synchronize()
                best = max(best, nbytes * passes / (e0.elapsed_time(e1) * 1e-3) / 1e9)
        finally:
            for k, v in zip(("probe_chunk_kb", "probe_slots", "probe_ctas"), old):
                set_option(k, v)
        if int(sink[1].item()) != 0:
            raise RpaLibraryError("stream_probe: a wait inside the probe ran out")
        return best


def decode_status(word: int) -> list[str]:
    return [txt for bit, txt in STATUS_TEXT.items() if word & bit]
