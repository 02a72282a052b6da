"""Host-side logic that needs no GPU: the registry and operator surface mirror the reference's,
the C-ABI library loads and exports every symbol include/ejk_rpa.h declares, and argument errors
are raised before any launch."""

import inspect
import re
from pathlib import Path

import pytest
import torch

import ejkernel_b200 as ej
from ejkernel_b200 import _cabi
from ejkernel_b200.kernels import Backend, KernelRegistry, Platform, kernel_registry
from ejkernel_b200.utils import make_ragged_batch

ROOT = Path(__file__).resolve().parent.parent

# (name, kind, default) of ejkernel/kernels/_xla/ragged_page_attention/_interface.py:27-47
REFERENCE_SIGNATURE = [
    ("queries", "POSITIONAL_OR_KEYWORD", inspect.Parameter.empty),
    ("kv_pages", "POSITIONAL_OR_KEYWORD", inspect.Parameter.empty),
    ("context_lens", "POSITIONAL_OR_KEYWORD", inspect.Parameter.empty),
    ("block_tables", "POSITIONAL_OR_KEYWORD", inspect.Parameter.empty),
    ("query_start_loc", "POSITIONAL_OR_KEYWORD", inspect.Parameter.empty),
    ("num_seqs", "POSITIONAL_OR_KEYWORD", inspect.Parameter.empty),
    ("softmax_scale", "KEYWORD_ONLY", None),
    ("logits_soft_cap", "KEYWORD_ONLY", None),
    ("compute_dtype", "KEYWORD_ONLY", torch.bfloat16),  # jnp.bfloat16 in the reference
    ("optimized", "KEYWORD_ONLY", False),
    ("sliding_window", "KEYWORD_ONLY", None),
    ("softmax_aux", "KEYWORD_ONLY", None),
    ("mask_value", "KEYWORD_ONLY", None),
    ("num_kv_pages_per_block", "KEYWORD_ONLY", None),
    ("num_queries_per_block", "KEYWORD_ONLY", None),
    ("vmem_limit_bytes", "KEYWORD_ONLY", None),
    ("num_warps", "KEYWORD_ONLY", None),
    ("num_stages", "KEYWORD_ONLY", None),
]


def test_registered_under_the_reference_name_and_signature():
    assert kernel_registry.list_algorithms() == ["page_attention", "ragged_page_attention", "ragged_page_attention_v3"]
    (spec,) = kernel_registry.list_implementations("ragged_page_attention")
    assert spec.platform is Platform.CUDA and spec.backend is Backend.GPU and spec.priority == 0
    impl = kernel_registry.get("ragged_page_attention", platform="cuda", backend="gpu")
    assert impl is spec.implementation
    assert kernel_registry.get("ragged_page_attention", platform="cuda", backend="any") is impl
    got = [(p.name, p.kind.name, p.default) for p in inspect.signature(impl).parameters.values()]
    assert got == REFERENCE_SIGNATURE
    with pytest.raises(ValueError):
        kernel_registry.get("ragged_page_attention", platform="xla")
    with pytest.raises(ValueError):
        kernel_registry.get("flash_attention")


def test_registry_priority_and_signature_validation():
    reg = KernelRegistry()

    @reg.register("op", "xla", "any")
    def a(x, *, scale=None): ...

    @reg.register("op", Platform.CUDA, Backend.GPU, priority=5)
    def b(x, *, scale=None): ...

    assert reg.get("op") is b and reg.get("op", platform="xla", backend="gpu") is a
    assert reg.validate_signatures("op") is True

    @reg.register("op", "triton", "gpu")
    def c(x, *, scale=1.0): ...

    with pytest.warns(UserWarning, match="Signature mismatch"):
        assert reg.validate_signatures("op") is False
    with pytest.raises(ValueError):
        reg.validate_signatures("nope")


def test_public_operator_surface():
    sig = inspect.signature(ej.ragged_page_attention)
    names = list(sig.parameters)
    assert names[:7] == ["queries", "kv_pages", "context_lens", "block_tables", "query_start_loc", "num_seqs", "softmax_aux"]
    assert all(sig.parameters[n].kind.name == "POSITIONAL_ONLY" for n in names[:7])
    assert names[7:] == ["softmax_scale", "logits_soft_cap", "compute_dtype", "optimized", "sliding_window", "mask_value",
                         "vmem_limit_bytes", "platform", "cfg", "mesh", "in_specs", "out_specs"]
    k = ej.RaggedPageAttention()
    cfg = k.heuristic_cfg()
    assert cfg.platform == "cuda" and cfg.num_warps == 4 and cfg.num_stages == 1
    assert k.candidate_cfgs() == [cfg]
    assert k.get_impl(cfg) is kernel_registry.get("ragged_page_attention", "cuda", "gpu")
    with pytest.raises(ValueError, match="only the CUDA"):
        k.get_impl(ej.RaggedPageAttentionConfig(platform="triton"))


def test_library_exports_every_declared_symbol(rpa_lib):
    header = (ROOT / "include" / "ejk_rpa.h").read_text()
    declared = set(re.findall(r"EJK_RPA_API\s+[\w\s\*]+?\b(ejk_\w+)\s*\(", header))
    assert declared == set(_cabi.EXPORTS), (declared, set(_cabi.EXPORTS))
    for name in declared:
        assert getattr(rpa_lib, name) is not None
    assert rpa_lib.ejk_rpa_version() == 2
    assert _cabi.error_string(0) == "ok" and "head_dim" in _cabi.error_string(-3)
    # option plumbing is host-only
    old = _cabi.get_option("waves")
    _cabi.set_option("waves", 5)
    assert _cabi.get_option("waves") == 5
    _cabi.set_option("waves", old)
    for name in ("waves", "min_chunk", "path", "prefill_rows", "prefill_share", "prefill_split", "sort_items", "overlap", "fused_merge", "wait_ms", "profile"):
        assert isinstance(_cabi.get_option(name), int), name  # every option the header documents is readable
    with pytest.raises(_cabi.RpaLibraryError):
        _cabi.set_option("no_such_option", 1)
    with pytest.raises(_cabi.RpaLibraryError):
        _cabi.set_option("min_chunk", 100)  # must be a multiple of the 64-token stage


def test_struct_layouts_match_the_header():
    header = (ROOT / "include" / "ejk_rpa.h").read_text()
    for struct, cls in (("ejk_rpa_shape", _cabi.Shape), ("ejk_rpa_attrs", _cabi.Attrs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = re.findall(r"(int32_t|float)\s+(\w+);", body)
        assert [n for _, n in fields] == [n for n, _ in cls._fields_]
        for (ctype, _), (_, pyt) in zip(fields, cls._fields_):
            assert (ctype == "float") == (pyt is _cabi.c_float)


def test_no_cpu_fallback_and_host_validation():
    from ejkernel_b200.kernels._cuda.ragged_page_attention import ragged_page_attention

    b = make_ragged_batch([1], [10], num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=8, seed=1)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ragged_page_attention(*b.args())
    with pytest.raises(Exception):  # rank mismatch: jaxtyping type-check error, as in the reference
        ragged_page_attention(b.queries[0], b.kv_pages, b.context_lens, b.block_tables, b.query_start_loc, b.num_seqs)
    with pytest.raises(Exception):  # context_lens and block_tables disagree on num_seqs
        ragged_page_attention(b.queries, b.kv_pages, torch.zeros(3, dtype=torch.int32), b.block_tables, b.query_start_loc, b.num_seqs)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_cabi.RpaLibraryError, match="no fallback"):
        _cabi.load()


def test_product_code_never_imports_the_oracle():
    for path in list((ROOT / "ejkernel_b200").rglob("*.py")):
        text = path.read_text()
        assert "oracle" not in re.sub(r'""".*?"""', "", text, flags=re.S).replace("# oracle", ""), path


@pytest.mark.gpu
def test_stream_probe_reads_a_buffer_and_refuses_bad_arguments(rpa_lib):
    """The read-only streaming probe (the practical ceiling of the split-KV kernel): runs, reports no expired wait and a
    plausible rate on a buffer larger than the L2; null, misaligned and too-short arguments get negative codes."""
    import torch

    from ejkernel_b200 import _cabi

    buf = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    buf.random_(0, 255)
    rate = _cabi.stream_probe_gbs(buf, passes=3)
    assert 1000.0 < rate < 12000.0, rate
    sink = torch.zeros(2, dtype=torch.int32, device="cuda")
    lib = _cabi.load()
    assert lib.ejk_rpa_stream_probe(None, 1 << 20, sink.data_ptr(), None) == -1
    assert lib.ejk_rpa_stream_probe(buf.data_ptr() + 4, 1 << 20, sink.data_ptr(), None) == -8
    assert lib.ejk_rpa_stream_probe(buf.data_ptr(), 100, sink.data_ptr(), None) == -6
    assert lib.ejk_rpa_last_launch_count() == 0
    torch.cuda.synchronize()
    assert int(sink.abs().sum()) == 0
