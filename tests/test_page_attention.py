"""``page_attention``: decode over separate paged key / value caches.  CPU: the oracle restatement
against the ragged oracle on the same data in the other layout.  GPU: the CUDA path through the C ABI
against the oracle, the reference's own test shapes, and bit-equality with ``ragged_page_attention`` on
the interleaved copy of the same cache (same kernels, different tensor map)."""

import numpy as np
import pytest
import torch

from ejkernel_b200.utils import make_ragged_batch, make_workload
from oracle.rpa_oracle import dense_reference, page_attention_reference
from tests.helpers import assert_parity


def _split(b):
    """Interleaved pool [P, page, 2Hkv, D] -> key_cache, value_cache [P, Hkv, page, D]."""
    kc = b.kv_pages[:, :, 0::2, :].permute(0, 2, 1, 3).contiguous()
    vc = b.kv_pages[:, :, 1::2, :].permute(0, 2, 1, 3).contiguous()
    return kc, vc


def _decode_batch(kv_lens, **kw):
    return make_ragged_batch([1] * len(kv_lens), kv_lens, **kw)


def test_oracle_page_attention_agrees_with_ragged_oracle():
    b = _decode_batch([300, 17, 64, 1], num_q_heads=8, num_kv_heads=2, head_dim=64, page_size=16, seed=71)
    kc, vc = _split(b)
    got = page_attention_reference(b.queries, kc, vc, b.context_lens, b.block_tables, attn_scale=b.softmax_scale)
    np.testing.assert_allclose(got, dense_reference(*b.args(), **b.kwargs()), atol=1e-12)
    capped = page_attention_reference(b.queries, kc, vc, b.context_lens, b.block_tables, attn_logits_soft_cap=5.0)
    np.testing.assert_allclose(capped, dense_reference(*b.args(), logits_soft_cap=5.0), atol=1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("page,hq,hkv,d", [(16, 8, 2, 128), (8, 8, 4, 64), (32, 16, 8, 256), (64, 4, 4, 128), (16, 32, 2, 128),
                                           (24, 8, 4, 64), (48, 8, 2, 128), (4, 8, 2, 128), (12, 8, 4, 64), (1, 4, 2, 128)])
# 24 and 48: 8- and 16-token TMA boxes; the last three (no multiple of 8): cp.async gather
def test_cuda_page_attention_matches_oracle(rpa_lib, page, hq, hkv, d):
    import ejkernel_b200 as ej

    b = _decode_batch([3000, 257, 64, 1, 900, 4500], num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, seed=page + d)
    kc, vc = _split(b)
    bc = b.to("cuda")
    out = ej.page_attention(bc.queries, kc.cuda(), vc.cuda(), bc.context_lens, bc.block_tables, attn_scale=b.softmax_scale)
    torch.cuda.synchronize()
    want = page_attention_reference(b.queries, kc, vc, b.context_lens, b.block_tables, attn_scale=b.softmax_scale)
    assert_parity(out, want, 6, what=f"page_attention page{page} d{d}")
    # same kernels, same bytes, other layout: bit-identical to the ragged operator (with the default configuration:
    # left alone, the operator measures its candidates on the first call and may cut the contexts differently)
    ref = ej.ragged_page_attention(*bc.args(), softmax_scale=b.softmax_scale, cfg=ej.RaggedPageAttention().heuristic_cfg())
    assert torch.equal(out, ref)


@pytest.mark.gpu
def test_cuda_page_attention_reference_test_shapes_soft_cap_and_errors(rpa_lib):
    import ejkernel_b200 as ej

    # test/kernels/_xla/test_page_attention.py: ones everywhere -> output is all ones
    q = torch.ones((2, 8, 64), dtype=torch.bfloat16, device="cuda")
    kc = torch.ones((8, 4, 16, 64), dtype=torch.bfloat16, device="cuda")
    vc = torch.ones_like(kc)
    out = ej.page_attention(q, kc, vc, torch.tensor([48, 32], dtype=torch.int32, device="cuda"),
                            torch.tensor([[0, 1, 2, 3], [4, 5, 6, 7]], dtype=torch.int32, device="cuda"))
    assert out.shape == (2, 8, 64) and torch.equal(out, torch.ones_like(out))
    b = _decode_batch([700, 90], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, seed=72)
    kcb, vcb = _split(b)
    bc = b.to("cuda")
    out = ej.page_attention(bc.queries, kcb.cuda(), vcb.cuda(), bc.context_lens, bc.block_tables, attn_logits_soft_cap=3.0)
    want = page_attention_reference(b.queries, kcb, vcb, b.context_lens, b.block_tables, attn_logits_soft_cap=3.0)
    assert_parity(out, want, 2, what="page_attention soft cap")
    zero = ej.page_attention(bc.queries, kcb.cuda(), vcb.cuda(), torch.zeros(2, dtype=torch.int32, device="cuda"), bc.block_tables)
    assert torch.count_nonzero(zero) == 0
    # block_size 4 (not expressible as a TMA box): still all ones
    small = ej.page_attention(q, kc[:, :, :4].contiguous(), vc[:, :, :4].contiguous(),
                              torch.tensor([4, 4], dtype=torch.int32, device="cuda"),
                              torch.tensor([[0], [1]], dtype=torch.int32, device="cuda"))
    assert torch.equal(small, torch.ones_like(small))
    with pytest.raises(ValueError):
        ej.page_attention(q, kc, vc, torch.tensor([48, 32], device="cuda"),
                          torch.tensor([[0, 1, 2, 3], [4, 5, 6, 7]], dtype=torch.int32, device="cuda"))


@pytest.mark.gpu
def test_cuda_page_attention_full_size_decode(rpa_lib):
    import ejkernel_b200 as ej

    b = make_workload("c2", num_seqs=128, device="cuda")
    kc, vc = _split(b)
    out = ej.page_attention(b.queries, kc, vc, b.context_lens, b.block_tables, attn_scale=b.softmax_scale)
    ref = ej.ragged_page_attention(*b.args(), softmax_scale=b.softmax_scale, cfg=ej.RaggedPageAttention().heuristic_cfg())
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
