"""The five benchmark workloads at FULL size on the GPU.  The CPU oracle cannot cover 4-23 GB of
KV in seconds, so each workload is checked (a) against the oracle on a seeded sample of its
sequences, whose pages are pulled out of the device pool, and (b) through size-independent
properties: renumbering the pool's pages leaves the output bit-identical, a constant V comes back
exactly, two runs agree bitwise, and a different split granularity agrees within tolerance; and (c) on
EVERY sequence against a plain-PyTorch float32 restatement of the operator that runs on the GPU and is
itself held against the oracle on a sample."""

import numpy as np
import pytest
import torch

from ejkernel_b200 import _cabi
from ejkernel_b200.utils import RaggedBatch, cdiv, make_workload
from oracle.rpa_oracle import compare, dense_reference
from tests.helpers import ATOL, REL_RMS, RTOL, run_cuda, status_word

pytestmark = pytest.mark.gpu


def _sample_to_host(b: RaggedBatch, seqs) -> RaggedBatch:
    """Sequences ``seqs`` of a device batch as a small host batch (pages compacted, ids renumbered)."""
    m = b.meta
    page = m["page_size"]
    kv_lens = [m["kv_lens"][s] for s in seqs]
    q_lens = [m["q_lens"][s] for s in seqs]
    npg = [cdiv(k, page) for k in kv_lens]
    ids = torch.cat([b.block_tables[s, :n] for s, n in zip(seqs, npg)]).long()
    pool = b.kv_pages[ids].cpu()
    tab = torch.zeros((len(seqs), max(npg)), dtype=torch.int32)
    off = 0
    for i, n in enumerate(npg):
        tab[i, :n] = torch.arange(off, off + n, dtype=torch.int32)
        off += n
    cu_dev = b.query_start_loc.cpu().tolist()
    q = torch.cat([b.queries[cu_dev[s] : cu_dev[s + 1]] for s in seqs]).cpu()
    cu = torch.zeros(len(seqs) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(q_lens), 0)
    return RaggedBatch(q, pool, torch.tensor(kv_lens, dtype=torch.int32), tab, cu,
                       torch.tensor([len(seqs)], dtype=torch.int32), b.softmax_scale, b.sliding_window,
                       b.logits_soft_cap, None, dict(m, kv_lens=kv_lens, q_lens=q_lens, total_tokens=int(cu[-1])))


@pytest.fixture(scope="module", params=["c2", "c3", "c4", "c5"])
def full(request, rpa_lib):
    b = make_workload(request.param, device="cuda")
    out = run_cuda(b)
    assert status_word(b) == 0
    yield request.param, b, out
    del b, out
    torch.cuda.empty_cache()


def test_sampled_sequences_match_oracle(full):
    name, b, out = full
    S = len(b.meta["kv_lens"])
    rng = np.random.default_rng(7)
    order = np.argsort(b.meta["kv_lens"])
    # shortest, longest, and a few random ones; for the mixed workload include a prefill chunk
    seqs = sorted({int(order[0]), int(order[-1]), *map(int, rng.choice(S, size=3, replace=False))} | ({S - 1} if name == "c3" else set()))
    if name == "c5":
        seqs = seqs[:3]
    host = _sample_to_host(b, seqs)
    want = dense_reference(*host.args(), **host.kwargs(), precision="fp32")
    cu = b.query_start_loc.cpu().tolist()
    got = torch.cat([out[cu[s] : cu[s + 1]] for s in seqs])
    r = compare(got, want, atol=ATOL, rtol=RTOL)
    assert r["finite"] and r["allclose"] and r["tight"] and r["max_rel_rms"] <= REL_RMS, (name, r)


def test_page_renumbering_is_bit_invariant(full):
    """Move every page to a new slot of the pool and rewrite the page table accordingly: the
    gathered bytes are the same, so the output must be bit-identical."""
    name, b, out = full
    P = b.kv_pages.shape[0]
    g = torch.Generator(device="cuda").manual_seed(3)
    perm = torch.randperm(P, device="cuda", generator=g)  # new_pool[perm[i]] = old_pool[i]
    b2 = b.to("cuda")
    new_pool = torch.empty_like(b.kv_pages)
    new_pool[perm] = b.kv_pages
    b2.kv_pages = new_pool
    b2.block_tables = perm[b.block_tables.long()].to(torch.int32)
    out2 = run_cuda(b2)
    del new_pool, b2
    assert torch.equal(out, out2), name


def test_rerun_is_bitwise_equal_and_split_granularity_is_within_tolerance(full):
    name, b, out = full
    assert torch.equal(out, run_cuda(b))
    old = _cabi.get_option("waves")
    try:
        _cabi.set_option("waves", 3 * old)
        out3 = run_cuda(b)
    finally:
        _cabi.set_option("waves", old)
    T = b.total_tokens
    r = compare(out3[:T], out[:T].float().cpu().numpy(), atol=ATOL, rtol=RTOL)
    assert r["allclose"] and r["tight"] and r["max_rel_rms"] <= REL_RMS, (name, r)


def test_constant_value_rows_come_back_exactly(rpa_lib):
    """softmax weights sum to one: with V_h = c_h everywhere the output row of head h is c_h,
    whatever the lengths, pages and splits (c_h a small integer, exact in bf16)."""
    b = make_workload("c2", device="cuda")
    Hkv = b.meta["num_kv_heads"]
    vals = torch.arange(1, Hkv + 1, device="cuda", dtype=torch.bfloat16)
    b.kv_pages[:, :, 1::2, :] = vals[None, None, :, None]
    out = run_cuda(b)[: b.total_tokens]
    G = b.meta["num_q_heads"] // Hkv
    want = vals.repeat_interleave(G)[None, :, None].expand_as(out)
    assert (out.float() - want.float()).abs().max().item() <= 2.0**-7 * Hkv  # one bf16 ulp of the largest value


def _float32_restatement_on_device(b: RaggedBatch) -> torch.Tensor:
    """Every sequence of a device batch with plain PyTorch float32 operations on the GPU: gather the sequence's pages,
    two einsums, scale, soft cap, causal / window mask, softmax -- the operator's definition
    (ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:105-177), independent of the CUDA kernels.  It is held
    against the CPU oracle on sampled sequences below, and the CUDA output is held against it on ALL of them."""
    m = b.meta
    page, Hkv = m["page_size"], m["num_kv_heads"]
    Hq, D = b.queries.shape[1], b.queries.shape[2]
    G = Hq // Hkv
    cu = b.query_start_loc.cpu().tolist()
    out = torch.zeros(b.queries.shape, dtype=torch.float32, device=b.queries.device)
    for s, (ql, kl) in enumerate(zip(m["q_lens"], m["kv_lens"])):
        if ql == 0:
            continue
        ids = b.block_tables[s, : cdiv(kl, page)].long()
        kv = b.kv_pages[ids].reshape(-1, 2 * Hkv, D)[:kl].float()
        k, v = kv[:, 0::2], kv[:, 1::2]  # [kl, Hkv, D]
        q = b.queries[cu[s] : cu[s] + ql].float().view(ql, Hkv, G, D)
        logits = torch.einsum("qhgd,khd->hgqk", q, k) * b.softmax_scale
        if b.logits_soft_cap is not None:
            logits = b.logits_soft_cap * torch.tanh(logits / b.logits_soft_cap)
        pos = (kl - ql + torch.arange(ql, device=q.device))[:, None]
        key = torch.arange(kl, device=q.device)[None, :]
        vis = key <= pos
        if b.sliding_window is not None:
            vis &= key > pos - b.sliding_window
        logits = logits.masked_fill(~vis[None, None], float("-inf"))
        p = torch.softmax(logits, dim=-1)
        out[cu[s] : cu[s] + ql] = torch.einsum("hgqk,khd->qhgd", p, v).reshape(ql, Hq, D)
        del kv, k, v, logits, p
    return out


def test_every_sequence_matches_a_float32_restatement_on_the_device(full):
    """Full coverage at full size: the sampled comparison against the CPU oracle pins a plain-PyTorch float32
    restatement that runs on the GPU, and the CUDA output is compared with that on every sequence of the workload."""
    name, b, out = full
    old_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = _float32_restatement_on_device(b)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_tf32
    torch.cuda.synchronize()
    T = b.total_tokens
    # (1) the restatement against the oracle on a sample (float32 against float32: tight)
    S = len(b.meta["kv_lens"])
    order = np.argsort(b.meta["kv_lens"])
    seqs = sorted({int(order[0]), int(order[S // 2]), S - 1})
    host = _sample_to_host(b, seqs)
    want = dense_reference(*host.args(), **host.kwargs(), precision="fp32")
    cu = b.query_start_loc.cpu().tolist()
    got = torch.cat([ref[cu[s] : cu[s + 1]] for s in seqs]).cpu().numpy()
    assert np.allclose(got, want, atol=2e-5, rtol=2e-4), (name, float(np.abs(got - want).max()))
    # (2) the CUDA output against the restatement, every sequence, per sequence (the tight criterion scales with
    # the rms of the expected rows, and short and long contexts differ tenfold)
    ref_np = ref[:T].cpu().numpy().astype(np.float64)
    out_np = out[:T].float().cpu().numpy()
    worst = 0.0
    for s in range(S):
        if cu[s + 1] == cu[s]:
            continue
        r = compare(out_np[cu[s] : cu[s + 1]], ref_np[cu[s] : cu[s + 1]], atol=ATOL, rtol=RTOL)
        assert r["finite"] and r["allclose"] and r["tight"] and r["max_rel_rms"] <= REL_RMS, (name, s, r)
        worst = max(worst, r["max_rel_rms"])
    assert torch.count_nonzero(out[T:]) == 0
    print(f"{name}: {S} sequences, worst error / rms {worst:.4f}")
