"""Regenerates tests/golden/rpa_reference_triton*.npz: outputs of the REFERENCE'S OWN kernels.

The reference's XLA implementation needs JAX, which is not installable where this was written.  Its
Triton implementation of the same operator, however, is two plain ``@triton.jit`` functions

    ejkernel/kernels/_triton/ragged_page_attention/_triton_impl_fwd.py:27-208   _ragged_paged_attn_fwd
    ejkernel/kernels/_triton/ragged_page_attention/_triton_impl_fwd.py:242-387  _ragged_paged_attn_qblock_fwd

whose module only needs ``jax`` for type annotations and ``ejkernel.callib.triton_call`` for the JAX
launch.  This script loads that file *by path from the reference checkout* (nothing of it is copied), with
empty stand-ins for those two imports, and launches the kernels directly on torch tensors with the grid,
strides, constexprs and output dtype that the reference's launchers compute (:485-613 for the default
kernel, :390-483 for the q-block kernel; restated in ``launch_default`` / ``launch_qblock`` below).

Two ways to execute them:

  --device cpu    Triton's interpreter (``TRITON_INTERPRET=1``): every ``tl.*`` operation of the reference
                  kernel runs as NumPy in float32.  Needs no GPU.  -> rpa_reference_triton.npz
  --device cuda   compiled by Triton for the GPU present (``tl.dot`` of float32 operands then runs as TF32).
                  -> rpa_reference_triton_cuda.npz

What these fixtures pin (the kernel states it in executable form): the K/V interleave of the combined-head
axis (K_h at 2h, V_h at 2h+1), token -> (page table entry, slot) addressing, q head -> kv head mapping,
the ``kv_len - q_len`` causal offset of a query row, the scale, the tail mask ``k < kv_len``, ragged batches.

Where the Triton kernels differ from the XLA implementation, and how the cases deal with it:
  * sliding window: the default kernel keeps keys ``[pos - W, pos]`` = W + 1 keys (:105-106,135), the XLA and
    Pallas implementations keep W.  The window case stores the window it gave to Triton *and* the equivalent
    XLA window (W + 1) a checker has to use.
  * soft cap: the default kernel computes ``a * tanh(logits * scale / a)`` with ``a = cap * log2(e)``
    (:161-167: the scaled logits are scaled a second time and the cap is stretched), not
    ``cap * tanh(logits / cap)``.  With ``softmax_scale = 1`` that is the XLA formula with cap ``a``; the soft-cap
    case therefore runs Triton with scale 1 and stores ``xla_logits_soft_cap = cap * log2(e)``.
  * the q-block kernel hard-codes ``SLIDING=True`` in its launcher (:441) and then starts at the tile of the
    block's own first key (:324-334), dropping earlier context; it is only right when the whole context lies
    in tile 0, so it is tried on a fresh-prefill case only (q_len <= 64, prior context < 32).  Under Triton 3.6
    it does not run at all: ``qpos[-1]`` (:318) indexes a tensor with an integer, which Triton rejects
    (interpreter: ``TypeError: 'int' object is not iterable``), and its soft cap calls ``tl.tanh`` (:358), which
    Triton 3.6 does not have.  The attempt and its error message are kept in the fixture file (``qblock_error``).
  * attention sinks are not implemented by either Triton kernel: unpinned.

    python tests/golden/make_reference_fixtures.py --device cpu --reference-root <checkout of erfanzar/ejkernel>
"""

from __future__ import annotations

import argparse
import importlib.util
import math
import os
import sys
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

REL = "ejkernel/kernels/_triton/ragged_page_attention/_triton_impl_fwd.py"
LOG2E = 1.4426950408889634


def load_reference_module(reference_root: Path):
    """Imports the reference's Triton file by path with stand-ins for ``jax`` and ``ejkernel.callib``."""
    import_names = ("jax", "jax.numpy", "ejkernel", "ejkernel.callib")
    saved = {n: sys.modules.get(n) for n in import_names}
    jax = types.ModuleType("jax")
    jnp = types.ModuleType("jax.numpy")
    jax.numpy, jax.Array = jnp, object
    jnp.float16, jnp.bfloat16, jnp.int32, jnp.float32 = "float16", "bfloat16", "int32", "float32"
    ej = types.ModuleType("ejkernel")
    callib = types.ModuleType("ejkernel.callib")
    callib.triton_call = None  # the JAX launcher; never called here
    ej.callib = callib
    sys.modules.update({"jax": jax, "jax.numpy": jnp, "ejkernel": ej, "ejkernel.callib": callib})
    try:
        path = reference_root / REL
        spec = importlib.util.spec_from_file_location("_reference_triton_rpa", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for n, m in saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
    return mod


def launch_default(mod, b, *, sliding_window=None, logits_soft_cap=None, softmax_scale=None, out_dtype=None,
                   block_m=128, block_npages=2):
    """``ragged_paged_attention_triton_call`` (:485-613) without JAX: same scalars, strides, constexprs, grid."""
    import torch
    import triton

    q, kv = b.queries, b.kv_pages
    T, Hq, D = map(int, q.shape)
    _P, page, C2, _ = map(int, kv.shape)
    page_size_tile = ((page + 15) // 16) * 16  # :507
    Hkv = C2 // 2
    S, pages_per_seq = map(int, b.block_tables.shape)
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else float(softmax_scale)  # :517-518
    if sliding_window is None:  # :520-534
        wl = wr = 0
        sliding = False
    else:
        wl, wr = int(sliding_window), 0
        sliding = wl > 0
    cap_val = 0.0 if logits_soft_cap is None else float(logits_soft_cap)  # :536-541
    block_dmodel = max(triton.next_power_of_2(D), 16)  # :545
    t_round = int(math.ceil(T / 128) * 128)  # :546
    out = torch.zeros((T, Hq, D), dtype=out_dtype or q.dtype, device=q.device)  # :554-557 (queries.dtype)
    lse = torch.zeros((Hq, t_round), dtype=torch.float32, device=q.device)
    grid = (triton.cdiv(T, block_m), Hq)  # :609
    mod._ragged_paged_attn_fwd[grid](
        q, kv, b.block_tables, b.context_lens, b.query_start_loc,
        scale, cap_val, T, S, Hq, Hkv, pages_per_seq, D, t_round, wl, wr,
        Hq * D, D, 1,  # q strides (:211-213)
        page * C2 * D, C2 * D, D, 1,  # kv strides (:216-218)
        pages_per_seq, 1,
        Hq * D, D, 1,
        t_round, 1,
        out, lse,  # triton_call appends the outputs after the inputs
        NUM_REPEATS=Hq // Hkv, IS_CAUSAL=True, SLIDING=bool(sliding), SOFTCAP=logits_soft_cap is not None,
        BLOCK_M=block_m, BLOCK_NPAGES=block_npages, BLOCK_DMODEL=block_dmodel, MAX_NUM_SEQS=S,
        PAGES_PER_SEQ=pages_per_seq, PAGE_SIZE=page, PAGE_SIZE_TILE=page_size_tile, COMPUTE_LSE=False,
    )
    return out


def launch_qblock(mod, b, *, out_dtype=None, block_q=64, tile_size=32):
    """``ragged_paged_attention_triton_call_qblock`` (:390-483) without JAX, soft cap off."""
    import torch

    q, kv = b.queries, b.kv_pages
    T, Hq, D = map(int, q.shape)
    _P, page, C2, _ = map(int, kv.shape)
    Hkv = C2 // 2
    S, pages_per_seq = map(int, b.block_tables.shape)
    scale = 1.0 / math.sqrt(D)  # :418-419
    head_padded = max(((D + 15) // 16) * 16, 16)  # :426
    n_blocks = T // block_q + S  # :428
    out = torch.zeros((T, Hq, D), dtype=out_dtype or q.dtype, device=q.device)
    mod._ragged_paged_attn_qblock_fwd[(n_blocks, Hq)](
        q, kv, b.block_tables, b.context_lens, b.query_start_loc,
        scale, 0.0, S, Hq, Hkv, pages_per_seq, page, D,
        Hq * D, D, 1,
        page * C2 * D, C2 * D, D, 1,
        pages_per_seq, 1,
        Hq * D, D, 1,
        out,
        NUM_REPEATS=Hq // Hkv, IS_CAUSAL=True, SLIDING=True, SOFTCAP=False,  # :437-446
        BLOCK_Q=block_q, TILE_SIZE=tile_size, HEAD_SIZE_PADDED=head_padded,
    )
    return out


def cases():
    """(name, batch, keywords for Triton's default kernel, keywords an XLA-semantics checker uses, q-block?)."""
    from ejkernel_b200.utils import make_ragged_batch, make_workload

    mk = lambda ql, kl, **kw: make_ragged_batch(ql, kl, num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, **kw)
    # shapes of test/kernels/_pallas/tpu/test_ragged_page_attention.py:465-508 and :510-554
    yield "tpu_a", mk([64, 64], [64, 96], pages_per_seq=8, num_pages=32, seed=11), {}, {}, False
    yield "tpu_b", mk([100, 50, 40, 10], [128, 64, 192, 96], pages_per_seq=12, num_pages=64, seed=12), {}, {}, False
    yield "c1", make_workload("c1"), {}, {}, False  # benchmark workload 1: 8 decode sequences
    yield ("mixed_gqa4", make_ragged_batch([1, 7, 1, 33], [200, 7, 17, 250], num_q_heads=8, num_kv_heads=2, head_dim=64,
                                          page_size=8, seed=21), {}, {}, False)
    yield ("window", mk([1, 20, 1], [230, 100, 40], seed=22), dict(sliding_window=63), dict(sliding_window=64), False)
    yield ("softcap", mk([1, 9, 30], [150, 60, 30], seed=23, softmax_scale=1.0),
           dict(logits_soft_cap=4.0, softmax_scale=1.0), dict(logits_soft_cap=4.0 * LOG2E, softmax_scale=1.0), False)
    yield "fresh_prefill", mk([64, 17, 40], [64, 17 + 31, 40 + 5], seed=24), {}, {}, True
    # few sequences x few pages: what Triton can also COMPILE in minutes (the kernel unrolls both loops)
    yield ("small_window", mk([1, 6], [70, 40], pages_per_seq=5, seed=25), dict(sliding_window=20), dict(sliding_window=21),
           False)
    yield ("small_softcap", mk([1, 5], [33, 64], pages_per_seq=4, seed=26, softmax_scale=1.0),
           dict(logits_soft_cap=3.0, softmax_scale=1.0), dict(logits_soft_cap=3.0 * LOG2E, softmax_scale=1.0), False)


# what --device cuda runs: at most 16 unrolled (sequence, page) bodies per kernel
COMPILED_CASES = ("tpu_a", "fresh_prefill", "small_window", "small_softcap")


def bits(t):
    import torch

    return t.contiguous().view(torch.int16).cpu().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", choices=("cpu", "cuda"), default="cpu")
    ap.add_argument("--reference-root", default=os.environ.get("EJK_REFERENCE_ROOT"),
                    help="checkout of erfanzar/ejkernel (v0.0.16) to load the Triton kernels from; or set EJK_REFERENCE_ROOT")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    if not a.reference_root:
        ap.error("--reference-root (or EJK_REFERENCE_ROOT) must name a checkout of the reference")
    if a.device == "cpu":
        os.environ["TRITON_INTERPRET"] = "1"  # must be set before triton is imported
    import numpy as np
    import torch
    import triton

    mod = load_reference_module(Path(a.reference_root))
    out = {"how": np.array(f"triton {triton.__version__}, "
                           + ("interpreter (NumPy float32)" if a.device == "cpu"
                              else f"compiled for {torch.cuda.get_device_name(0)} (tl.dot float32 -> TF32)"))}
    dst = a.out or str(Path(__file__).parent / ("rpa_reference_triton.npz" if a.device == "cpu"
                                                 else "rpa_reference_triton_cuda.npz"))
    for name, b, tri_kw, xla_kw, qblock in cases():
        if a.device == "cuda" and name not in COMPILED_CASES:
            continue  # e.g. 4 sequences x 12 pages unrolled at compile time: Triton needs more than five minutes for it
        T = b.total_tokens
        b = b.to(a.device)
        b.queries = b.queries[:T].contiguous()
        try:
            o16 = launch_default(mod, b, **tri_kw)  # the launcher's own output dtype (= queries.dtype)
            o32 = launch_default(mod, b, out_dtype=torch.float32, **tri_kw)  # same kernel, unrounded store
        except Exception as e:
            if a.device != "cuda":
                raise
            # e.g. the soft-cap branch declares a constexpr inside the unrolled page loop (:162), which the compiler
            # rejects from the second page on ("LOG2_CONST is already defined"); the interpreter does not mind
            out[f"{name}.error"] = np.array(f"{type(e).__name__}: {e}"[-400:])
            print(name, "did not compile:", out[f"{name}.error"], flush=True)
            np.savez_compressed(dst, **out)
            continue
        out[f"{name}.out"] = bits(o16)
        out[f"{name}.out_f32"] = o32.cpu().numpy()
        if qblock:
            try:
                out[f"{name}.out_qblock"] = bits(launch_qblock(mod, b))
                out[f"{name}.out_qblock_f32"] = launch_qblock(mod, b, out_dtype=torch.float32).cpu().numpy()
            except Exception as e:  # recorded, not hidden: the fixture file says why this kernel has no outputs
                out["qblock_error"] = np.array(f"{type(e).__name__}: {e}"[:500])
                print("q-block kernel did not run:", out["qblock_error"])
        if a.device == "cuda":  # same seeded inputs as the interpreter file, which holds them
            print(name, tuple(o16.shape), "rms", float(o32.float().pow(2).mean().sqrt()), flush=True)
            np.savez_compressed(dst, **out)  # after every case: a compile that runs out of time loses only itself
            continue
        out[f"{name}.queries"] = bits(b.queries)
        # pages no table entry of a live sequence names are never read (the kernel masks them): stored as zeros
        live = torch.zeros(b.kv_pages.shape[0], dtype=torch.bool)
        for s_, n_ in enumerate(-(-b.context_lens.cpu()[: int(b.num_seqs[0])] // b.kv_pages.shape[1])):
            live[b.block_tables[s_, : int(n_)].cpu().long()] = True
        out[f"{name}.kv_pages"] = bits(b.kv_pages.cpu() * live[:, None, None, None])
        out[f"{name}.context_lens"] = b.context_lens.cpu().numpy()
        out[f"{name}.block_tables"] = b.block_tables.cpu().numpy()
        out[f"{name}.query_start_loc"] = b.query_start_loc.cpu().numpy()
        out[f"{name}.num_seqs"] = b.num_seqs.cpu().numpy()
        out[f"{name}.softmax_scale"] = np.float64(xla_kw.get("softmax_scale", b.softmax_scale))
        out[f"{name}.sliding_window"] = np.int64(xla_kw.get("sliding_window", 0))  # 0 = none
        out[f"{name}.logits_soft_cap"] = np.float64(xla_kw.get("logits_soft_cap", 0.0))  # 0 = none
        print(name, tuple(o16.shape), "rms", float(o32.float().pow(2).mean().sqrt()))
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
