"""Regenerates tests/golden/rpa_golden.npz.

The reference holds no golden vectors for ``ragged_page_attention`` and cannot be run here (it
needs JAX), so these fixtures are produced by the CPU restatement ``oracle.rpa_oracle.dense_reference``
(float64) on seeded inputs:

  c1        -- benchmark workload 1 (8 decode sequences, Hq 8 / Hkv 2 / D 128, page 16)
  tpu_a     -- shape of test/kernels/_pallas/tpu/test_ragged_page_attention.py:465-508
               (query_start_loc [0,64,128], context_lens [64,96], page 16, 32 pages)
  tpu_b     -- shape of the same file :510-554 ([0,100,150,190,200], [128,64,192,96], 64 pages)
  win_cap   -- sliding window + soft cap + sinks on a small ragged batch

Only shapes and seeds come from the reference's tests; every value is computed.  Each entry stores
the expected output and a checksum of the generated inputs, so a drift of the input generator is
detected separately from a drift of the oracle.

    python tests/golden/make_golden.py
"""

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from ejkernel_b200.utils import make_ragged_batch, make_workload  # noqa: E402
from oracle.rpa_oracle import dense_reference  # noqa: E402


def cases():
    yield "c1", make_workload("c1")
    yield "tpu_a", make_ragged_batch([64, 64], [64, 96], num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16,
                                     pages_per_seq=8, num_pages=32, seed=11)
    yield "tpu_b", make_ragged_batch([100, 50, 40, 10], [128, 64, 192, 96], num_q_heads=8, num_kv_heads=2,
                                     head_dim=128, page_size=16, pages_per_seq=12, num_pages=64, seed=12)
    b = make_ragged_batch([1, 5, 1, 12], [300, 70, 2000, 150], num_q_heads=8, num_kv_heads=2, head_dim=64,
                          page_size=8, seed=13, sliding_window=100, logits_soft_cap=20.0)
    b.softmax_aux = torch.tensor([[0.5, -1.0], [2.0, 0.0]])
    yield "win_cap", b


def input_checksum(b) -> np.ndarray:
    q = b.queries.float().double().sum().item()
    kv = b.kv_pages.float().double().sum().item()
    idx = int(b.block_tables.long().sum() + b.context_lens.long().sum() + b.query_start_loc.long().sum())
    return np.array([q, kv, float(idx)])


def main():
    out = {}
    for name, b in cases():
        out[f"{name}.out"] = dense_reference(*b.args(), **b.kwargs()).astype(np.float32)
        out[f"{name}.chk"] = input_checksum(b)
    np.savez_compressed(Path(__file__).parent / "rpa_golden.npz", **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
