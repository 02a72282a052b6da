"""Host-side pieces of ``bench.py`` (no GPU): the two arms describe the same workload, the weak-scaling batch repeats
the single-GPU lengths, the work counts behind the rooflines, and the parity sample really checks."""

import argparse
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
bench = importlib.util.module_from_spec(spec)
sys.modules["bench_module"] = bench
spec.loader.exec_module(bench)

from ejkernel_b200.utils import algorithmic_kv_bytes, make_workload  # noqa: E402
from oracle.rpa_oracle import dense_reference  # noqa: E402


def _args(**kw):
    a = argparse.Namespace(workload="c2", num_seqs=None, len_scale=1.0, strong=False, kv_dtype="bf16")
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_both_arms_print_the_same_config():
    # the config object is a function of the command line only
    for world in (1, 2, 8):
        assert bench.make_config(_args(), world) == bench.make_config(_args(), world)
    c1, c8 = bench.make_config(_args(), 1), bench.make_config(_args(), 8)
    assert c1["workload"] == "c2: 256 seqs" and c8["workload"] == "c2: 2048 seqs"
    assert "4.4 GiB per GPU" in c1["l2"] and "4.4 GiB per GPU" in c8["l2"]  # weak scaling: the same bytes per GPU
    assert "e4m3" in bench.make_config(_args(kv_dtype="e4m3"), 1)["workload"]


def test_weak_batch_repeats_the_single_gpu_lengths():
    q1, kv1, shape1, _ = bench.workload_spec("c2")
    q4, kv4, shape4, _ = bench.workload_spec("c2", tile=4)
    assert len(kv4) == 4 * len(kv1) and np.array_equal(kv4.reshape(4, -1), np.tile(kv1, (4, 1)))
    assert shape1 == shape4 and np.array_equal(q4, np.ones(1024, dtype=np.int64))


def test_work_counts_split_decode_bytes_and_prefill_flops():
    b = make_workload("c3", num_seqs=10, len_scale=0.05)
    w = bench.work_counts(b)
    assert w["decode_kv_bytes"] + w["prefill_kv_bytes"] == algorithmic_kv_bytes(b)
    m = b.meta
    flops = 0
    for ql, kl in zip(m["q_lens"], m["kv_lens"]):
        if ql > 1:
            flops += 4 * m["num_q_heads"] * m["head_dim"] * (ql * (kl - ql) + ql * (ql + 1) // 2)
    assert w["prefill_flops"] == flops and flops > 0
    win = make_workload("c4", num_seqs=3, len_scale=0.1)  # windowed decode: only the keys inside the window count
    assert bench.work_counts(win)["decode_kv_bytes"] == algorithmic_kv_bytes(win)


def test_parity_sample_accepts_the_oracle_and_rejects_a_wrong_row():
    b = make_workload("c3", num_seqs=10, len_scale=0.05)
    good = torch.from_numpy(dense_reference(*b.args(), **b.kwargs())).to(torch.bfloat16)
    r = bench.parity_sample(b, good)
    assert r["ok"] and r["checked"] == 4 and 0 in r["seqs"]
    bad = good.clone()
    bad[0] += 0.5  # sequence 0 is always among the sampled ones
    assert not bench.parity_sample(b, bad)["ok"]
    # an e4m3 pool is checked against the weight-rounding bound
    b8 = make_workload("c2", num_seqs=6, len_scale=0.05, kv_dtype=torch.float8_e4m3fn)
    good8 = torch.from_numpy(dense_reference(*b8.args(), **b8.kwargs())).to(torch.bfloat16)
    assert bench.parity_sample(b8, good8)["ok"]
    bad8 = good8.clone()
    bad8[0] = -bad8[0] + 1.0
    assert not bench.parity_sample(b8, bad8)["ok"]
