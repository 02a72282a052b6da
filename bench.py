#!/usr/bin/env python
"""Benchmark of the ragged paged attention hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload c2]

One "step" is one ``ragged_page_attention`` call over one synthetic batch.  At N = 1 the
workload is the Llama-3-8B-shaped decode batch ("c2": 256 sequences, q_len 1, kv_len uniform in
[128, 8192], Hq 32 / Hkv 8 / D 128, page 16, bf16).  At N > 1 the batch is those 256 sequences'
lengths repeated N times (256*N sequences) and every rank serves Hkv/N kv heads of all of them
(KV-head sharding, no collective in the data path), so the bytes per GPU are exactly those of N = 1:
weak scaling.  ``--workload`` / ``--num-seqs`` / ``--len-scale`` select other cases (used for profiling
small captures; ``--strong`` keeps the batch fixed and splits its kv heads).

Prints ONE JSON line (rank 0):  value = query tokens/s of the whole job with inputs resident in
HBM; ``hbm_tbs`` = algorithmic KV bytes / time; ``roofline`` for the attention kernel timed with
CUDA events inside the run; ``e2e`` = the same metric through the public operator with the step's
inputs copied from pinned host memory and the output copied back, every step; ``cpu_baseline`` =
the CPU restatement of the reference's XLA algorithm timed on this host's cores on a bounded
sample of the same batch.  ``--impl reference`` times only that CPU restatement.

Outside the headline's timed region the default run also measures the other benchmark workloads and
checks results:
  ``per_workload`` (N = 1)  c2 on a float8 (e4m3) KV pool; c3 (mixed prefill + decode: the tensor-tile kernel against the bf16 tensor peak and the
                            split-KV kernel against the HBM peak, each timed on its own), c4 (window + soft cap,
                            head_dim 256) and c5 (long context), each with step time, kernel time and roofline;
  ``c5_strong`` (N > 1)     the SAME 64 long-context sequences with Hkv/N kv heads per rank: strong scaling;
  ``parity_sample``         every rank compares a few sequences of every batch it ran with the CPU oracle
                            (float32 contractions) and the results and status words of all ranks are reduced.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "paged_attn_query_tokens_per_s"
UNIT = "tokens/s"
# DRAM traffic of the attention kernel relative to its algorithmic KV bytes, from an ncu capture of a
# 48-sequence slice of the same workload: (dram__bytes_read.sum 788.25 MB + dram__bytes_write.sum 5.55 MB) over
# 786.06 MB of KV.  Traffic grows in proportion to the KV bytes (every byte is read once), so the ratio scales.
NCU_TRAFFIC_RATIO = {"c2": (788.25 + 5.55) / 786.06}
BASE_SEQS = {"c1": 8, "c2": 256, "c3": 68, "c4": 128, "c5": 64}
PREFILL_ROWS = 32  # default of the library option "prefill_rows": sequences with q_len * G >= this use tensor tiles


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--num-seqs", type=int, default=None, help="override the number of sequences (per GPU-equivalent)")
    ap.add_argument("--len-scale", type=float, default=1.0)
    ap.add_argument("--strong", action="store_true", help="keep the batch fixed and split its kv heads over the ranks")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--waves", type=int, default=None)
    ap.add_argument("--path", type=int, default=None)
    ap.add_argument("--headline-only", action="store_true", help="skip per_workload / c5_strong / parity_sample")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="on ONE GPU, run the shard one rank of an N-way kv-head split would get (profiling aid)")
    ap.add_argument("--fused-merge", type=int, default=None)
    ap.add_argument("--prefill-share", type=int, default=None, help="library option prefill_share (percent, 0 = off)")
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "e4m3"], help="dtype of the KV pool of the headline batch")
    return ap.parse_args()


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs
    (read-only queries)."""

    BAD = {
        0x8: "hw_slowdown",
        0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown",
    }
    NOTE = {0x4: "sw_power_cap", 0x80: "hw_power_brake", 0x2: "applications_clocks_setting"}

    def __init__(self, index: int, period_s: float = 0.02):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        self.period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            # CUDA_VISIBLE_DEVICES may remap indices; match by UUID when possible
            uuid = torch.cuda.get_device_properties(index).uuid
            self.h = None
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if str(uuid) in u:
                    self.h = h
                    break
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in {**self.BAD, **self.NOTE}.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# --------------------------------------------------------------------------------------------
# CPU restatement of the reference (the "reference arm" and the cpu_baseline leg)
# --------------------------------------------------------------------------------------------
def cpu_reference_rate(batch_cpu_sample, seconds: float, steps: int = 1, warmup: int = 0):
    """Times oracle.blocked_as_written (the reference's XLA algorithm as written) on all host
    threads over the given sample of sequences.  Returns (tokens/s, GB/s of algorithmic KV bytes,
    ms per pass, cores)."""
    from ejkernel_b200.utils import algorithmic_kv_bytes
    from oracle.rpa_oracle import blocked_as_written

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    b = batch_cpu_sample
    for _ in range(warmup):
        blocked_as_written(*b.args(), **b.kwargs())
    t0 = time.perf_counter()
    n = 0
    while True:
        blocked_as_written(*b.args(), **b.kwargs())
        n += 1
        if n >= steps or time.perf_counter() - t0 > seconds:
            break
    dt = (time.perf_counter() - t0) / n
    toks = b.total_tokens
    return toks / dt, algorithmic_kv_bytes(b) / dt / 1e9, dt * 1e3, cores


def compact_sample(batch, n_seqs: int):
    """First ``n_seqs`` sequences of a (device) batch with their pages gathered into a small pool
    on the host, page ids renumbered; lets the CPU leg run without copying a multi-GB pool."""
    from ejkernel_b200.utils import RaggedBatch, cdiv

    m = batch.meta
    n = min(n_seqs, len(m["kv_lens"]))
    page = m["page_size"]
    kv_lens, q_lens = m["kv_lens"][:n], m["q_lens"][:n]
    npg = [cdiv(k, page) for k in kv_lens]
    tab = batch.block_tables[:n].clone()
    ids = torch.cat([tab[s, : npg[s]] for s in range(n)]).long()
    pool = batch.kv_pages[ids].cpu()
    new_tab = torch.zeros((n, tab.shape[1]), dtype=torch.int32)
    off = 0
    for s in range(n):
        new_tab[s, : npg[s]] = torch.arange(off, off + npg[s], dtype=torch.int32)
        off += npg[s]
    T = int(sum(q_lens))
    cu = torch.zeros(n + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(q_lens), 0)
    q = batch.queries[:T].cpu()
    # 8 trailing rows keep the as-written 8-row block of the last sequence inside the array
    q = torch.cat([q, torch.zeros((16, *q.shape[1:]), dtype=q.dtype)], 0)
    meta = dict(m)
    meta.update(kv_lens=kv_lens, q_lens=q_lens, total_tokens=T, num_pages=pool.shape[0])
    return RaggedBatch(
        q, pool, torch.tensor(kv_lens, dtype=torch.int32), new_tab, cu, torch.tensor([n], dtype=torch.int32),
        batch.softmax_scale, batch.sliding_window, batch.logits_soft_cap, None, meta,
    )


def pick_sample_size(batch, seconds: float) -> int:
    """Sequences whose as-written CPU pass should take roughly ``seconds`` (assumes ~1.5 GB/s of
    KV traffic on the host; the real rate is what gets reported)."""
    m = batch.meta
    per_tok = 2 * m["num_kv_heads"] * m["head_dim"] * 2
    budget = seconds * 1.5e9
    acc, n = 0, 0
    for k in m["kv_lens"]:
        acc += k * per_tok
        n += 1
        if acc > budget:
            break
    return max(1, n)


# --------------------------------------------------------------------------------------------
# workloads, configs, work counts
# --------------------------------------------------------------------------------------------
def workload_spec(name: str, *, num_seqs=None, len_scale=1.0, tile: int = 1):
    """Lengths and static shape of a named workload.  ``tile`` repeats the sequences' lengths that many times
    (the weak-scaling batch: the N = 1 draw repeated, so every GPU gets exactly the bytes of the N = 1 run)."""
    from ejkernel_b200.utils import workload_lengths

    q_l, kv_l, shape, extra = workload_lengths(name, num_seqs=num_seqs, len_scale=len_scale)
    if tile > 1:
        q_l, kv_l = np.tile(q_l, tile), np.tile(kv_l, tile)
    return q_l, kv_l, shape, extra


def make_config(args, world: int) -> dict:
    """The ``config`` object of the JSON line; a function of the command line only, so both arms print the same."""
    n = args.num_seqs or BASE_SEQS[args.workload]
    weak = not args.strong
    total = n * (world if weak else 1)
    q_l, kv_l, shape, _ = workload_spec(args.workload, num_seqs=n, len_scale=args.len_scale, tile=world if weak else 1)
    pages = int(sum(-(-int(k) // shape["page_size"]) for k in kv_l))
    pool = int(shape.get("num_pages") or -(-pages * 11 // 10)) * shape["page_size"] * 2 * shape["num_kv_heads"] * shape["head_dim"] * 2
    pool_rank = pool // world
    return {
        "workload": f"{args.workload}: {total} seqs" + (f" x len_scale {args.len_scale}" if args.len_scale != 1.0 else "")
                    + (" on a float8 e4m3 KV pool" if getattr(args, "kv_dtype", "bf16") == "e4m3" else ""),
        "partition": (f"kv-head sharded over {world} GPU(s), {'weak: the N=1 lengths repeated N times' if weak else 'strong'}"
                      if world > 1 else "single GPU"),
        "l2": (f"KV pool {pool_rank / 2**30:.1f} GiB per GPU, far larger than the 126 MB L2: no flush needed"
               if pool_rank >= 4 * 126 * (1 << 20) else
               f"KV pool {pool_rank / 2**20:.0f} MiB per GPU <= 4x L2: 256 MiB written between timed steps to flush L2"),
    }


def work_counts(batch) -> dict:
    """Algorithmic work of one call on this rank's shard: KV bytes of the decode rows (served by the split-KV
    kernel), KV bytes and FLOPs (4 * D per (row, visible key) pair) of the sequences served by tensor tiles."""
    m = batch.meta
    G = m["num_q_heads"] // m["num_kv_heads"]
    per_tok = 2 * m["num_kv_heads"] * m["head_dim"] * batch.kv_pages.element_size()
    W = batch.sliding_window
    dec_bytes = pre_bytes = 0
    pre_flops = 0
    for ql, kl in zip(m["q_lens"], m["kv_lens"]):
        if ql == 0:
            continue
        lo = max(0, (kl - ql) - W + 1) if W else 0
        if ql * G >= PREFILL_ROWS:
            pre_bytes += (kl - lo) * per_tok
            for r in range(ql):
                pos = kl - ql + r
                vis = pos + 1 - (max(0, pos - W + 1) if W else 0)
                pre_flops += 4 * m["num_q_heads"] * m["head_dim"] * vis
        else:
            dec_bytes += (kl - lo) * per_tok
    return {"decode_kv_bytes": dec_bytes, "prefill_kv_bytes": pre_bytes, "prefill_flops": pre_flops}


def load_peaks():
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        d = json.loads(pk.read_text())
        return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


# --------------------------------------------------------------------------------------------
# parity sample: a few sequences of a device batch against the CPU oracle (checker only, never timed)
# --------------------------------------------------------------------------------------------
def parity_sample(batch, out, n_check: int = 4) -> dict:
    from ejkernel_b200.utils import RaggedBatch, cdiv
    from oracle.rpa_oracle import compare, dense_reference

    m = batch.meta
    S = len(m["kv_lens"])
    if S == 0:
        return {"ok": True, "checked": 0, "max_err_over_rms": 0.0}
    # first, last, and evenly spaced sequences in between; always the longest multi-token sequence too
    ids = sorted({0, S - 1, *[(S * i) // n_check for i in range(1, n_check)][: max(0, n_check - 2)]})
    multi = [s for s in range(S) if m["q_lens"][s] > 1]
    if multi:
        ids = sorted(set(ids[: n_check - 1]) | {max(multi, key=lambda s: m["kv_lens"][s])})
    page = m["page_size"]
    npg = [cdiv(m["kv_lens"][s], page) for s in ids]
    pool_ids = torch.cat([batch.block_tables[s, :n].long() for s, n in zip(ids, npg)])
    pool = batch.kv_pages[pool_ids].cpu()
    tab = torch.zeros((len(ids), batch.block_tables.shape[1]), dtype=torch.int32)
    off = 0
    for i, n in enumerate(npg):
        tab[i, :n] = torch.arange(off, off + n, dtype=torch.int32)
        off += n
    cu_dev = batch.query_start_loc.cpu()
    rows = torch.cat([torch.arange(int(cu_dev[s]), int(cu_dev[s + 1])) for s in ids])
    q_lens = [m["q_lens"][s] for s in ids]
    cu = torch.zeros(len(ids) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(q_lens), 0)
    sub = RaggedBatch(batch.queries[rows.to(batch.queries.device)].cpu(), pool,
                      torch.tensor([m["kv_lens"][s] for s in ids], dtype=torch.int32), tab, cu,
                      torch.tensor([len(ids)], dtype=torch.int32), batch.softmax_scale, batch.sliding_window,
                      batch.logits_soft_cap, None, {})
    got = out[rows.to(out.device)].float().cpu().numpy()
    if batch.kv_pages.element_size() == 1:
        # e4m3 cache: the probabilities enter P.V as e4m3, each weight within 2^-4 relative, so an output element is
        # within 2^-4 * (P @ |V|) of the exact one (plus the bf16 rounding of the output)
        want, wb = dense_reference(*sub.args(), **sub.kwargs(), precision="fp32", return_weight_bound=True)
        err = np.abs(got - want)
        ok = bool(np.isfinite(got).all() and (err <= 2.0**-4 * 1.02 * wb + 2.0**-8 * np.abs(want) + 1e-3).all())
        rms = float(np.sqrt(np.mean(want * want)))
        return {"ok": ok, "checked": len(ids), "seqs": ids, "max_err_over_rms": float(err.max() / max(rms, 1e-30))}
    want = dense_reference(*sub.args(), **sub.kwargs(), precision="fp32")
    r = compare(got, want, atol=2e-2, rtol=2e-2)
    return {"ok": bool(r["finite"] and r["allclose"] and r["tight"]), "checked": len(ids), "seqs": ids,
            "max_err_over_rms": r["max_rel_rms"]}


# --------------------------------------------------------------------------------------------
def emit(line: dict, out_fd: int) -> None:
    os.write(out_fd, (json.dumps(line) + "\n").encode())


def main():
    args = parse_args()
    # The contract is ONE line on stdout.  Libraries loaded below may write there too (NCCL prints its version to stdout
    # when NCCL_DEBUG is set), so everything but the result line is sent to stderr: file descriptor 1 is pointed at
    # stderr for the run, and the JSON line goes to the original stdout.
    sys.stdout.flush()
    try:
        out_fd = os.dup(1)
        os.dup2(2, 1)
    except OSError:  # no usable stderr: leave stdout alone
        out_fd = 1
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world

    from ejkernel_b200.utils import WORKLOADS, algorithmic_kv_bytes, make_ragged_batch

    n_seqs = args.num_seqs or BASE_SEQS[args.workload]
    weak = not args.strong
    total_seqs = n_seqs * (world if weak else 1)
    config = make_config(args, world)

    def build(name, device, kv_head_slice, *, num_seqs=None, len_scale=1.0, tile=1, pad_query_rows=0, kv_dtype=None):
        q_l, kv_l, shape, extra = workload_spec(name, num_seqs=num_seqs, len_scale=len_scale, tile=tile)
        return make_ragged_batch(q_l, kv_l, dtype=torch.bfloat16, device=device, seed=1000 + WORKLOADS.index(name) + 1,
                                 kv_head_slice=kv_head_slice, pad_query_rows=pad_query_rows, kv_dtype=kv_dtype,
                                 **shape, **extra)

    # ---------------- reference arm: CPU restatement only, rank 0 only ----------------
    if args.impl == "reference":
        if rank != 0:
            return
        # build only the sampled sequences on the host (the full pool is never needed)
        q_l, kv_l, shape, extra = workload_spec(args.workload, num_seqs=n_seqs, len_scale=args.len_scale,
                                                tile=world if weak else 1)
        per_tok = 2 * shape["num_kv_heads"] * shape["head_dim"] * 2
        n = 0
        acc = 0
        for k in kv_l:
            acc += int(k) * per_tok
            n += 1
            if acc > 1.2e9:
                break
        sub_shape = dict(shape)
        sub_shape.pop("num_pages", None)
        b = make_ragged_batch(q_l[:n], kv_l[:n], dtype=torch.bfloat16, device="cpu",
                              seed=1000 + WORKLOADS.index(args.workload) + 1, pad_query_rows=16, **sub_shape, **extra)
        for _ in range(min(args.warmup, 1)):
            cpu_reference_rate(b, 1e9, steps=1)
        steps_done = max(1, min(args.steps, 5))
        tps, gbs, ms, cores = cpu_reference_rate(b, 1e9, steps=steps_done)
        sample = f"first {n} of {total_seqs} sequences of the batch, {steps_done} pass(es)"
        line = {
            "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps_done, "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak" if weak else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config, "hbm_tbs": gbs / 1e3,
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        emit(line, out_fd)
        return

    # ---------------- our arm ----------------
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from ejkernel_b200 import _cabi
    from ejkernel_b200.kernels._cuda.ragged_page_attention import RpaWorkspace, ragged_page_attention_into
    from ejkernel_b200.kernels._cuda.ragged_page_attention._interface import _shape_of
    from ejkernel_b200.modules import ragged_page_attention as public_op

    _cabi.load()
    if args.waves:
        _cabi.set_option("waves", args.waves)
    if args.path is not None:
        _cabi.set_option("path", args.path)
    if args.fused_merge is not None:
        _cabi.set_option("fused_merge", args.fused_merge)
    if args.prefill_share is not None:
        _cabi.set_option("prefill_share", args.prefill_share)
    hbm_peak, tensor_peak, peak_src = load_peaks()

    def head_slice_for(name):
        Hkv = {"c1": 2}.get(name, 8)
        if Hkv % world:
            raise SystemExit(f"num_kv_heads={Hkv} cannot be split over {world} ranks")
        per = Hkv // world
        if world == 1 and args.shard_of > 1:
            return (0, Hkv // args.shard_of)
        return (rank * per, (rank + 1) * per) if world > 1 else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world > 1:
            t = torch.tensor([x], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return x

    def measure(batch, steps: int, warmup: int, clock=None):
        """Device-timed steps of one resident batch through the C ABI (caller-owned output and workspace), then
        the same call with CUDA events around each kernel.  Returns the record and the output of the last call."""
        ws = RpaWorkspace(_shape_of(batch.queries, batch.kv_pages, batch.block_tables), dev)
        out = torch.empty_like(batch.queries)
        kw = dict(softmax_scale=batch.softmax_scale, sliding_window=batch.sliding_window,
                  logits_soft_cap=batch.logits_soft_cap)

        def step():
            ragged_page_attention_into(out, ws, *batch.args(), **kw)

        for _ in range(max(3, warmup)):
            step()
        barrier()
        launches = _cabi.load().ejk_rpa_last_launch_count()
        pool_bytes = batch.kv_pages.numel() * batch.kv_pages.element_size()
        flush = pool_bytes < 4 * 126 * (1 << 20)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        if not flush:  # inputs far larger than L2
            e0.record()
            for _ in range(steps):
                step()
            e1.record()
            barrier()
            ms_total = e0.elapsed_time(e1)
        else:  # L2 overwritten between steps, each step timed on its own
            scrub = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            for a, b_ in evs:
                scrub.fill_(1)
                a.record()
                step()
                b_.record()
            barrier()
            ms_total = sum(a.elapsed_time(b_) for a, b_ in evs)
            del scrub
        ms_step = max_over_ranks(ms_total) / steps
        status = int(ws.status.item())
        _cabi.set_option("profile", 1)
        prof = []
        for _ in range(min(steps, 50)):
            step()
            prof.append(_cabi.profile_read_kernels())
        _cabi.set_option("profile", 0)
        plan_ms, prefill_ms, splitkv_ms, merge_ms = (max_over_ranks(statistics.mean(c)) for c in zip(*prof))
        step()
        torch.cuda.synchronize()
        rec = {"ms_per_step": ms_step, "plan_ms": plan_ms, "prefill_ms": prefill_ms, "splitkv_ms": splitkv_ms,
               "merge_ms": merge_ms, "status_word": status, "launches_per_step": launches, "step": step, "kw": kw}
        return rec, out

    def rooflines(batch, rec) -> dict:
        """Per kernel: algorithmic work of this rank's shard over the kernel's own CUDA-event time."""
        w = work_counts(batch)
        r = {}
        if rec["splitkv_ms"] > 0 and w["decode_kv_bytes"]:
            a = w["decode_kv_bytes"] / (rec["splitkv_ms"] * 1e-3) / 1e9
            r["splitkv"] = {"bound": "hbm", "kernel": "rpa_splitkv_tma_kernel (gather + QK^T + softmax + PV)", "achieved": a,
                            "peak": hbm_peak, "unit": "GB/s", "frac": a / hbm_peak, "frac_of_nominal_8tbs": a / 8000.0,
                            "peak_source": peak_src, "kernel_ms": rec["splitkv_ms"], "kv_bytes": w["decode_kv_bytes"]}
        if rec["prefill_ms"] > 0 and w["prefill_flops"]:
            a = w["prefill_flops"] / (rec["prefill_ms"] * 1e-3) / 1e12
            r["prefill"] = {"bound": "tensor", "kernel": "rpa_prefill_tc_kernel (tcgen05 tiles)", "achieved": a,
                            "peak": tensor_peak, "unit": "TFLOP/s", "frac": a / tensor_peak, "peak_source": peak_src,
                            "kernel_ms": rec["prefill_ms"], "flops": w["prefill_flops"]}
        return r

    parity = {"ok": True, "checked": 0, "max_err_over_rms": 0.0, "batches": []}

    def add_parity(name, batch, out):
        if args.headline_only:
            return
        p = parity_sample(batch, out)
        parity["ok"] = parity["ok"] and p["ok"]
        parity["checked"] += p["checked"]
        parity["max_err_over_rms"] = max(parity["max_err_over_rms"], p["max_err_over_rms"])
        parity["batches"].append(name)

    # ---------------- headline: resident inputs, device timed ----------------
    batch = build(args.workload, dev, head_slice_for(args.workload), num_seqs=n_seqs, len_scale=args.len_scale,
                  tile=world if weak else 1, kv_dtype=torch.float8_e4m3fn if args.kv_dtype == "e4m3" else None)
    T = batch.total_tokens
    kv_bytes_rank = algorithmic_kv_bytes(batch)
    with ClockSampler(local_rank) as clk:
        rec, out = measure(batch, args.steps, args.warmup)
    ms_step = rec["ms_per_step"]
    status_all = rec["status_word"]
    add_parity(args.workload, batch, out)
    k_ms = rec["prefill_ms"] + rec["splitkv_ms"]
    kw = rec["kw"]

    # ---------------- end-to-end leg: public operator, host buffers ----------------
    e2e, e2e_zero_copy = None, None
    if not args.no_e2e:
        # The step's inputs live in ONE pinned host buffer and ONE device buffer (each operand a 256-byte
        # aligned view), so a step costs one host->device copy instead of five.
        srcs = (batch.queries, batch.context_lens, batch.block_tables, batch.query_start_loc, batch.num_seqs)
        offs, total = [], 0
        for t in srcs:
            offs.append(total)
            total += (t.numel() * t.element_size() + 255) // 256 * 256
        host_buf = torch.empty(total, dtype=torch.uint8).pin_memory()
        dev_buf = torch.empty(total, dtype=torch.uint8, device=dev)

        def views(buf):
            return [buf[o:o + t.numel() * t.element_size()].view(t.dtype).view(t.shape) for o, t in zip(offs, srcs)]

        for hv, t in zip(views(host_buf), srcs):
            hv.copy_(t.cpu())
        dev_in = views(dev_buf)
        host_out = torch.empty(batch.queries.shape, dtype=batch.queries.dtype).pin_memory()
        h2d = total  # bytes actually copied per step (operands padded to 256 B)
        d2h = host_out.numel() * host_out.element_size()

        def e2e_step():
            dev_buf.copy_(host_buf, non_blocking=True)
            o = public_op(dev_in[0], batch.kv_pages, dev_in[1], dev_in[2], dev_in[3], dev_in[4], **kw)
            host_out.copy_(o, non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the host reads the result every step

        for _ in range(3):
            e2e_step()
        barrier()
        n_e2e = min(args.steps, 100)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / n_e2e
        e2e = {"value": T / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": ms_e2e,
               "note": "queries, lengths, page table copied in and output copied out every step; the paged KV pool is the "
                       "resident cache the operator reads, not a per-step input"}
        # The same step with no staging copies for the two large operands: the kernels read the query rows from, and
        # write the output rows to, pinned host memory themselves (page-locked memory is mapped into the device's
        # address space), so only lengths, offsets and the page table are copied.  Reported beside `e2e`, which stays
        # the conservative form with explicit copies of every operand.
        host_in = views(host_buf)
        ws_zc = RpaWorkspace(_shape_of(batch.queries, batch.kv_pages, batch.block_tables), dev)
        small = total - offs[1]  # everything but the queries, which lie first in the buffer

        def zc_step():
            dev_buf[offs[1]:].copy_(host_buf[offs[1]:], non_blocking=True)
            ragged_page_attention_into(host_out, ws_zc, host_in[0], batch.kv_pages, dev_in[1], dev_in[2], dev_in[3], dev_in[4], **kw)
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            zc_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            zc_step()
        e1.record()
        barrier()
        ms_zc = max_over_ranks(e0.elapsed_time(e1)) / n_e2e
        e2e_zero_copy = {"value": T / (ms_zc * 1e-3), "unit": UNIT, "ms_per_step": ms_zc, "h2d_copied_bytes_per_step": small,
                         "h2d_read_by_kernel_bytes_per_step": offs[1], "d2h_written_by_kernel_bytes_per_step": d2h,
                         "status_word": int(ws_zc.status.item()),
                         "note": "ragged_page_attention_into with queries and out in pinned host memory: the kernels read and "
                                 "write them over PCIe directly; lengths, offsets and page table copied as in e2e"}
        del host_buf, dev_buf, host_out, ws_zc

    # ---------------- cpu baseline (rank 0, N = 1 only) ----------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        n = pick_sample_size(batch, 4.0)
        sample = compact_sample(batch, n)
        tps, gbs, ms, cores = cpu_reference_rate(sample, args.cpu_seconds, steps=3, warmup=0)
        cpu = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "gb_per_s": gbs,
               "sample": f"first {len(sample.meta['kv_lens'])} of {total_seqs} sequences (their pages compacted to a host pool), "
                         f"as-written XLA algorithm restated with torch CPU ops, {ms:.0f} ms per pass"}

    head_roof = rooflines(batch, rec)
    plan_ms, merge_ms, launches_per_step = rec["plan_ms"], rec["merge_ms"], rec["launches_per_step"]
    # The denominator of `frac` is a copy benchmark (it reads and writes); what a read-only stream reaches on this GPU is
    # measured here with the library's probe: the same bulk copies into shared memory the split-KV kernel gathers pages
    # with, two CTAs per SM, nothing done with the data, over the whole KV pool (far larger than the L2).
    read_ceiling = None
    try:
        read_ceiling = _cabi.stream_probe_gbs(batch.kv_pages, passes=5)
    except Exception as exc:  # a diagnostic: the bench line does not depend on it
        print(f"bench.py: stream probe failed: {exc}", file=sys.stderr)
    del batch, out, rec
    torch.cuda.empty_cache()

    # ---------------- the other workloads (outside the headline's timed region) ----------------
    per_workload, c5_strong = None, None
    default_run = (args.workload == "c2" and args.num_seqs is None and args.len_scale == 1.0 and not args.strong
                   and args.kv_dtype == "bf16" and args.shard_of == 1)
    if default_run and not args.headline_only:
        k_steps = max(5, min(args.steps, 30))
        # "c2_e4m3_kv": the headline batch on a float8 (e4m3) pool -- half the KV bytes per token
        names = ("c3", "c4", "c5", "c2_e4m3_kv") if world == 1 else ("c5",)
        records = {}
        for name in names:
            e4m3 = name.endswith("_e4m3_kv")
            b = build(name.split("_")[0], dev, head_slice_for(name.split("_")[0]),
                      kv_dtype=torch.float8_e4m3fn if e4m3 else None)
            r, o = measure(b, k_steps, 3)
            add_parity(name, b, o)
            status_all |= r["status_word"]
            bytes_rank = algorithmic_kv_bytes(b)
            records[name] = {
                "workload": f"{name}: {len(b.meta['kv_lens'])} seqs, {b.total_tokens} query tokens, KV cache {b.kv_pages.dtype}"
                            + (f", {b.meta['num_kv_heads']} of 8 kv heads per GPU" if world > 1 else ""),
                "ms_per_step": r["ms_per_step"], "kernel_ms": r["prefill_ms"] + r["splitkv_ms"], "plan_ms": r["plan_ms"],
                "merge_ms": r["merge_ms"], "tokens_per_s": b.total_tokens / (r["ms_per_step"] * 1e-3),
                "hbm_tbs": bytes_rank * world / (r["ms_per_step"] * 1e-3) / 1e12,
                "hbm_gbs_per_gpu": bytes_rank / (r["ms_per_step"] * 1e-3) / 1e9,
                "roofline": rooflines(b, r), "steps": k_steps, "launches_per_step": r["launches_per_step"],
            }
            del b, o, r
            torch.cuda.empty_cache()
        if world == 1:
            per_workload = records
        else:
            c5_strong = records["c5"]
            c5_strong["scaling"] = "strong: the same 64 sequences at every N, kv heads split over the ranks"

    if world > 1:
        # one flag per status bit plus the parity result, MAX over ranks = OR
        bits = torch.tensor([(status_all >> i) & 1 for i in range(8)] + [0 if parity["ok"] else 1], device=dev,
                            dtype=torch.int64)
        dist.all_reduce(bits, op=dist.ReduceOp.MAX)
        bits = bits.tolist()
        status_all = int(sum(int(v) << i for i, v in enumerate(bits[:8])))
        parity["ok"] = bits[8] == 0
        parity["max_err_over_rms"] = max_over_ranks(parity["max_err_over_rms"])
        parity["checked"] = int(max_over_ranks(float(parity["checked"]))) * world
    parity["ranks"] = world

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    total_bytes = kv_bytes_rank * world
    achieved = kv_bytes_rank / (k_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC,
        "value": T / (ms_step * 1e-3),
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(3, args.warmup),
        "ms_per_step": ms_step,
        "higher_is_better": True,
        "scaling": "weak" if weak else "strong",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": config,
        "hbm_tbs": total_bytes / (ms_step * 1e-3) / 1e12,
        "kv_bytes_per_step": total_bytes,
        "roofline": {
            "bound": "hbm", "kernel": "rpa attention (gather + QK^T + softmax + PV)", "achieved": achieved,
            "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src,
            "frac_of_nominal_8tbs": achieved / 8000.0, "kernel_ms": k_ms, "plan_ms": plan_ms, "merge_ms": merge_ms,
            "read_only_stream_gbs": read_ceiling, "frac_of_read_only_stream": (achieved / read_ceiling) if read_ceiling else None,
            "traffic": (kv_bytes_rank * NCU_TRAFFIC_RATIO[args.workload]) if args.workload in NCU_TRAFFIC_RATIO else None,
            "traffic_note": "dram bytes per launch = KV bytes x 1.010, the ratio ncu measured on a 48-sequence slice of this "
                            "workload (dram__bytes_read.sum + dram__bytes_write.sum over algorithmic KV bytes)",
            "per_kernel": head_roof,
        },
        "cpu_baseline": cpu,
        "e2e": e2e,
        "e2e_zero_copy": e2e_zero_copy,
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clk.summary(),
        "status_word": status_all,
        "parity_sample": None if args.headline_only else parity,
    }
    if per_workload is not None:
        line["per_workload"] = per_workload
    if c5_strong is not None:
        line["c5_strong"] = c5_strong
    emit(line, out_fd)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
