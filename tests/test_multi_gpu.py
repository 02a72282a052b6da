"""KV-head sharding on real GPUs: two processes, one GPU each, NCCL.  Each rank runs the CUDA operator
on its head shard through the public shard-map style entry; the head-sharded output needs no
collective, the replicated one is an NCCL all-gather of the output heads; that test is skipped unless the
box has at least two GPUs.  The partitioning alone (shards run one after another) is checked on any box."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from ejkernel_b200.utils import make_ragged_batch
from oracle.rpa_oracle import compare, dense_reference
from tests.helpers import ATOL, REL_RMS, RTOL

pytestmark = pytest.mark.gpu


def _batch():
    return make_ragged_batch([1, 1, 20, 1], [3000, 257, 900, 64], num_q_heads=16, num_kv_heads=4, head_dim=128,
                             page_size=16, seed=17, sliding_window=2048)


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    import ejkernel_b200 as ej
    from ejkernel_b200.sharding import Mesh1D, head_sharded_specs, local_shard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        b = _batch()
        q, kv, _ = local_shard(b.queries, b.kv_pages, rank, world)
        dev = f"cuda:{rank}"
        args = [t.to(dev) for t in (q, kv, b.context_lens, b.block_tables, b.query_start_loc, b.num_seqs)]
        mesh = Mesh1D("kv")
        outs = {}
        for replicate in (False, True):
            in_specs, out_specs = head_sharded_specs("kv", replicate_output=replicate)
            o = ej.ragged_page_attention(*args, softmax_scale=b.softmax_scale, sliding_window=b.sliding_window,
                                         mesh=mesh, in_specs=in_specs, out_specs=out_specs)
            torch.cuda.synchronize()
            outs[replicate] = o.float().cpu().numpy()
        ret[rank] = outs
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_head_sharding_matches_oracle(rpa_lib):
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        outs = [ret[r] for r in range(world)]
    b = _batch()
    want = dense_reference(*b.args(), **b.kwargs())
    sharded = np.concatenate([o[False] for o in outs], axis=1)
    r = compare(sharded, want, atol=ATOL, rtol=RTOL)
    assert r["finite"] and r["allclose"] and r["tight"] and r["max_rel_rms"] <= REL_RMS, r
    for o in outs:
        np.testing.assert_array_equal(o[True], sharded)  # the all-gather moves bits, it does not change them


@pytest.mark.parametrize("world", [2, 4])
def test_head_shards_run_one_after_another_on_one_gpu(rpa_lib, world):
    """The partitioning itself needs no second GPU to be checked: the KV-head shards are independent problems, so
    running them one after another on one device and joining the heads must give the operator's answer."""
    import ejkernel_b200 as ej
    from ejkernel_b200.sharding import local_shard

    b = _batch()
    rest = [t.cuda() for t in (b.context_lens, b.block_tables, b.query_start_loc, b.num_seqs)]
    parts = []
    for rank in range(world):
        q, kv, _ = local_shard(b.queries, b.kv_pages, rank, world)
        parts.append(ej.ragged_page_attention(q.cuda(), kv.cuda(), *rest, softmax_scale=b.softmax_scale,
                                              sliding_window=b.sliding_window))
    torch.cuda.synchronize()
    joined = torch.cat(parts, dim=1).float().cpu().numpy()
    r = compare(joined, dense_reference(*b.args(), **b.kwargs()), atol=ATOL, rtol=RTOL)
    assert r["finite"] and r["allclose"] and r["tight"] and r["max_rel_rms"] <= REL_RMS, r
