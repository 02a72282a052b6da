"""KV-head sharding across ranks, exercised with two gloo ranks on CPU.  The local compute of each
rank is the oracle (injected by overriding ``RaggedPageAttention.run``) because the CUDA kernels
need a GPU; what is under test is the host logic: the shard slicing, the spec checks, the absence of
any collective for a head-sharded output, and the output all-gather for a replicated one."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ejkernel_b200.modules.operations.ragged_page_attention import RaggedPageAttention
from ejkernel_b200.sharding import Mesh1D, P, head_sharded_specs, kv_head_range, local_shard
from ejkernel_b200.utils import make_ragged_batch
from oracle.rpa_oracle import dense_reference


class _OracleBacked(RaggedPageAttention):
    def run(self, queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, **kw):
        out = dense_reference(queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs,
                              softmax_scale=kw.get("softmax_scale"), sliding_window=kw.get("sliding_window"),
                              logits_soft_cap=kw.get("logits_soft_cap"), softmax_aux=kw.get("softmax_aux"))
        return torch.from_numpy(out).to(queries.dtype)


def _batch():
    b = make_ragged_batch([1, 6, 1], [120, 40, 77], num_q_heads=8, num_kv_heads=4, head_dim=64, page_size=8, seed=6,
                          sliding_window=50)
    b.softmax_aux = torch.linspace(-1, 1, 8).reshape(4, 2)
    return b


def _worker(rank, world, port, replicate, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b = _batch()
        q, kv, aux = local_shard(b.queries, b.kv_pages, rank, world, b.softmax_aux)
        mesh = Mesh1D("kv")
        in_specs, out_specs = head_sharded_specs("kv", replicate_output=replicate, sinks="sharded")
        fn, args = _OracleBacked().create_shard_map_wrapper(
            q, kv, b.context_lens, b.block_tables, b.query_start_loc, b.num_seqs, softmax_scale=b.softmax_scale,
            sliding_window=b.sliding_window, softmax_aux=aux, mesh=mesh, in_specs=in_specs, out_specs=out_specs)
        out = fn(*args)
        ret[rank] = out.float().numpy()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("replicate", [False, True])
def test_two_rank_head_sharding(replicate):
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), replicate, ret), nprocs=world, join=True)
        outs = [ret[r] for r in range(world)]
    b = _batch()
    want = torch.from_numpy(dense_reference(*b.args(), **b.kwargs())).to(torch.bfloat16).float().numpy()
    if replicate:
        for o in outs:
            np.testing.assert_array_equal(o, want)
    else:
        np.testing.assert_array_equal(np.concatenate(outs, axis=1), want)


def test_shard_helpers_and_spec_checks():
    assert kv_head_range(8, 3, 4) == (6, 8)
    with pytest.raises(ValueError):
        kv_head_range(2, 0, 4)
    b = _batch()
    q, kv, aux = local_shard(b.queries, b.kv_pages, 1, 2, b.softmax_aux)
    assert q.shape[1] == 4 and kv.shape[2] == 4 and aux.shape == (2, 2)
    assert torch.equal(q, b.queries[:, 4:8]) and torch.equal(kv, b.kv_pages[:, :, 4:8])
    in_specs, out_specs = head_sharded_specs()
    assert len(in_specs) == 7 and out_specs == P(None, "kv", None) and in_specs[2] == P()
    k = _OracleBacked()
    with pytest.raises(AssertionError):  # the reference asserts len(in_specs) == 7 as well
        k.create_shard_map_wrapper(*b.args(), mesh=Mesh1D(), in_specs=in_specs[:6], out_specs=out_specs)
    # a mesh of one rank needs no process group and no collective
    fn, args = k.create_shard_map_wrapper(*b.args(), softmax_scale=b.softmax_scale, sliding_window=b.sliding_window,
                                          softmax_aux=b.softmax_aux, mesh=Mesh1D(), in_specs=in_specs, out_specs=P())
    assert fn(*args).shape == b.queries.shape
