"""KV-head sharding across the GPUs of one box, one process per GPU.

The reference distributes the operator by wrapping it in ``jax.shard_map`` with caller-supplied
``PartitionSpec``s (ejkernel/modules/operations/ragged_page_attention.py:114-208): queries and
kv_pages split along their head axes, the index arrays replicated, and the output either left
split along heads (no communication) or replicated (one all-gather).  Query head ``h`` belongs to kv
head ``h // G`` (_xla_impl_fwd.py:46), so contiguous blocks of kv heads with their query groups are
independent problems: no rank ever reads another rank's KV pool.

Without JAX the same contract is expressed with ``torch.distributed``: every process already holds
its local shards, ``Mesh1D`` names the process group, and the only collective is the optional
output all-gather (NCCL over NVLink on GPUs, gloo in CPU tests).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


class PartitionSpec(tuple):
    """Tuple of mesh-axis names (or None) per array dimension; ``PartitionSpec()`` = replicated."""

    def __new__(cls, *axes):
        return super().__new__(cls, axes)

    def sharded_dim(self, axis_name: str) -> int | None:
        for i, a in enumerate(self):
            if a == axis_name:
                return i
        return None


P = PartitionSpec


@dataclass
class Mesh1D:
    """A one-axis device mesh: the ranks of ``group`` laid out along ``axis_name``."""

    axis_name: str = "kv"
    group: object | None = None  # torch.distributed.ProcessGroup; None = the default group

    @property
    def size(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group) if dist.is_initialized() else 0


def kv_head_range(num_kv_heads: int, rank: int, world: int) -> tuple[int, int]:
    if num_kv_heads % world != 0:
        raise ValueError(f"num_kv_heads={num_kv_heads} is not divisible by the mesh size {world}")
    per = num_kv_heads // world
    return rank * per, (rank + 1) * per


def head_sharded_specs(axis: str = "kv", replicate_output: bool = False, sinks: str | None = None):
    """The (in_specs, out_specs) of the KV-head partitioning, in the reference's argument order
    (queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, softmax_aux)."""
    aux = P() if sinks in (None, "replicated") else P(axis, None)
    in_specs = (P(None, axis, None), P(None, None, axis, None), P(), P(), P(), P(), aux)
    out_specs = P() if replicate_output else P(None, axis, None)
    return in_specs, out_specs


def local_shard(queries, kv_pages, rank: int, world: int, softmax_aux=None):
    """Slice global ``queries`` / ``kv_pages`` (and per-head sinks) down to one rank's KV heads."""
    Hkv = kv_pages.shape[2] // 2
    G = queries.shape[1] // Hkv
    h0, h1 = kv_head_range(Hkv, rank, world)
    q = queries[:, h0 * G : h1 * G, :].contiguous()
    kv = kv_pages[:, :, 2 * h0 : 2 * h1, :].contiguous()
    aux = softmax_aux
    if softmax_aux is not None and softmax_aux.ndim == 2:
        if softmax_aux.shape[0] == Hkv:
            aux = softmax_aux[h0:h1].contiguous()
        else:
            aux = softmax_aux[h0 * G : h1 * G].contiguous()
    return q, kv, aux


def all_gather_heads(local_out: torch.Tensor, mesh: Mesh1D) -> torch.Tensor:
    """Replicate a head-sharded output ``[T, Hq/n, D]`` as ``[T, Hq, D]`` on every rank."""
    n = mesh.size
    if n == 1:
        return local_out
    T, Hl, D = local_out.shape
    src = local_out.contiguous()
    if local_out.is_cuda:
        buf = torch.empty((n, T, Hl, D), dtype=local_out.dtype, device=local_out.device)
        dist.all_gather_into_tensor(buf, src, group=mesh.group)
    else:
        # gloo (CPU tests): list form, 16-bit floats moved as raw bytes
        raw = src.view(torch.uint8) if src.element_size() == 2 else src
        parts = [torch.empty_like(raw) for _ in range(n)]
        dist.all_gather(parts, raw, group=mesh.group)
        buf = torch.stack(parts, 0).view(local_out.dtype).reshape(n, T, Hl, D)
    return buf.permute(1, 0, 2, 3).reshape(T, n * Hl, D)
