"""Public ``ragged_page_attention`` operator: the ops-layer entry for the CUDA path.

Mirrors ejkernel/modules/operations/ragged_page_attention.py:80-641 -- a ``RaggedPageAttention``
kernel object (``get_impl`` / ``run`` / ``create_shard_map_wrapper`` / ``heuristic_cfg`` /
``candidate_cfgs``) and the module-level function with seven positional-only arrays and the same
keywords -- minus the reference's multi-backend selection: there is exactly one implementation, it
is looked up in the registry under ``Platform.CUDA`` and nothing else is ever tried.  Asking for
another platform raises.

What the reference's ``Executor`` does around ``run`` (ejkernel/ops/execution/executor.py:209-406) is done by
``_select_cfg`` and ``_stamped`` below: the configuration comes from the selection chain (explicit ``cfg``,
overlay, memory cache, persistent cache, autotune on the first call of a signature, heuristic;
``EJKERNEL_AUTOTUNE_POLICY=autotune|heuristics``), and with ``EJKERNEL_OPS_STAMP=hash|json`` the launch is wrapped in
an NVTX range labelled ``ejkernel_ops#ragged_page_attention@v0:<call key>`` (the reference stamps the same label
into the HLO, :131-207, :373-380).
"""

from __future__ import annotations

import contextlib
import json
import os
from typing import Literal

import torch

from ...kernels._registry import Backend, Platform, kernel_registry
from ...sharding import Mesh1D, PartitionSpec, all_gather_heads
from .configs import RaggedPageAttentionConfig
from .tuning import (AutotunePolicy, ConfigSelectorChain, PersistentCache, call_key, cuda_event_timer,
                     device_fingerprint, pick_best)
from . import tuning as _tuning

Array = torch.Tensor
OP_ID = "ragged_page_attention"
OP_VERSION = "0"  # "ragged_page_attention@v0", ejkernel/ops/core/kernel.py:137-161


def _resolve_platform(platform) -> Platform:
    """The reference's ``detect_platform`` (ejkernel/modules/base.py:45-111) picks among four
    platforms; here "auto"/None/"cuda" all mean CUDA and anything else is an error."""
    if platform in (None, "auto", "cuda", Platform.CUDA):
        return Platform.CUDA
    raise ValueError(
        f"platform={platform!r} is not available: this package provides only the CUDA (sm_100a) "
        "implementation of ragged_page_attention"
    )


class RaggedPageAttention:
    """Kernel object of the operator (reference: ``RaggedPageAttention(Kernel)``, :80-523)."""

    op_id = OP_ID
    version = OP_VERSION

    def __init__(self, cache: PersistentCache | None = None, policy: AutotunePolicy | None = None, on_event=None):
        # ``cache``: tuned configurations kept across runs (None = memory only); ``policy``: what a call whose
        # signature is in no cache does -- measure the candidates once (the reference's default) or take the heuristic
        self.cache = cache
        self.selector = ConfigSelectorChain(policy=policy or AutotunePolicy.from_env(), persistent=cache, on_event=on_event)
        self._fast: dict[tuple, RaggedPageAttentionConfig] = {}  # static call signature -> chosen cfg, no hashing
        self._fingerprints: dict[int | None, str] = {}

    @property
    def op_id_v(self) -> str:
        return f"{self.op_id}@v{self.version}"

    def get_impl(self, cfg: RaggedPageAttentionConfig):
        platform = _resolve_platform(cfg.platform)
        backend = Backend.GPU if cfg.backend in (None, "any", Backend.ANY) else cfg.backend
        return kernel_registry.get(OP_ID, platform=platform, backend=backend)

    def heuristic_cfg(self, inv=None) -> RaggedPageAttentionConfig:
        return RaggedPageAttentionConfig(
            num_kv_pages_per_block=None, num_queries_per_block=None, num_warps=4, num_stages=1,
            platform="cuda", backend="gpu",
        )

    def candidate_cfgs(self, inv=None, page_size: int | None = None) -> list[RaggedPageAttentionConfig]:
        """The heuristic (the device planner sizes KV chunks from the lengths at run time) plus, when
        the page size is known, a few floors for the KV chunk and thresholds for the tensor tiles.
        The reference's GPU candidate list is a single entry (:478-499)."""
        out = [self.heuristic_cfg(inv)]
        if page_size:
            for chunk_tokens in (128, 512, 1024, 2048):
                out.append(RaggedPageAttentionConfig(
                    num_kv_pages_per_block=max(1, chunk_tokens // page_size), num_queries_per_block=None,
                    platform="cuda", backend="gpu"))
            for q_tokens in (4, 64):
                out.append(RaggedPageAttentionConfig(
                    num_kv_pages_per_block=None, num_queries_per_block=q_tokens, platform="cuda", backend="gpu"))
        return out

    def lookup_cfg(self, queries, kv_pages, block_tables, *, sliding_window=None, logits_soft_cap=None,
                   softmax_aux=None) -> RaggedPageAttentionConfig:
        """The tuned configuration of this call signature on this device, else the heuristic."""
        if self.cache is not None:
            hit = self.cache.get(device_fingerprint(queries.device), self.op_id_v,
                                 call_key(queries, kv_pages, block_tables, sliding_window=sliding_window,
                                          logits_soft_cap=logits_soft_cap, softmax_aux=softmax_aux))
            if hit is not None:
                return hit
        return self.heuristic_cfg()

    def autotune(self, queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, *,
                 softmax_scale=None, logits_soft_cap=None, sliding_window=None, softmax_aux=None,
                 candidates=None, timer=cuda_event_timer) -> RaggedPageAttentionConfig:
        """Measures every candidate on the given operands (reference: ``Tuner.measure``,
        ejkernel/ops/config/selection.py:226-245), stores the fastest under
        ``device|ragged_page_attention@v0|call_key`` if a cache is attached, and returns it."""
        cands = list(candidates) if candidates is not None else self.candidate_cfgs(page_size=kv_pages.shape[1])
        pages_per_seq = block_tables.shape[1]
        cands = [c for c in cands if c.num_kv_pages_per_block is None or c.num_kv_pages_per_block <= pages_per_seq]

        def run_with(cfg):
            return lambda: self.run(queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs,
                                    softmax_scale=softmax_scale, logits_soft_cap=logits_soft_cap,
                                    sliding_window=sliding_window, softmax_aux=softmax_aux, cfg=cfg)

        best, times = pick_best(cands, run_with, timer, margin=0.02)
        if os.environ.get("EJKERNEL_LOG_AUTOTUNE", "0") == "1":  # the reference's switch (ejkernel/ops/config/selection.py:328,338)
            for c, t in zip(cands, times):
                print(f"[ejkernel_b200 autotune] {self.op_id_v} num_kv_pages_per_block={c.num_kv_pages_per_block} "
                      f"num_queries_per_block={c.num_queries_per_block}: {t:.4f} ms" + ("  <- chosen" if c is best else ""))
        if self.cache is not None:
            self.cache.put(device_fingerprint(queries.device), self.op_id_v,
                           call_key(queries, kv_pages, block_tables, sliding_window=sliding_window,
                                    logits_soft_cap=logits_soft_cap, softmax_aux=softmax_aux), best)
        return best

    candidate_cfgs_gpu = candidate_cfgs
    candidate_cfgs_shard_map_gpu = candidate_cfgs

    def select_cfg(self, queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, *, cfg=None,
                   softmax_scale=None, logits_soft_cap=None, sliding_window=None, softmax_aux=None):
        """The configuration for this call, in the order of the reference's ``ConfigSelectorChain.choose``
        (ejkernel/ops/config/selection.py:384-566).  Returns ``(cfg, call_key or None)``.  Calls whose static
        signature (shapes, dtypes, window, cap, sinks shape, device) was resolved before take a dictionary look-up."""
        # token count and pool size enter as their bit lengths (= rounded up to a power of two, as in ``call_key``)
        fast = (queries.device.index, (queries.shape[0] - 1).bit_length(), queries.shape[1:], queries.dtype,
                (kv_pages.shape[0] - 1).bit_length(), kv_pages.shape[1:], kv_pages.dtype,
                tuple(block_tables.shape), sliding_window, logits_soft_cap,
                None if softmax_aux is None else tuple(softmax_aux.shape))
        if cfg is None and not _tuning._overlays:
            hit = self._fast.get(fast)
            if hit is not None:
                return hit, None
        dev = self._fingerprints.get(queries.device.index)
        if dev is None:
            dev = self._fingerprints[queries.device.index] = device_fingerprint(queries.device)
        key = call_key(queries, kv_pages, block_tables, sliding_window=sliding_window, logits_soft_cap=logits_soft_cap,
                       softmax_aux=softmax_aux)
        # measuring needs a device it can synchronise: not while the stream is being captured into a graph
        can_measure = queries.is_cuda and not torch.cuda.is_current_stream_capturing()
        chosen = self.selector.choose(
            dev, self.op_id_v, key, override=cfg, may_autotune=can_measure, heuristic=self.heuristic_cfg,
            autotune=lambda: self.autotune(queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs,
                                           softmax_scale=softmax_scale, logits_soft_cap=logits_soft_cap,
                                           sliding_window=sliding_window, softmax_aux=softmax_aux))
        if cfg is None and not _tuning._overlays and self.selector.cache.get(dev, self.op_id_v, key) is chosen:
            if len(self._fast) > 4096:  # a serving loop with ever new shapes must not grow this without bound
                self._fast.clear()
            self._fast[fast] = chosen
        return chosen, key

    def run(
        self,
        queries: Array,
        kv_pages: Array,
        context_lens: Array,
        block_tables: Array,
        query_start_loc: Array,
        num_seqs: Array | int,
        platform: Literal["triton", "pallas", "cuda", "xla", "auto"] | None = None,
        softmax_scale: float | None = None,
        logits_soft_cap: float | None = None,
        compute_dtype=torch.bfloat16,
        optimized: bool = False,
        sliding_window: int | None = None,
        softmax_aux: Array | None = None,
        mask_value: float | None = None,
        vmem_limit_bytes: int | None = None,
        *,
        cfg: RaggedPageAttentionConfig,
    ) -> Array:
        if platform is not None:
            cfg = RaggedPageAttentionConfig(
                num_kv_pages_per_block=cfg.num_kv_pages_per_block,
                num_queries_per_block=cfg.num_queries_per_block,
                num_warps=cfg.num_warps,
                num_stages=cfg.num_stages,
                platform=platform,
                backend=cfg.backend,
            )
        impl = self.get_impl(cfg)
        return impl(
            queries=queries,
            kv_pages=kv_pages,
            context_lens=context_lens,
            block_tables=block_tables,
            query_start_loc=query_start_loc,
            num_seqs=num_seqs,
            softmax_scale=softmax_scale,
            logits_soft_cap=logits_soft_cap,
            compute_dtype=compute_dtype,
            optimized=optimized,
            sliding_window=sliding_window,
            softmax_aux=softmax_aux,
            mask_value=mask_value,
            num_kv_pages_per_block=cfg.num_kv_pages_per_block,
            num_queries_per_block=cfg.num_queries_per_block,
            vmem_limit_bytes=vmem_limit_bytes,
            num_warps=cfg.num_warps,
            num_stages=cfg.num_stages,
        )

    def create_shard_map_wrapper(
        self,
        queries: Array,
        kv_pages: Array,
        context_lens: Array,
        block_tables: Array,
        query_start_loc: Array,
        num_seqs: Array | int,
        softmax_scale: float | None = None,
        logits_soft_cap: float | None = None,
        compute_dtype=torch.bfloat16,
        optimized: bool = False,
        sliding_window: int | None = None,
        softmax_aux: Array | None = None,
        mask_value: float | None = None,
        vmem_limit_bytes: int | None = None,
        platform=None,
        cfg: RaggedPageAttentionConfig | None = None,
        mesh: Mesh1D | None = None,
        in_specs: tuple[PartitionSpec, ...] | None = None,
        out_specs: PartitionSpec | None = None,
        check_vma: bool = False,
    ):
        """Returns ``(fn, call_args)`` like the reference (:114-208).  Every process passes its LOCAL
        shards; ``fn`` runs the kernel on them and, if ``out_specs`` does not shard the head axis,
        all-gathers the heads so each rank returns the full output."""
        assert mesh is not None, "mesh must be provided for shard_map execution"
        assert in_specs is not None, "in_specs must be provided for shard_map execution"
        assert out_specs is not None, "out_specs must be provided for shard_map execution"
        cfg = cfg or self.heuristic_cfg()
        axis = mesh.axis_name
        call_args = (queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, softmax_aux)
        assert len(in_specs) == len(call_args), f"in_specs length {len(in_specs)} != call_args length {len(call_args)}"
        q_spec, kv_spec = PartitionSpec(*in_specs[0]), PartitionSpec(*in_specs[1])
        if mesh.size > 1:
            if q_spec.sharded_dim(axis) != 1 or kv_spec.sharded_dim(axis) != 2:
                raise NotImplementedError(
                    "only the KV-head partitioning is supported: queries P(None, axis, None), "
                    "kv_pages P(None, None, axis, None)"
                )
            for i in (2, 3, 4, 5):
                if PartitionSpec(*in_specs[i]).sharded_dim(axis) is not None:
                    raise NotImplementedError("context_lens, block_tables, query_start_loc and num_seqs must be replicated")
        gather = mesh.size > 1 and PartitionSpec(*out_specs).sharded_dim(axis) is None

        def fn(queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, softmax_aux=None):
            out = self.run(
                queries=queries, kv_pages=kv_pages, context_lens=context_lens, block_tables=block_tables,
                query_start_loc=query_start_loc, num_seqs=num_seqs, softmax_scale=softmax_scale,
                logits_soft_cap=logits_soft_cap, compute_dtype=compute_dtype, optimized=optimized,
                sliding_window=sliding_window, softmax_aux=softmax_aux, mask_value=mask_value,
                vmem_limit_bytes=vmem_limit_bytes, platform=platform, cfg=cfg,
            )
            return all_gather_heads(out, mesh) if gather else out

        return fn, call_args


def _cache_from_env() -> PersistentCache | None:
    """``EJKERNEL_B200_TUNING_CACHE=<file.json>`` attaches a persistent cache to the module-level
    operator (the reference reads its cache location from the environment too,
    ejkernel/ops/config/selection.py:328)."""
    import os

    path = os.environ.get("EJKERNEL_B200_TUNING_CACHE")
    return PersistentCache(OP_ID, path, cfg_type=RaggedPageAttentionConfig) if path else None


_kernel = RaggedPageAttention(cache=_cache_from_env())


def ragged_page_attention(
    queries: Array,
    kv_pages: Array,
    context_lens: Array,
    block_tables: Array,
    query_start_loc: Array,
    num_seqs: Array | int,
    softmax_aux: Array | None = None,
    /,
    *,
    softmax_scale: float | None = None,
    logits_soft_cap: float | None = None,
    compute_dtype=torch.bfloat16,
    optimized: bool = False,
    sliding_window: int | None = None,
    mask_value: float | None = None,
    vmem_limit_bytes: int | None = None,
    platform: Literal["triton", "pallas", "cuda", "xla", "auto"] | None = None,
    cfg: RaggedPageAttentionConfig | None = None,
    mesh: Mesh1D | None = None,
    in_specs: tuple[PartitionSpec | None, ...] | None = None,
    out_specs: PartitionSpec | None = None,
) -> Array:
    """Ragged paged attention (reference: ejkernel/modules/operations/ragged_page_attention.py:540-641).

    ``queries [T,Hq,D]``, ``kv_pages [P,page,2*Hkv,D]``, ``context_lens [S]``, ``block_tables
    [S,pages_per_seq]``, ``query_start_loc [S+1]``, ``num_seqs`` (int32 ``[1]`` tensor or int), optional
    ``softmax_aux`` sinks.  With ``mesh``, ``in_specs`` and ``out_specs`` all given the call runs in
    shard-map mode on this process's local shards (see ``create_shard_map_wrapper``).
    """
    cfg, key = _kernel.select_cfg(queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, cfg=cfg,
                                  softmax_scale=softmax_scale, logits_soft_cap=logits_soft_cap,
                                  sliding_window=sliding_window, softmax_aux=softmax_aux)
    common = dict(
        softmax_scale=softmax_scale, logits_soft_cap=logits_soft_cap, compute_dtype=compute_dtype,
        optimized=optimized, sliding_window=sliding_window, softmax_aux=softmax_aux, mask_value=mask_value,
        vmem_limit_bytes=vmem_limit_bytes, platform=platform, cfg=cfg,
    )
    with _stamped(queries, kv_pages, block_tables, key, cfg, sliding_window, logits_soft_cap, softmax_aux):
        if mesh is not None and in_specs is not None and out_specs is not None:
            fn, call_args = _kernel.create_shard_map_wrapper(
                queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs,
                mesh=mesh, in_specs=in_specs, out_specs=out_specs, **common,
            )
            return fn(*call_args)
        return _kernel.run(queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, **common)


_STAMP_MODE = os.environ.get("EJKERNEL_OPS_STAMP", "none").lower()
_STAMP_PREFIX = os.environ.get("EJKERNEL_OPS_PREFIX", "ejkernel_ops")


def stamp_label(queries, kv_pages, block_tables, key, cfg, sliding_window=None, logits_soft_cap=None, softmax_aux=None,
                mode: str = "hash") -> str:
    """``<prefix>#ragged_page_attention@v0:<call key>`` (mode "hash"), or the prefix followed by a JSON description of
    the call (mode "json") -- the labels of the reference's ``Executor._stamp_hash`` / ``_stamp_json``
    (ejkernel/ops/execution/executor.py:131-184)."""
    if mode == "json":
        payload = json.dumps(dict(
            op_id=_kernel.op_id_v, queries=[list(queries.shape), str(queries.dtype)],
            kv_pages=[list(kv_pages.shape), str(kv_pages.dtype)], block_tables=list(block_tables.shape),
            sliding_window=sliding_window, logits_soft_cap=logits_soft_cap,
            cfg=dict(num_kv_pages_per_block=cfg.num_kv_pages_per_block, num_queries_per_block=cfg.num_queries_per_block),
        ), sort_keys=True)
        return f"{_STAMP_PREFIX}:{payload}"
    if key is None:
        key = call_key(queries, kv_pages, block_tables, sliding_window=sliding_window, logits_soft_cap=logits_soft_cap,
                       softmax_aux=softmax_aux)
    return f"{_STAMP_PREFIX}#{_kernel.op_id_v}:{key}"


@contextlib.contextmanager
def _stamped(queries, kv_pages, block_tables, key, cfg, sliding_window, logits_soft_cap, softmax_aux):
    """NVTX range around the launch when ``EJKERNEL_OPS_STAMP`` is ``hash`` or ``json`` (read at import); nothing,
    and no cost, otherwise."""
    if _STAMP_MODE not in ("hash", "json") or not queries.is_cuda:
        yield
        return
    torch.cuda.nvtx.range_push(stamp_label(queries, kv_pages, block_tables, key, cfg, sliding_window, logits_soft_cap,
                                           softmax_aux, mode=_STAMP_MODE))
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
