/*
 * C ABI of the sm_100a ragged paged attention path.
 *
 * This is the boundary a host runtime binds to.  It replaces, for the CUDA platform, what
 * the reference reaches through its registry entry
 *   ejkernel/kernels/_xla/ragged_page_attention/_interface.py:25-109   (operator signature)
 *   ejkernel/kernels/_triton/ragged_page_attention/_triton_impl_fwd.py:485-613 (GPU launch wrapper:
 *       dense row-major strides, int32 index arrays, one output, the caller's stream)
 * and what a `jax.ffi` custom call for the operator would hand to a GPU handler
 *   ejkernel/callib/_triton_call.py:737-757 (operands in, results out, XLA's stream, no host sync).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current CUDA device unless stated otherwise; `queries` and `out` of the
 *     launch entry points may also point to page-locked host memory that is mapped into the device's address space
 *     (cudaHostAlloc / cudaHostRegister under unified addressing): the kernels read each query row once per work item
 *     and write each output row once, so host-resident queries and results need no staging copies;
 *   - tensors are dense row-major:
 *       queries          [total_tokens, num_q_heads, head_dim]
 *       kv_pages         [num_pages, page_size, 2*num_kv_heads, head_dim]  (K_h at 2h, V_h at 2h+1)
 *       context_lens     [max_num_seqs]                 int32
 *       block_tables     [max_num_seqs, pages_per_seq]  int32
 *       query_start_loc  [max_num_seqs + 1]             int32
 *       num_seqs         [1]                            int32
 *       out              [total_tokens, num_q_heads, head_dim], dtype of queries
 *   - calls only enqueue work on `stream`; they never allocate, synchronise or read device
 *     memory from the host, which is what an XLA custom call requires of its handler;
 *   - return value: 0 = ok, negative = invalid argument (EJK_RPA_E_*), positive = cudaError_t;
 *   - nothing throws.
 */
#ifndef EJK_RPA_H_
#define EJK_RPA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EJK_RPA_VERSION 2

#if defined(__GNUC__)
#define EJK_RPA_API __attribute__((visibility("default")))
#else
#define EJK_RPA_API
#endif

/* dtype codes for queries / kv_pages / out */
#define EJK_RPA_BF16 0
#define EJK_RPA_F16 1
/* dtype code of an 8-bit cache (ejk_rpa_shape.kv_dtype): float8 e4m3 ("e4m3fn": no infinities, maximum 448) */
#define EJK_RPA_E4M3 2

/* invalid-argument codes */
#define EJK_RPA_E_NULL (-1)      /* a required pointer is null */
#define EJK_RPA_E_SHAPE (-2)     /* a dimension is <= 0 or beyond its limit, Hq % Hkv != 0, ... */
#define EJK_RPA_E_HEAD_DIM (-3)  /* head_dim not in {64, 128, 256} */
#define EJK_RPA_E_DTYPE (-4)     /* unknown dtype code */
#define EJK_RPA_E_WORKSPACE (-5) /* workspace smaller than ejk_rpa_workspace_bytes_min() / misaligned */
#define EJK_RPA_E_ARG (-6)       /* sliding_window / logits_soft_cap / sinks out of contract */
#define EJK_RPA_E_DEVICE (-7)    /* current device is not sm_100 class */
#define EJK_RPA_E_ALIGN (-8)     /* a tensor base pointer is not 16-byte aligned */
#define EJK_RPA_E_SCRATCH (-9)   /* shape needs more than EJK_RPA_STATIC_SCRATCH_BYTES of scratch */

/* bits of the device-side status word (OR-ed in by the kernels; 0 = clean).  Inputs that
 * break the operator's contract never fault: the offending value is clamped or the sequence
 * skipped, and the bit records it.  Contract: _pallas_impl_fwd.py:124-230 of the reference. */
#define EJK_RPA_ST_NUM_SEQS 1u  /* num_seqs[0] > max_num_seqs */
#define EJK_RPA_ST_QLEN 2u      /* q_len < 0, q_len > kv_len, or query rows past total_tokens */
#define EJK_RPA_ST_KVLEN 4u     /* kv_len < 0 or > pages_per_seq * page_size */
#define EJK_RPA_ST_PAGE_ID 8u   /* a page id outside [0, num_pages) was met (read as page 0) */
#define EJK_RPA_ST_INTERNAL 16u /* planner produced more work items than the workspace holds */
#define EJK_RPA_ST_TIMEOUT 32u  /* a bounded wait inside a kernel ran out (outputs are invalid) */

/* Static problem description: everything here is known from array shapes at trace time.
 * Limits (EJK_RPA_E_SHAPE beyond them): total_tokens * num_q_heads < 2^30, max_num_seqs < 2^24,
 * pages_per_seq * page_size < 2^30 -- row, sequence and token positions are 32-bit in the work lists. */
typedef struct ejk_rpa_shape {
  int32_t total_tokens;  /* rows of queries / out */
  int32_t max_num_seqs;  /* block_tables.shape[0] */
  int32_t pages_per_seq; /* block_tables.shape[1] */
  int32_t num_pages;     /* kv_pages.shape[0] */
  int32_t page_size;     /* kv_pages.shape[1] */
  int32_t num_q_heads;
  int32_t num_kv_heads;  /* kv_pages.shape[2] / 2 */
  int32_t head_dim;      /* 64, 128 or 256 */
  int32_t dtype;         /* EJK_RPA_BF16 | EJK_RPA_F16: queries and out (and the cache, unless kv_dtype says otherwise) */
  int32_t kv_dtype;      /* 0 = the cache has `dtype`; EJK_RPA_E4M3 = kv_pages / kv_cache hold e4m3 bytes (the fp8 KV cache of
                            the v3 operator, ejkernel/kernels/_xla/ragged_page_attention_v3/_kernel.py:45-57,157-159,249-291).
                            Needs head_dim 128 or 256 and a page_size that is a multiple of 8 (head_dim 64 only through
                            ejk_rpa_v3_launch, whose cache pads a row to 128 bytes: it is attended as head_dim 128 with
                            the queries' upper half zero); every sequence is then served by the split-KV kernel.  The v3 cache pads its combined-head axis to a multiple of four
                            (the reference packs four e4m3 heads per 32-bit word), i.e. by two heads when num_kv_heads is
                            odd: ejk_rpa_v3_launch derives that stride itself, ejk_rpa_launch reads a dense
                            [P, page, 2*num_kv_heads, D] pool. */
} ejk_rpa_shape;

/* Scalar attributes of one call (the keyword arguments of the reference operator). */
typedef struct ejk_rpa_attrs {
  float softmax_scale;   /* must be given; the Python layer substitutes head_dim**-0.5 for None
                            (_interface.py:94-95) */
  float logits_soft_cap; /* 0 = none (the reference rejects 0.0 as a cap, _pallas_impl_fwd.py:222) */
  int32_t sliding_window;/* <= 0 = none; W keeps keys (pos-W, pos] (_xla_impl_fwd.py:128-134) */
  int32_t num_sinks;     /* 0 = no softmax_aux */
  int32_t sink_rows;     /* rows of softmax_aux: num_q_heads, num_kv_heads, or 1 (_xla_impl_fwd.py:60-77) */
  int32_t num_kv_pages_per_block; /* tile hint of RaggedPageAttentionConfig (configs.py:242-258), 0 = auto: the
                                     smallest KV chunk, in pages, a row tile is split into (overrides option
                                     "min_chunk" for this call) */
  int32_t num_queries_per_block;  /* tile hint, 0 = auto: sequences with at least this many query tokens are served
                                     by 128-row tensor tiles (overrides option "prefill_rows" for this call) */
  float q_scale;         /* 0 = none: the queries are divided by it, clipped to the finite range of the cache dtype and
                            rounded to it as they are staged (_kernel.py:249-254); with an e4m3 cache Q.K^T then runs on
                            e4m3 operands.  The caller folds q_scale (and k_scale) into softmax_scale, as the reference
                            multiplies the logits back (:262-265).  Every sequence is then served by the split-KV kernel;
                            needs a page_size the TMA gather supports (a multiple of 8). */
  float out_scale;       /* 0 = none (1.0): factor applied to the normalised output in float32, before the cast to
                            the output dtype -- `v_scale` of the v3 operator
                            (ejkernel/kernels/_xla/ragged_page_attention_v3/_kernel.py:283-284) */
} ejk_rpa_attrs;

/* Library version (EJK_RPA_VERSION of the build).  No reference counterpart; the reference
 * versions operators as "ragged_page_attention@v0" in ejkernel/ops/core/kernel.py:137-161. */
EJK_RPA_API int ejk_rpa_version(void);

/* Human-readable text for a return code of this library.  Host pointer, static storage. */
EJK_RPA_API const char* ejk_rpa_error_string(int code);

/* Bytes of scratch the launch needs for this static shape on the current device (split-KV
 * partials, the device-built work list, the merge list).  Depends on shapes only, never on
 * lengths, so a tracing runtime can allocate it as an extra result buffer.  It also grows with the
 * process-wide option "waves" (more work items per CTA need more partial slots): size the workspace
 * after setting that option, or a later launch answers EJK_RPA_E_WORKSPACE.  Returns 0 on an
 * invalid shape.  The reference has no scratch: XLA materialises its own temporaries
 * (_xla_impl_fwd.py:113-114). */
EJK_RPA_API size_t ejk_rpa_workspace_bytes(const ejk_rpa_shape* shape);

/* The smallest workspace a launch accepts for this shape.  It is smaller than
 * ejk_rpa_workspace_bytes() for shapes that can hold multi-token sequences: the difference is the
 * room in which prefill items cut along KV park their parts (option "prefill_split"); with the
 * smaller workspace those items are scheduled whole.  No reference counterpart. */
EJK_RPA_API size_t ejk_rpa_workspace_bytes_min(const ejk_rpa_shape* shape);

/* Enqueue one ragged paged attention call on `stream` (a cudaStream_t).
 * Replaces _ragged_paged_attention (_xla_impl_fwd.py:25-201) / ragged_paged_attention_triton_call
 * (_triton_impl_fwd.py:485-613).  `workspace` must be 256-byte aligned and hold
 * ejk_rpa_workspace_bytes(shape) bytes; its contents need not be initialised.  `status`
 * (device int32, may be null) gets EJK_RPA_ST_* bits OR-ed in; the caller zeroes it.
 * `softmax_aux` is float32 [sink_rows, num_sinks] or null.  Rows of `out` past the last sequence
 * (>= query_start_loc[num_seqs]) are zero-filled, as in the reference, whose result starts as zeros
 * (_xla_impl_fwd.py:58); `out` therefore needs no initialisation.  Rows of a sequence whose entry breaks the
 * contract (a status bit is set) are unspecified. */
EJK_RPA_API int ejk_rpa_launch(const void* queries, const void* kv_pages, const int32_t* context_lens,
                   const int32_t* block_tables, const int32_t* query_start_loc, const int32_t* num_seqs,
                   const float* softmax_aux, void* out, void* workspace, size_t workspace_bytes,
                   int32_t* status, const ejk_rpa_shape* shape, const ejk_rpa_attrs* attrs, void* stream);

/* The v3 operator: write this step's new key/value rows into the paged cache, then attend.
 * Replaces ragged_paged_attention of ejkernel/kernels/_xla/ragged_page_attention_v3/_kernel.py:143-318:
 * `keys` / `values` are [total_tokens, num_kv_heads, head_dim]; row r of sequence s goes to cache
 * position kv_len - q_len + r (:227-229); `kv_cache` is updated IN PLACE (the reference donates it,
 * :141) and is the reference's [num_pages, page_size, 2*Hkv/pack, pack, align_to(head_dim, 128)]
 * array, whose bytes are those of the [num_pages, page_size, 2*Hkv, head_dim] layout of
 * ejk_rpa_launch when head_dim is a multiple of 128; otherwise the rows are padded to the next
 * multiple (:45-57): the page write zero-fills the padding of the rows it writes and the attention
 * kernels step over it.  `block_tables` is the same table flattened; `distribution` is int32[3] whose
 * last entry is the number of sequences (:211).  Everything else as ejk_rpa_launch (no sinks in v3). */
EJK_RPA_API int ejk_rpa_v3_launch(const void* queries, const void* keys, const void* values, void* kv_cache,
                                  const int32_t* kv_lens, const int32_t* block_tables,
                                  const int32_t* query_start_loc, const int32_t* distribution, void* out,
                                  void* workspace, size_t workspace_bytes, int32_t* status,
                                  const ejk_rpa_shape* shape, const ejk_rpa_attrs* attrs, void* stream);

/* Decode-only paged attention over SEPARATE key / value caches
 *   key_cache, value_cache [num_blocks, num_kv_heads, block_size, head_dim],  query / out [num_seqs, num_q_heads, head_dim],
 *   context_lens [num_seqs], block_tables [num_seqs, max_blocks]
 * -- the reference's `page_attention` operator (ejkernel/kernels/_xla/page_attention/_xla_impl_fwd.py:22-97;
 * Triton split-KV + reduce version ejkernel/kernels/_triton/page_attention/_interface.py:88-369).  Same
 * kernels as ejk_rpa_launch with a different tensor map: every sequence has one query row that sees all
 * keys below its context length.  `shape`: total_tokens = max_num_seqs = num_seqs, pages_per_seq =
 * max_blocks, num_pages = num_blocks, page_size = block_size (a multiple of 8 for the TMA gather; any other size takes the cp.async gather).
 * `attrs`: softmax_scale = attn_scale, logits_soft_cap = attn_logits_soft_cap (0 = none); the rest 0. */
EJK_RPA_API int ejk_page_attention_launch(const void* query, const void* key_cache, const void* value_cache,
                                          const int32_t* context_lens, const int32_t* block_tables, void* out,
                                          void* workspace, size_t workspace_bytes, int32_t* status,
                                          const ejk_rpa_shape* shape, const ejk_rpa_attrs* attrs, void* stream);

/* Size of the scratch buffer built into the library for ejk_rpa_launch_static_scratch. */
#define EJK_RPA_STATIC_SCRATCH_BYTES (32u << 20)

/* Same operation as ejk_rpa_launch for callers that have no way to obtain device memory at the
 * point of the call: a custom-call handler whose runtime gave it only operand and result buffers,
 * a plugin running under another framework's memory pool that forbids foreign cudaMalloc, or code
 * on a latency-critical path where an allocation (which may synchronise the device) is not
 * acceptable.  It has no counterpart in the reference, whose XLA path lets the compiler allocate
 * temporaries.
 *
 * The scratch comes from a fixed EJK_RPA_STATIC_SCRATCH_BYTES (32 MiB) array compiled into the
 * library's device image; each GPU that loads the library keeps that much memory reserved until
 * the process exits.  The caller still passes every input, `out` and `status` exactly as for
 * ejk_rpa_launch.  The call itself performs no cudaMalloc / cudaFree and calls no allocating
 * library routine.
 *   - A shape whose ejk_rpa_workspace_bytes_min() exceeds the array is refused with
 *     EJK_RPA_E_SCRATCH (roughly: decode batches up to a few hundred sequences fit, batches with
 *     thousands of prefill rows do not); nothing is launched in that case.
 *   - The first call on each device looks up the array's device address (a one-time set-up with
 *     that device current); make that first call outside any stream capture.
 *   - All calls on one GPU share the one array, and it keeps whatever the previous call left in
 *     it.  Nothing in it needs clearing between calls -- the planner kernel rewrites every word
 *     that is later read -- but two calls whose kernels overlap on the GPU (different streams, or
 *     different host threads) would overwrite each other's work lists and partial results: issue
 *     them on one stream, or otherwise order them.
 *   - Refused with EJK_RPA_E_ARG while option "profile" is 1. */
EJK_RPA_API int ejk_rpa_launch_static_scratch(const void* queries, const void* kv_pages, const int32_t* context_lens,
                                              const int32_t* block_tables, const int32_t* query_start_loc,
                                              const int32_t* num_seqs, const float* softmax_aux, void* out,
                                              int32_t* status, const ejk_rpa_shape* shape,
                                              const ejk_rpa_attrs* attrs, void* stream);

/* Process-wide tuning knobs (host side, not thread safe against concurrent launches):
 *   "waves"      work items per resident CTA the device planner aims for (default 4)
 *   "min_chunk"  smallest KV chunk, in tokens, a split may have (default 256)
 *   "path"       0 = auto, 1 = force the cp.async gather, 2 = force the TMA gather
 *   "prefill_rows" sequences with at least this many (query token, head-in-group) rows per kv head are
 *                served by 128-row tcgen05 tiles instead of 8-row split-KV tiles (default 32; 0 = never)
 *   "prefill_share" percent (default 125; 0 = off): in a batch that mixes multi-token sequences with decode rows the
 *                tensor-tile kernel keeps only as many CTAs as make it finish about when the bandwidth-bound split-KV
 *                kernel does (estimated on the device from the plan, times this percentage) and leaves the other SMs to
 *                that kernel from the start
 *   "prefill_split" 1 (default) = when the workspace has the size ejk_rpa_workspace_bytes reports, prefill items are
 *                cut along KV at per-CTA quota boundaries and their parts combined by the last one to finish;
 *                0 = whole items from a longest-first queue (also what a smaller workspace gets);
 *                2 = cut at every quota boundary, whatever the rule says (a measurement aid)
 *   "sort_items" 1 (default) = the planner queues split-KV work items longest first, 0 = in sequence order
 *   "overlap"    1 (default) = the kernels of one call are launched as programmatic dependents: each starts under
 *                the tail of the one before and waits on the device for what it needs.  The first of them, the
 *                planner, is launched the same way behind whatever precedes the call in the stream and waits for
 *                that work's completion before it touches memory, so the call is ordered exactly as in plain
 *                stream order; only launch latency is hidden.  0 = plain stream order
 *   "fused_merge" 1 (default) = where a row tile gets few KV chunks (decided from the static shapes) the split-KV
 *                kernel's last-finishing chunk combines the chunks of its tile; 0 = always a separate merge kernel;
 *                2 = always fused
 *   "test_withhold" test hook, 0 in production: bit 0 / bit 1 make the CTA of the split-KV / prefill kernel that takes
 *                work item 0 never announce the item's first KV stage, so that the waits on it run out and the call reports
 *                EJK_RPA_ST_TIMEOUT (no fault, no hang; the context stays usable)
 *   "wait_ms"    wall-time bound, in milliseconds, of every wait inside a kernel (default 2000)
 *   "profile"    1 = record CUDA events around each kernel of a launch (see ejk_rpa_profile_read)
 *   "probe_chunk_kb", "probe_slots", "probe_ctas"  shape of ejk_rpa_stream_probe: KB per copy (a power of two up to 64),
 *                copies in flight per CTA (up to 12), CTAs per SM (up to 8); 0 = the defaults 32 / 3 / 2, the shape the
 *                split-KV kernel itself runs with
 * Returns 0, or EJK_RPA_E_ARG for an unknown name.  Counterpart of the reference's
 * EJKERNEL_* environment switches (ejkernel/ops/config/selection.py:328). */
EJK_RPA_API int ejk_rpa_set_option(const char* name, int value);
EJK_RPA_API int ejk_rpa_get_option(const char* name, int* value);

/* Number of kernels the last ejk_rpa_launch on this thread enqueued (host-side counter, for
 * benchmark bookkeeping). */
EJK_RPA_API int ejk_rpa_last_launch_count(void);

/* Diagnostic: enqueue one read-only pass over `bytes` of device memory at `src` (16-byte aligned, at least 64 KiB; rounded down to
 * whole 32 KiB copies) with the bulk asynchronous copies the split-KV kernel gathers KV pages with, two
 * CTAs per SM, nothing done with the data.  Timed with events around it, it gives the practical ceiling of that kernel
 * on this device: a copy benchmark reads and writes, a read-only stream can be faster.  `sink` points to 8 bytes of
 * device memory the caller zeroed: word 1 is set to 1 if a wait inside the probe ran out (option "wait_ms").  No
 * reference counterpart. */
EJK_RPA_API int ejk_rpa_stream_probe(const void* src, size_t bytes, void* sink, void* stream);

/* With option "profile" = 1, waits for the calling thread's last launch and returns the device
 * time of its planner, gather/attention and merge kernels in milliseconds (null pointers are
 * skipped).  EJK_RPA_E_ARG if no profiled launch exists.  This call synchronises; it is the
 * measuring hook that replaces the reference's wall-clock Tuner.measure
 * (ejkernel/ops/config/selection.py:226-245). */
EJK_RPA_API int ejk_rpa_profile_read(float* plan_ms, float* main_ms, float* merge_ms);

/* The same with the two attention kernels apart: `prefill_ms` is the tensor-tile kernel that serves sequences
 * with many query rows (0 when the batch shape has none), `splitkv_ms` the split-KV kernel of the decode rows;
 * main_ms above is their sum.  A bench uses it to hold each kernel against its own roofline (tensor / HBM). */
EJK_RPA_API int ejk_rpa_profile_read_kernels(float* plan_ms, float* prefill_ms, float* splitkv_ms, float* merge_ms);

#ifdef __cplusplus
}
#endif
#endif /* EJK_RPA_H_ */
