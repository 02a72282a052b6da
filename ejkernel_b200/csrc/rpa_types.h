// Shared host/device declarations of the ragged paged attention path.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "ejk_rpa.h"

namespace ejk {

// Rows of one small-q tile are (query token, head-in-group) pairs of ONE kv head, flattened
// as row = q_token * G + g, so a decode token with G <= 8 fills one 8-row tile and one read of a
// KV page serves the whole GQA group.
constexpr int kTileTokens = 64;  // KV tokens per pipeline stage (4 warps x 16)
constexpr int kPrefillRows = 128;  // rows of one prefill tile (the M of a tcgen05.mma)

// Work item of the split-KV kernel: one (sequence, row tile, KV chunk); the kv head is the fastest
// index of the flattened work id, so neighbouring CTAs read neighbouring heads of the same page.
struct Unit {
  int32_t seq;
  int32_t row0;      // first row of the tile in (q_token*G+g) space
  int32_t kv_begin;  // first key of the chunk (multiple of kTileTokens)
  int32_t kv_end;    // one past the last key of the chunk
  int32_t slot;      // partial slot, or -1: the chunk is the whole range, write the output directly
  int32_t q_start;   // query_start_loc[seq]
  int32_t q_len;
  int32_t kv_len;
  int32_t merge_idx;  // index of the tile's MergeItem (chunks > 1), else -1
  int32_t chunk_idx;  // which chunk of the tile this is
  int32_t n_chunks;
  int32_t pad;
};
static_assert(sizeof(Unit) == 48, "Unit is read as three 16-byte words");

// One row tile whose chunks must be combined (by the last chunk to finish, or by the merge kernel).
struct MergeItem {
  int32_t row0;
  int32_t slot0;     // partial slots slot0 .. slot0+n_chunks-1
  int32_t n_chunks;
  int32_t q_start;
  int32_t q_len;
  int32_t pad[3];
};

// int32 header at the start of the workspace, written by the planner.
enum HeaderWord {
  kHdrNumUnits = 0,
  kHdrNumMerge = 1,
  kHdrChunk = 2,
  kHdrQueue = 3,      // work queue head of the gather kernel
  kHdrNumSlots = 4,
  kHdrTotalKeys = 5,
  kHdrNumPrefill = 6,     // work items of the tcgen05 prefill-tile kernel
  kHdrPrefillQueue = 7,   // its work queue head
  kHdrPrefillStages = 8,  // sum of the items' 64-token KV stages (per kv head)
  kHdrTailStart = 9,      // first row of `out` past the last sequence: rows [this, T) are zero-filled
  kHdrWords = 64,
};

struct WorkspaceLayout {
  size_t header_off, units_off, merge_off, part_o_off, part_ml_off, punits_off, tickets_off, total;
  // optional tail, used when the caller's workspace has room for it (total_split bytes): prefill items are
  // then cut along KV at CTA-quota boundaries and their parts combined by the part that finishes last
  size_t pprefix_off, ptickets_off, ppart_ml_off, ppart_o_off, total_split;
  int32_t ppart_slots;
  int32_t max_units, max_merge, max_slots, rows_per_tile, target_units, target_units_max, max_punits;
};

struct Params {
  const void* q;
  const void* kv;        // interleaved pool [P, page, 2*Hkv, D], or the key cache when v_cache is set
  const void* v_cache;   // null, or the value cache of the split layout [P, Hkv, page, D] (page_attention)
  const int32_t* context_lens;
  const int32_t* block_tables;
  const int32_t* query_start_loc;
  const int32_t* num_seqs;
  const float* sinks;
  void* out;
  int32_t* header;
  Unit* units;
  Unit* punits;    // prefill items: row0 is a multiple of prefill_item_rows, slot unused
  MergeItem* merge;
  // KV split of prefill items (all null / 0 when off)
  int32_t* pprefix;   // [num prefill items + 1] exclusive prefix of the items' stage counts, queue order
  int32_t* ptickets;  // [items][Hkv][tiles][4 row quarters] arrival counters, zeroed by the planner
  float2* ppart_ml;   // [2 * CTAs][tiles][128] (m, l) of a part
  float* ppart_o;     // [2 * CTAs][tiles][128][D] unnormalised O of a part
  int32_t prefill_split;
  int32_t* tickets; // [max_merge][Hkv] arrival counters of the chunks of one (tile, kv head); zeroed by the planner
  int32_t fused_merge; // 1: the split-KV kernel combines the chunks itself (last arriver), no merge kernel
  float* part_o;   // [max_slots][Hkv][rows_per_tile][D]
  float2* part_ml; // [max_slots][Hkv][rows_per_tile]  (m in log2 domain, l)
  int32_t* status; // may be null
  int32_t T, S_max, pages_per_seq, num_pages, page_size, Hq, Hkv, G, D;
  int32_t rows_per_tile;
  int32_t max_units, max_merge, max_slots, target_units, min_chunk;
  int32_t target_units_max;  // the planner may aim for this many items instead (see its pass 1); sizes the workspace
  int32_t max_punits;
  int32_t prefill_item_rows; // rows one prefill work item covers (128 per tile, 1 or 2 tiles per CTA)
  int32_t Dkv;               // elements between consecutive combined heads of kv_pages (head_dim, or the padded
                             // head_dim of a v3 cache)
  int32_t Dq;                // elements of a row of queries / out: D, except for an e4m3 v3 cache of head_dim 64, whose rows
                             // are padded to 128 bytes and are attended as head_dim 128 (the queries' upper half reads as zeros)
  int32_t C2;                // combined heads per token row in memory: 2 * Hkv, or more in a v3 cache that pads them to
                             // a multiple of the packing (four e4m3 heads per 32-bit word)
  int32_t sort_items;        // 1: split-KV work items are queued longest first, 0: in sequence order
  int32_t test_withhold;     // test hook: bit 0 / bit 1 = the CTA of the split-KV / prefill kernel that takes work item 0
                             // never announces the item's first KV stage, so that the waits on it run out
                             // (EJK_RPA_ST_TIMEOUT); 0 in production
  int32_t pdl;               // bit 0: the prefill kernel, bit 1: the split-KV kernel must pdl_wait() before reading the plan
  int32_t prefill_min_rows;  // sequences with q_len*G >= this go to the prefill-tile kernel; 0 = never
  int32_t prefill_share;     // percent: in a mixed batch the tile kernel keeps this share of the CTAs its estimate asks for (0 = all CTAs always)
  int32_t window;      // <= 0: none
  int32_t num_sinks, sink_rows;
  int32_t kv8;         // 1: the cache holds e4m3 bytes (queries / out keep their 16-bit dtype)
  float inv_q_scale;   // e4m3 cache only: != 0 quantises the staged queries to e4m3 after multiplying by this
  float out_scale;     // factor on the normalised output (v_scale of the v3 operator), 1 otherwise
  float scale;         // softmax_scale
  float scale_log2;    // softmax_scale * log2(e)
  float cap;           // 0: none
  float cap_log2;      // cap * log2(e)
  float inv_cap_scale; // softmax_scale / cap
  int32_t page_shift;  // log2(page_size) if a power of two, else -1
  int32_t tma_block_tokens;  // tokens per TMA box = min(page_size, kTileTokens)
  int32_t tma_block_shift;   // log2 of the above
  int32_t wait_timeout_ms;   // wall-time bound of every in-kernel mbarrier wait
};

// launchers (each returns cudaError_t of the launch)
cudaError_t launch_plan(const Params& p, cudaStream_t stream, bool pdl);
cudaError_t launch_splitkv(const Params& p, int dtype, int n_sm, cudaStream_t stream);
bool tma_path_supported(const Params& p);
cudaError_t launch_splitkv_tma(const Params& p, int dtype, int n_sm, cudaStream_t stream, bool pdl);
// Params conventions for the split layout (page_attention): query_start_loc == nullptr means one
// query row per sequence (row s belongs to sequence s); num_seqs == nullptr means all S_max sequences.
bool prefill_path_supported(const Params& p);
int prefill_rows_per_item(int head_dim);
cudaError_t launch_prefill(const Params& p, int dtype, int n_sm, cudaStream_t stream, bool pdl);

// <<<>>> with, optionally, the programmatic-stream-serialization attribute: the kernel may then begin
// while the previous kernel of the stream is still running (see pdl_wait / pdl_trigger).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
cudaError_t launch_merge(const Params& p, int dtype, int n_sm, cudaStream_t stream, bool pdl);
// read-only streaming probe (rpa_stream_probe.cu): reads `bytes` (rounded down to whole 32 KiB chunks) into shared memory
cudaError_t launch_stream_probe(const void* src, size_t bytes, unsigned* sink, int n_sm, int wait_ms, int chunk_kb, int slots,
                                int ctas_per_sm, cudaStream_t stream);
cudaError_t launch_kv_update(const void* k_new, const void* v_new, void* cache, const int32_t* kv_lens,
                             const int32_t* block_tables, const int32_t* query_start_loc, const int32_t* num_seqs,
                             int32_t* status, int T, int S_max, int pages_per_seq, int num_pages, int page_size, int Hkv,
                             int C2, int D, int Dalign, int elem_bytes, cudaStream_t stream);

}  // namespace ejk
