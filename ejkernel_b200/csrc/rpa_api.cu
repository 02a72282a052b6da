// C ABI of the ragged paged attention path (declared in include/ejk_rpa.h).
#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>

#include "rpa_types.h"

namespace ejk {
namespace {

// Process-wide options.  Atomic because ejk_rpa_set_option may be called from one host thread while another
// launches; a launch reads each option once.
struct Options {
  std::atomic<int> waves{4};           // split-KV work items per CTA (with longest-first queueing, fewer and longer items win)
  std::atomic<int> min_chunk{256};
  std::atomic<int> path{0};
  std::atomic<int> profile{0};
  std::atomic<int> prefill_split{1};   // prefill items are cut along KV at CTA-quota boundaries (needs the larger workspace)
  std::atomic<int> sort_items{1};      // split-KV work items longest first
  std::atomic<int> test_withhold{0};   // test hook, see Params::test_withhold
  std::atomic<int> overlap{1};         // programmatic dependent launches: kernels of one call overlap where they are independent
  std::atomic<int> fused_merge{1};     // the TMA split-KV kernel combines the chunks of a tile itself (no merge kernel)
  std::atomic<int> wait_ms{2000};      // bound of every in-kernel wait; expiry sets EJK_RPA_ST_TIMEOUT
  // Sequences with at least this many (token, head-in-group) rows use 128-row tensor tiles.  8-row split-KV
  // tiles re-read a sequence's KV once per tile, so from four tiles on (8 query tokens at G = 4) the
  // tensor-tile kernel, which reads it once, is faster even with three quarters of its rows empty:
  // 256 x 8 tokens at kv 128..8192 1.45 -> 1.18 ms, 256 x 12 tokens 2.16 -> 1.22 ms; at 17-31 rows it
  // depends on the lengths (faster at kv <= 1024, 7 % slower on long ragged contexts).
  std::atomic<int> prefill_rows{32};
  std::atomic<int> prefill_share{125};
  // shape of the read-only streaming probe (0 = its defaults): KB per copy, slots per CTA, CTAs per SM
  std::atomic<int> probe_chunk_kb{0}, probe_slots{0}, probe_ctas{0};  // see Params::prefill_share; 0 = the tile kernel always uses every SM
};
Options g_opt;
thread_local int t_last_launches = 0;

// cudaEvents around the three kernels of a launch; only touched when option "profile" is 1
struct ProfileEvents {  // before the planner, after it, after the prefill-tile kernel, after the split-KV kernel, after the merge
  cudaEvent_t ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
  bool created = false, recorded = false;
  int device = -1;  // the device the events belong to (events cannot time work of another device)
};
thread_local ProfileEvents t_prof;

struct DeviceInfo {
  std::atomic<bool> known{false};
  int sm_count = 0;
  int cc_major = 0;
};
DeviceInfo g_dev[64];
std::mutex g_dev_mutex;  // first-use set-up per device; launches may come from several host threads

const DeviceInfo* device_info() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  DeviceInfo& d = g_dev[dev];
  if (!d.known.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    if (!d.known.load(std::memory_order_relaxed)) {
      int sm = 0, cc = 0;
      if (cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
      if (cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return nullptr;
      d.sm_count = sm;
      d.cc_major = cc;
      d.known.store(true, std::memory_order_release);
    }
  }
  return &d;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int check_shape(const ejk_rpa_shape* s) {
  if (!s) return EJK_RPA_E_NULL;
  if (s->total_tokens <= 0 || s->max_num_seqs <= 0 || s->pages_per_seq <= 0 || s->num_pages <= 0 ||
      s->page_size <= 0 || s->num_q_heads <= 0 || s->num_kv_heads <= 0)
    return EJK_RPA_E_SHAPE;
  if (s->num_q_heads % s->num_kv_heads != 0) return EJK_RPA_E_SHAPE;
  if (s->head_dim != 64 && s->head_dim != 128 && s->head_dim != 256) return EJK_RPA_E_HEAD_DIM;
  if (s->dtype != EJK_RPA_BF16 && s->dtype != EJK_RPA_F16) return EJK_RPA_E_DTYPE;
  if ((long long)s->pages_per_seq * s->page_size > 0x3fffffffLL) return EJK_RPA_E_SHAPE;
  // row, tile and work-item counts are 32-bit in the planner and the work lists
  if ((long long)s->total_tokens * s->num_q_heads > 0x3fffffffLL || s->max_num_seqs > 0x00ffffff) return EJK_RPA_E_SHAPE;
  if (s->kv_dtype != 0 && s->kv_dtype != EJK_RPA_E4M3) return EJK_RPA_E_DTYPE;
  if (s->kv_dtype == EJK_RPA_E4M3) {
    // head_dim 64 only in the v3 cache, whose rows are padded to 128 bytes (launch_impl checks the row stride)
    if (s->page_size < 8 || s->page_size % 8 != 0) return EJK_RPA_E_SHAPE;
  }
  return 0;
}

// Everything is sized from static shapes: the planner never needs more than
//   target_units + max_tiles   work items / partial slots   (sum_t ceil(L_t/C) <= sum L/C + tiles)
WorkspaceLayout layout_for(const ejk_rpa_shape& s, int n_sm) {
  WorkspaceLayout L;
  const int G = s.num_q_heads / s.num_kv_heads;
  L.rows_per_tile = (G > 8) ? 16 : 8;
  const long long rows = (long long)s.total_tokens * G;
  const long long max_tiles = rows / L.rows_per_tile + s.max_num_seqs;
  const int ctas = n_sm * 2;
  long long tgt = ((long long)ctas * g_opt.waves + s.num_kv_heads - 1) / s.num_kv_heads;
  if (tgt < 1) tgt = 1;
  L.target_units = (int)tgt;
  L.target_units_max = (int)(2 * tgt);  // what the planner switches to when every row tile gets many chunks
  L.max_units = (int)(2 * tgt + max_tiles);
  L.max_merge = (int)max_tiles;
  L.max_slots = (int)(2 * tgt + max_tiles);
  L.max_punits = (int)(rows / kPrefillRows + s.max_num_seqs);
  size_t off = 0;
  L.header_off = off;
  off = align_up(off + kHdrWords * sizeof(int32_t), 256);
  L.units_off = off;
  off = align_up(off + (size_t)L.max_units * sizeof(Unit), 256);
  L.merge_off = off;
  off = align_up(off + (size_t)L.max_merge * sizeof(MergeItem), 256);
  L.punits_off = off;
  off = align_up(off + (size_t)L.max_punits * sizeof(Unit), 256);
  L.tickets_off = off;
  off = align_up(off + (size_t)L.max_merge * s.num_kv_heads * sizeof(int32_t), 256);
  L.part_ml_off = off;
  off = align_up(off + (size_t)L.max_slots * s.num_kv_heads * L.rows_per_tile * sizeof(float2), 256);
  L.part_o_off = off;
  // an e4m3 cache of head_dim 64 is attended as head_dim 128 (its rows are padded to 128 bytes): partials are that wide
  const int d_part = (s.kv_dtype == EJK_RPA_E4M3 && s.head_dim == 64) ? 128 : s.head_dim;
  off = align_up(off + (size_t)L.max_slots * s.num_kv_heads * L.rows_per_tile * d_part * sizeof(float), 256);
  L.total = off;
  {
    const int nt = prefill_rows_per_item(s.head_dim) / kPrefillRows;
    L.ppart_slots = 2 * n_sm;
    L.pprefix_off = off;
    off = align_up(off + ((size_t)L.max_punits + 1) * sizeof(int32_t), 256);
    L.ptickets_off = off;
    off = align_up(off + (size_t)L.max_punits * s.num_kv_heads * nt * 4 * sizeof(int32_t), 256);
    L.ppart_ml_off = off;
    off = align_up(off + (size_t)L.ppart_slots * nt * kPrefillRows * sizeof(float2), 256);
    L.ppart_o_off = off;
    off = align_up(off + (size_t)L.ppart_slots * nt * kPrefillRows * s.head_dim * sizeof(float), 256);
    L.total_split = off;
  }
  return L;
}

}  // namespace
}  // namespace ejk

using namespace ejk;

extern "C" {

int ejk_rpa_version(void) { return EJK_RPA_VERSION; }

const char* ejk_rpa_error_string(int code) {
  switch (code) {
    case 0: return "ok";
    case EJK_RPA_E_NULL: return "a required pointer is null";
    case EJK_RPA_E_SHAPE: return "invalid shape (non-positive dimension, num_q_heads % num_kv_heads != 0, or kv capacity too large)";
    case EJK_RPA_E_HEAD_DIM: return "head_dim must be 64, 128 or 256";
    case EJK_RPA_E_DTYPE: return "dtype must be bf16 or f16";
    case EJK_RPA_E_WORKSPACE: return "workspace too small or not 256-byte aligned";
    case EJK_RPA_E_ARG: return "invalid attribute (sliding_window, logits_soft_cap, softmax_aux or option name)";
    case EJK_RPA_E_DEVICE: return "current CUDA device is not an sm_100-class GPU";
    case EJK_RPA_E_ALIGN: return "queries, kv_pages and out must be 16-byte aligned";
    case EJK_RPA_E_SCRATCH:
      return "this shape needs more scratch than the library's built-in static buffer holds "
             "(EJK_RPA_STATIC_SCRATCH_BYTES); use ejk_rpa_launch with a caller-provided workspace";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown error code";
}

size_t ejk_rpa_workspace_bytes(const ejk_rpa_shape* shape) {
  if (check_shape(shape) != 0) return 0;
  const DeviceInfo* d = device_info();
  if (!d) return 0;
  const WorkspaceLayout L = layout_for(*shape, d->sm_count);
  // shapes that can hold a multi-token sequence also get room for the KV split of prefill items; a
  // launch with only L.total bytes still works, without that split
  const bool multi = shape->total_tokens > shape->max_num_seqs;
  const int ps = shape->page_size;
  return (multi && ps >= 8 && ps % 8 == 0) ? L.total_split : L.total;
}

// Shared body of the launch entry points.  `value_cache` != null selects the split cache layout
// (kv_pages is then the key cache); with it, null query_start_loc / num_seqs mean "one query row per
// sequence, all sequences".
// Every host-side check of a launch, with nothing enqueued: entry points that enqueue work of their own
// before the attention kernels (the v3 page write) call it first, so that an invalid argument returns its
// negative code with no kernel launched and nothing modified.  `workspace` may be null when the caller
// supplies it later (workspace_bytes is then not checked either).
static int validate(const void* queries, const void* kv_pages, const void* value_cache, const int32_t* context_lens,
                    const int32_t* block_tables, const int32_t* query_start_loc, const int32_t* num_seqs,
                    const float* softmax_aux, const void* out, const void* workspace, size_t workspace_bytes,
                    bool need_workspace, const ejk_rpa_shape* shape, const ejk_rpa_attrs* attrs,
                    const DeviceInfo** dev_out) {
  if (!queries || !kv_pages || !context_lens || !block_tables || !out || !shape || !attrs) return EJK_RPA_E_NULL;
  if (need_workspace && !workspace) return EJK_RPA_E_NULL;
  if (!value_cache && (!query_start_loc || !num_seqs)) return EJK_RPA_E_NULL;
  if (int e = check_shape(shape)) return e;
  const ejk_rpa_shape& s = *shape;
  const ejk_rpa_attrs& a = *attrs;
  if (!(a.softmax_scale == a.softmax_scale) || std::isinf(a.softmax_scale)) return EJK_RPA_E_ARG;
  if (!(a.logits_soft_cap == a.logits_soft_cap) || std::isinf(a.logits_soft_cap)) return EJK_RPA_E_ARG;
  if (!(a.out_scale == a.out_scale) || std::isinf(a.out_scale)) return EJK_RPA_E_ARG;
  if (!(a.q_scale == a.q_scale) || std::isinf(a.q_scale) || a.q_scale < 0.f) return EJK_RPA_E_ARG;
  if (a.q_scale != 0.f && (value_cache || g_opt.path == 1)) return EJK_RPA_E_ARG;  // done where the TMA kernel stages Q
  if (s.kv_dtype == EJK_RPA_E4M3 && (value_cache || g_opt.path == 1)) return EJK_RPA_E_ARG;
  if (a.num_sinks < 0 || (a.num_sinks > 0 && !softmax_aux)) return EJK_RPA_E_ARG;
  if (a.num_sinks > 0 && a.sink_rows != s.num_q_heads && a.sink_rows != s.num_kv_heads && a.sink_rows != 1)
    return EJK_RPA_E_ARG;
  if ((reinterpret_cast<uintptr_t>(queries) | reinterpret_cast<uintptr_t>(kv_pages) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return EJK_RPA_E_ALIGN;
  const DeviceInfo* d = device_info();
  if (!d) return EJK_RPA_E_DEVICE;
  if (d->cc_major != 10) return EJK_RPA_E_DEVICE;
  if (need_workspace) {
    const WorkspaceLayout L = layout_for(s, d->sm_count);
    if (workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return EJK_RPA_E_WORKSPACE;
  }
  if (g_opt.path == 2 || a.q_scale != 0.f || s.kv_dtype == EJK_RPA_E4M3) {
    // the TMA gather was forced, or is the only kernel that serves the call (re-rounded queries, e4m3 cache):
    // refuse here, before anything is enqueued, what it cannot serve
    Params probe;
    std::memset(&probe, 0, sizeof(probe));
    probe.page_size = s.page_size;
    if (!tma_path_supported(probe)) return EJK_RPA_E_ARG;
  }
  if (dev_out) *dev_out = d;
  return 0;
}

static int launch_impl(const void* queries, const void* kv_pages, const void* value_cache, const int32_t* context_lens,
                       const int32_t* block_tables, const int32_t* query_start_loc, const int32_t* num_seqs,
                       const float* softmax_aux, void* out, void* workspace, size_t workspace_bytes,
                       int32_t* status, const ejk_rpa_shape* shape, const ejk_rpa_attrs* attrs, void* stream,
                       int kv_dim = 0, int kv_heads_alloc = 0) {
  t_last_launches = 0;
  const DeviceInfo* d = nullptr;
  if (int e = validate(queries, kv_pages, value_cache, context_lens, block_tables, query_start_loc, num_seqs,
                       softmax_aux, out, workspace, workspace_bytes, true, shape, attrs, &d))
    return e;
  const ejk_rpa_shape& s = *shape;
  const ejk_rpa_attrs& a = *attrs;
  const WorkspaceLayout L = layout_for(s, d->sm_count);

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  Params p;
  std::memset(&p, 0, sizeof(p));
  p.q = queries;
  p.kv = kv_pages;
  p.v_cache = value_cache;
  p.context_lens = context_lens;
  p.block_tables = block_tables;
  p.query_start_loc = query_start_loc;
  p.num_seqs = num_seqs;
  p.sinks = softmax_aux;
  p.out = out;
  p.header = reinterpret_cast<int32_t*>(ws + L.header_off);
  p.units = reinterpret_cast<Unit*>(ws + L.units_off);
  p.punits = reinterpret_cast<Unit*>(ws + L.punits_off);
  p.merge = reinterpret_cast<MergeItem*>(ws + L.merge_off);
  p.tickets = reinterpret_cast<int32_t*>(ws + L.tickets_off);
  if (workspace_bytes >= L.total_split && g_opt.prefill_split) {
    p.pprefix = reinterpret_cast<int32_t*>(ws + L.pprefix_off);
    p.ptickets = reinterpret_cast<int32_t*>(ws + L.ptickets_off);
    p.ppart_ml = reinterpret_cast<float2*>(ws + L.ppart_ml_off);
    p.ppart_o = reinterpret_cast<float*>(ws + L.ppart_o_off);
    p.prefill_split = g_opt.prefill_split;
  }
  p.part_o = reinterpret_cast<float*>(ws + L.part_o_off);
  p.part_ml = reinterpret_cast<float2*>(ws + L.part_ml_off);
  p.status = status;
  p.T = s.total_tokens;
  p.S_max = s.max_num_seqs;
  p.pages_per_seq = s.pages_per_seq;
  p.num_pages = s.num_pages;
  p.page_size = s.page_size;
  p.Hq = s.num_q_heads;
  p.Hkv = s.num_kv_heads;
  p.G = s.num_q_heads / s.num_kv_heads;
  p.D = s.head_dim;
  p.Dq = s.head_dim;
  p.Dkv = kv_dim > 0 ? kv_dim : s.head_dim;
  if (s.kv_dtype == EJK_RPA_E4M3 && s.head_dim == 64) {
    // 64 e4m3 bytes are half a 128-byte swizzle row: served only where the cache pads the row to 128 bytes (the v3
    // layout), as head_dim 128 with the queries' upper half zero; the padding lanes of K meet those zeros, those of
    // V land in output columns that are not stored
    if (p.Dkv != 128) return EJK_RPA_E_HEAD_DIM;
    p.D = 128;
  }
  p.C2 = kv_heads_alloc > 0 ? kv_heads_alloc : 2 * s.num_kv_heads;
  p.rows_per_tile = L.rows_per_tile;
  p.max_units = L.max_units;
  p.max_merge = L.max_merge;
  p.max_slots = L.max_slots;
  p.max_punits = L.max_punits;
  p.target_units = L.target_units;
  p.target_units_max = L.target_units_max;
  // Per-call tile hints of the reference's RaggedPageAttentionConfig (configs.py:242-258) override
  // the process-wide options: num_kv_pages_per_block = smallest KV chunk a row tile is split into
  // (in pages; rounded up to whole 64-token stages), num_queries_per_block = query tokens from
  // which on a sequence is served by 128-row tensor tiles.
  p.min_chunk = g_opt.min_chunk;
  if (a.num_kv_pages_per_block > 0) {
    long long c = (long long)a.num_kv_pages_per_block * s.page_size;
    c = ((c + kTileTokens - 1) / kTileTokens) * kTileTokens;
    if (c > 0x40000000ll) c = 0x40000000ll;
    p.min_chunk = (int)c;
  }
  int prefill_rows = g_opt.prefill_rows;
  if (a.num_queries_per_block > 0) {
    const long long r = (long long)a.num_queries_per_block * (s.num_q_heads / s.num_kv_heads);
    prefill_rows = r > 0x40000000ll ? 0x40000000 : (int)r;
  }
  p.window = a.sliding_window > 0 ? a.sliding_window : 0;
  p.num_sinks = a.num_sinks;
  p.sink_rows = a.sink_rows;
  const float log2e = 1.4426950408889634f;
  p.out_scale = (a.out_scale != 0.f) ? a.out_scale : 1.f;
  p.kv8 = s.kv_dtype == EJK_RPA_E4M3;
  p.inv_q_scale = (a.q_scale != 0.f) ? 1.f / a.q_scale : 0.f;
  p.scale = a.softmax_scale;
  p.scale_log2 = a.softmax_scale * log2e;
  p.cap = a.logits_soft_cap;
  p.cap_log2 = a.logits_soft_cap * log2e;
  p.inv_cap_scale = (a.logits_soft_cap != 0.f) ? a.softmax_scale / a.logits_soft_cap : 0.f;
  p.page_shift = -1;
  if ((s.page_size & (s.page_size - 1)) == 0) {
    int sh = 0;
    while ((1 << sh) < s.page_size) ++sh;
    p.page_shift = sh;
  }

  // tokens per TMA box: the largest power of two that divides the page size, at most one 64-token stage -- a box
  // never straddles a page, and boxes are whole 8-token swizzle atoms (page sizes that are no multiple of 8 take
  // the cp.async gather).  16 -> 16, 128 -> 64, 24 -> 8, 48 -> 16.
  p.tma_block_tokens = 1;
  while (p.tma_block_tokens < kTileTokens && s.page_size % (p.tma_block_tokens * 2) == 0) p.tma_block_tokens *= 2;
  p.tma_block_shift = 0;
  while ((1 << p.tma_block_shift) < p.tma_block_tokens) ++p.tma_block_shift;
  p.wait_timeout_ms = g_opt.wait_ms;
  p.test_withhold = g_opt.test_withhold;
  p.sort_items = g_opt.sort_items;
  const bool use_tma = (g_opt.path == 2) || (g_opt.path == 0 && tma_path_supported(p));
  if (use_tma && !tma_path_supported(p)) return EJK_RPA_E_ARG;
  // Batches that can hold a sequence with many query rows also get the tcgen05 prefill-tile
  // kernel; whether any sequence actually qualifies is decided by the planner on the device.
  if ((p.kv8 || p.inv_q_scale != 0.f) && !use_tma) return EJK_RPA_E_ARG;
  // an e4m3 cache and re-rounded queries (q_scale) are served by the split-KV kernel alone
  const bool use_prefill = use_tma && !p.kv8 && p.inv_q_scale == 0.f && prefill_rows > 0 && prefill_path_supported(p) &&
                           (long long)s.total_tokens * p.G >= prefill_rows &&
                           s.total_tokens > s.max_num_seqs;  // more query rows than sequences: some are multi-token
  p.prefill_min_rows = use_prefill ? prefill_rows : 0;
  p.prefill_share = g_opt.prefill_share;
  // The last-arriver merge inside the split-KV kernel saves a launch, but the chunk that arrives last
  // combines its tile alone: with many chunks per tile (few query rows, long contexts) the separate
  // merge kernel, which spreads the rows over the whole GPU, is faster.  Decided from static shapes:
  // fused when a tile can get at most ~2 chunks -- on average over the batch (work items per query
  // token) or because the longest possible context is that short.  (Option value 2 forces it.)
  {
    const long long max_kv = (long long)s.pages_per_seq * s.page_size;
    const long long by_len = (max_kv + p.min_chunk - 1) / p.min_chunk;
    const bool few = (long long)L.target_units <= 2ll * s.total_tokens || by_len <= 2;
    p.fused_merge = (use_tma && (g_opt.fused_merge == 2 || (g_opt.fused_merge == 1 && few))) ? 1 : 0;
  }
  p.prefill_item_rows = prefill_rows_per_item(s.head_dim);

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool prof = g_opt.profile != 0;
  if (prof) {
    int dev = -1;
    if (cudaError_t ce = cudaGetDevice(&dev); ce != cudaSuccess) return static_cast<int>(ce);
    if (t_prof.created && t_prof.device != dev) {  // the thread moved to another GPU: its events stay behind
      for (auto& ev : t_prof.ev) cudaEventDestroy(ev);
      t_prof.created = false;
    }
    if (!t_prof.created) {
      for (auto& ev : t_prof.ev)
        if (cudaError_t ce = cudaEventCreate(&ev); ce != cudaSuccess) return static_cast<int>(ce);
      t_prof.created = true;
      t_prof.device = dev;
    }
  }
  t_prof.recorded = false;
  if (prof) cudaEventRecord(t_prof.ev[0], st);
  // Programmatic dependent launches (not while profiling: the event records in between would
  // serialise the kernels anyway).  The prefill kernel starts under the planner's tail and waits for
  // the plan on the device; the split-KV kernel starts as soon as every prefill CTA has seen the plan
  // and takes over the SMs that prefill CTAs leave -- the two kernels write different rows.  Without
  // a prefill kernel the split-KV kernel is the planner's dependent and waits for the plan itself.
  const bool pdl = g_opt.overlap != 0 && !prof && use_tma;
  p.pdl = pdl ? (use_prefill ? 1 : 2) : 0;
  cudaError_t e = launch_plan(p, st, pdl);
  if (e != cudaSuccess) return static_cast<int>(e);
  ++t_last_launches;
  if (prof) cudaEventRecord(t_prof.ev[1], st);
  if (use_prefill) {
    e = launch_prefill(p, s.dtype, d->sm_count, st, pdl);
    if (e != cudaSuccess) return static_cast<int>(e);
    ++t_last_launches;
  }
  if (prof) cudaEventRecord(t_prof.ev[2], st);
  e = use_tma ? launch_splitkv_tma(p, s.dtype, d->sm_count, st, pdl) : launch_splitkv(p, s.dtype, d->sm_count, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  ++t_last_launches;
  if (prof) cudaEventRecord(t_prof.ev[3], st);
  if (!p.fused_merge) {
    e = launch_merge(p, s.dtype, d->sm_count, st, pdl);
    if (e != cudaSuccess) return static_cast<int>(e);
    ++t_last_launches;
  }
  if (prof) {
    cudaEventRecord(t_prof.ev[4], st);
    t_prof.recorded = true;
  }
  return 0;
}

size_t ejk_rpa_workspace_bytes_min(const ejk_rpa_shape* shape) {
  if (check_shape(shape) != 0) return 0;
  const DeviceInfo* d = device_info();
  if (!d) return 0;
  return layout_for(*shape, d->sm_count).total;
}

int ejk_rpa_launch(const void* queries, const void* kv_pages, const int32_t* context_lens,
                   const int32_t* block_tables, const int32_t* query_start_loc, const int32_t* num_seqs,
                   const float* softmax_aux, void* out, void* workspace, size_t workspace_bytes,
                   int32_t* status, const ejk_rpa_shape* shape, const ejk_rpa_attrs* attrs, void* stream) {
  return launch_impl(queries, kv_pages, nullptr, context_lens, block_tables, query_start_loc, num_seqs, softmax_aux, out,
                     workspace, workspace_bytes, status, shape, attrs, stream);
}

int ejk_page_attention_launch(const void* query, const void* key_cache, const void* value_cache,
                              const int32_t* context_lens, const int32_t* block_tables, void* out, void* workspace,
                              size_t workspace_bytes, int32_t* status, const ejk_rpa_shape* shape,
                              const ejk_rpa_attrs* attrs, void* stream) {
  t_last_launches = 0;
  if (!value_cache) return EJK_RPA_E_NULL;
  if (shape && shape->total_tokens != shape->max_num_seqs) return EJK_RPA_E_SHAPE;  // one query row per sequence
  if (reinterpret_cast<uintptr_t>(value_cache) & 15) return EJK_RPA_E_ALIGN;
  return launch_impl(query, key_cache, value_cache, context_lens, block_tables, nullptr, nullptr, nullptr, out, workspace,
                     workspace_bytes, status, shape, attrs, stream);
}

int ejk_rpa_v3_launch(const void* queries, const void* keys, const void* values, void* kv_cache,
                      const int32_t* kv_lens, const int32_t* block_tables, const int32_t* query_start_loc,
                      const int32_t* distribution, void* out, void* workspace, size_t workspace_bytes, int32_t* status,
                      const ejk_rpa_shape* shape, const ejk_rpa_attrs* attrs, void* stream) {
  t_last_launches = 0;
  if (!keys || !values || !kv_cache || !distribution) return EJK_RPA_E_NULL;
  // every host check of the attention launch comes before the page write: a call that is going to be refused
  // must not have modified the cache (a retry would apply the write twice) nor have launched anything
  if (int e = validate(queries, kv_cache, nullptr, kv_lens, block_tables, query_start_loc, distribution + 2, nullptr, out,
                       workspace, workspace_bytes, true, shape, attrs, nullptr))
    return e;
  // the v3 cache pads head_dim to a multiple of 128 (align_to(D, 128), _kernel.py:45-57); the page write
  // zero-fills the padding like merge_kv does and the attention kernels step over it
  const int d_align = (shape->head_dim + 127) / 128 * 128;
  if ((reinterpret_cast<uintptr_t>(keys) | reinterpret_cast<uintptr_t>(values)) & 15) return EJK_RPA_E_ALIGN;
  const int32_t* num_seqs = distribution + 2;  // distribution = (decode_end, prefill_end, num_seqs), _kernel.py:211
  // the cache also pads the combined heads to a multiple of the packing -- 32 bits' worth of elements, i.e. 2 at 16
  // bits (never any padding) and 4 for e4m3 (an odd number of kv heads leaves two padding heads), _kernel.py:45-57
  const int pack = shape->kv_dtype == EJK_RPA_E4M3 ? 4 : 2;
  const int c2 = (2 * shape->num_kv_heads + pack - 1) / pack * pack;
  cudaError_t ce = launch_kv_update(keys, values, kv_cache, kv_lens, block_tables, query_start_loc, num_seqs, status,
                                    shape->total_tokens, shape->max_num_seqs, shape->pages_per_seq, shape->num_pages,
                                    shape->page_size, shape->num_kv_heads, c2, shape->head_dim, d_align,
                                    shape->kv_dtype == EJK_RPA_E4M3 ? 1 : 2, static_cast<cudaStream_t>(stream));
  if (ce != cudaSuccess) return static_cast<int>(ce);
  const int rc = launch_impl(queries, kv_cache, nullptr, kv_lens, block_tables, query_start_loc, num_seqs, nullptr, out,
                             workspace, workspace_bytes, status, shape, attrs, stream, d_align, c2);
  if (rc == 0) ++t_last_launches;
  return rc;
}

// ---------------------------------------------------------------------------------------------
// Launch without a caller-provided workspace.
//
// The scratch (work list, merge list, split-KV partials) lives in this file-scope device array,
// so the call path contains no allocation of any kind.  The array is part of the loaded module:
// every GPU that loads the library holds EJK_RPA_STATIC_SCRATCH_BYTES of it until the process
// exits.  In host code the name `g_static_scratch` is only a handle for the runtime, not a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, looked up once per device
// (with that device current) on the first call there.
static __device__ __align__(256) unsigned char g_static_scratch[EJK_RPA_STATIC_SCRATCH_BYTES];

namespace {
std::atomic<void*> g_static_scratch_ptr[64];
}

int ejk_rpa_launch_static_scratch(const void* queries, const void* kv_pages, const int32_t* context_lens,
                                  const int32_t* block_tables, const int32_t* query_start_loc,
                                  const int32_t* num_seqs, const float* softmax_aux, void* out, int32_t* status,
                                  const ejk_rpa_shape* shape, const ejk_rpa_attrs* attrs, void* stream) {
  t_last_launches = 0;
  if (g_opt.profile) return EJK_RPA_E_ARG;  // the profiling hook creates CUDA events; not on this path
  // the same argument and device checks as ejk_rpa_launch, before anything touches the runtime: a null
  // pointer or a GPU of another generation gets its EJK_RPA_E_* code, not a raw CUDA error from the look-up
  const DeviceInfo* d = nullptr;
  if (int e = validate(queries, kv_pages, nullptr, context_lens, block_tables, query_start_loc, num_seqs, softmax_aux,
                       out, nullptr, 0, false, shape, attrs, &d))
    return e;
  if (layout_for(*shape, d->sm_count).total > (size_t)EJK_RPA_STATIC_SCRATCH_BYTES) return EJK_RPA_E_SCRATCH;
  int dev = 0;
  if (cudaError_t ce = cudaGetDevice(&dev); ce != cudaSuccess) return static_cast<int>(ce);
  if (dev < 0 || dev >= 64) return EJK_RPA_E_DEVICE;
  void* ptr = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    // two host threads may both get here on their first call: both look up the same address
    if (cudaError_t ce = cudaGetSymbolAddress(&ptr, g_static_scratch); ce != cudaSuccess) return static_cast<int>(ce);
    g_static_scratch_ptr[dev].store(ptr, std::memory_order_release);
  }
  return ejk_rpa_launch(queries, kv_pages, context_lens, block_tables, query_start_loc, num_seqs, softmax_aux, out, ptr,
                        (size_t)EJK_RPA_STATIC_SCRATCH_BYTES, status, shape, attrs, stream);
}

int ejk_rpa_set_option(const char* name, int value) {
  if (!name) return EJK_RPA_E_NULL;
  if (!std::strcmp(name, "waves")) {
    if (value < 1 || value > 4096) return EJK_RPA_E_ARG;
    g_opt.waves = value;
  } else if (!std::strcmp(name, "min_chunk")) {
    if (value < kTileTokens || value % kTileTokens) return EJK_RPA_E_ARG;
    g_opt.min_chunk = value;
  } else if (!std::strcmp(name, "path")) {
    if (value < 0 || value > 2) return EJK_RPA_E_ARG;
    g_opt.path = value;
  } else if (!std::strcmp(name, "profile")) {
    g_opt.profile = value ? 1 : 0;
  } else if (!std::strcmp(name, "overlap")) {
    g_opt.overlap = value ? 1 : 0;
  } else if (!std::strcmp(name, "prefill_split")) {
    if (value < 0 || value > 2) return EJK_RPA_E_ARG;
    g_opt.prefill_split = value;
  } else if (!std::strcmp(name, "sort_items")) {
    g_opt.sort_items = value ? 1 : 0;
  } else if (!std::strcmp(name, "test_withhold")) {
    if (value < 0 || value > 3) return EJK_RPA_E_ARG;
    g_opt.test_withhold = value;
  } else if (!std::strcmp(name, "fused_merge")) {
    if (value < 0 || value > 2) return EJK_RPA_E_ARG;
    g_opt.fused_merge = value;
  } else if (!std::strcmp(name, "wait_ms")) {
    if (value < 1) return EJK_RPA_E_ARG;
    g_opt.wait_ms = value;
  } else if (!std::strcmp(name, "prefill_rows")) {
    if (value < 0) return EJK_RPA_E_ARG;
    g_opt.prefill_rows = value;
  } else if (!std::strcmp(name, "prefill_share")) {
    if (value < 0 || value > 1000) return EJK_RPA_E_ARG;
    g_opt.prefill_share = value;
  } else if (!std::strcmp(name, "probe_chunk_kb")) {
    if (value < 0 || value > 64 || (value & (value - 1))) return EJK_RPA_E_ARG;  // a power of two, at most 64
    g_opt.probe_chunk_kb = value;
  } else if (!std::strcmp(name, "probe_slots")) {
    if (value < 0 || value > 12) return EJK_RPA_E_ARG;
    g_opt.probe_slots = value;
  } else if (!std::strcmp(name, "probe_ctas")) {
    if (value < 0 || value > 8) return EJK_RPA_E_ARG;
    g_opt.probe_ctas = value;
  } else {
    return EJK_RPA_E_ARG;
  }
  return 0;
}

int ejk_rpa_get_option(const char* name, int* value) {
  if (!name || !value) return EJK_RPA_E_NULL;
  if (!std::strcmp(name, "waves")) *value = g_opt.waves;
  else if (!std::strcmp(name, "min_chunk")) *value = g_opt.min_chunk;
  else if (!std::strcmp(name, "path")) *value = g_opt.path;
  else if (!std::strcmp(name, "profile")) *value = g_opt.profile;
  else if (!std::strcmp(name, "overlap")) *value = g_opt.overlap;
  else if (!std::strcmp(name, "prefill_split")) *value = g_opt.prefill_split;
  else if (!std::strcmp(name, "sort_items")) *value = g_opt.sort_items;
  else if (!std::strcmp(name, "test_withhold")) *value = g_opt.test_withhold;
  else if (!std::strcmp(name, "fused_merge")) *value = g_opt.fused_merge;
  else if (!std::strcmp(name, "wait_ms")) *value = g_opt.wait_ms;
  else if (!std::strcmp(name, "prefill_rows")) *value = g_opt.prefill_rows;
  else if (!std::strcmp(name, "prefill_share")) *value = g_opt.prefill_share;
  else if (!std::strcmp(name, "probe_chunk_kb")) *value = g_opt.probe_chunk_kb;
  else if (!std::strcmp(name, "probe_slots")) *value = g_opt.probe_slots;
  else if (!std::strcmp(name, "probe_ctas")) *value = g_opt.probe_ctas;
  else return EJK_RPA_E_ARG;
  return 0;
}

int ejk_rpa_last_launch_count(void) { return t_last_launches; }

int ejk_rpa_stream_probe(const void* src, size_t bytes, void* sink, void* stream) {
  t_last_launches = 0;
  if (!src || !sink) return EJK_RPA_E_NULL;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(sink) & 7)) return EJK_RPA_E_ALIGN;
  if (bytes < 65536) return EJK_RPA_E_ARG;
  const DeviceInfo* d = device_info();
  if (!d || d->cc_major != 10) return EJK_RPA_E_DEVICE;
  cudaError_t e = launch_stream_probe(src, bytes, static_cast<unsigned*>(sink), d->sm_count, g_opt.wait_ms,
                                      g_opt.probe_chunk_kb, g_opt.probe_slots, g_opt.probe_ctas,
                                      static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  t_last_launches = 1;
  return 0;
}

int ejk_rpa_profile_read_kernels(float* plan_ms, float* prefill_ms, float* splitkv_ms, float* merge_ms) {
  if (!t_prof.recorded) return EJK_RPA_E_ARG;
  cudaError_t e = cudaEventSynchronize(t_prof.ev[4]);
  if (e != cudaSuccess) return static_cast<int>(e);
  float* dst[4] = {plan_ms, prefill_ms, splitkv_ms, merge_ms};
  for (int i = 0; i < 4; ++i) {
    float ms = 0.f;
    e = cudaEventElapsedTime(&ms, t_prof.ev[i], t_prof.ev[i + 1]);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dst[i]) *dst[i] = ms;
  }
  return 0;
}

int ejk_rpa_profile_read(float* plan_ms, float* main_ms, float* merge_ms) {
  float pre = 0.f, skv = 0.f;
  const int rc = ejk_rpa_profile_read_kernels(plan_ms, &pre, &skv, merge_ms);
  if (rc == 0 && main_ms) *main_ms = pre + skv;
  return rc;
}

}  // extern "C"
