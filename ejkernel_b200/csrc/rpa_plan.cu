// Device-side planner: turns (context_lens, query_start_loc, num_seqs), which live in device
// memory and must not be read by the host, into the work list of the split-KV kernel.
//
// The reference walks sequences, 8-row query blocks and 64-page KV blocks in nested
// data-dependent loops (ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:187-201).
// Here the same iteration space is flattened into (sequence, row tile, KV chunk) items of nearly
// equal size so that 148 SMs stay evenly loaded when lengths differ by 64x.
#include "rpa_device.cuh"
#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kPlanThreads = 1024;
constexpr int kLenBuckets = 1024;  // prefill tiles are queued longest first (bucketed by stage count)
constexpr int kSeqCache = 2048;    // sequences whose lengths stay in shared memory between the passes

struct SeqInfo {
  int q_start, q_len, kv_len, rows, tiles;
  bool ok;
  bool prefill;  // many query rows: 128-row tiles for the tcgen05 kernel, no KV split
};

// The three passes of the planner need every sequence's (query start, query end, kv length); the
// first pass reads them from global memory and parks them in shared memory (`cache`, three rows of
// kSeqCache), the later passes take them from there: a global round trip per pass is most of a
// pass's latency.
__device__ __forceinline__ SeqInfo load_seq(const Params& p, int s, unsigned& flags, int (*cache)[kSeqCache], bool fill) {
  SeqInfo si;
  int q0, q1, kv;
  if (!fill && s < kSeqCache) {
    q0 = cache[0][s];
    q1 = cache[1][s];
    kv = cache[2][s];
  } else {
    // no query_start_loc: a pure decode batch, one query row per sequence (page_attention)
    q0 = p.query_start_loc ? p.query_start_loc[s] : s;
    q1 = p.query_start_loc ? p.query_start_loc[s + 1] : s + 1;
    kv = p.context_lens[s];
    if (fill && s < kSeqCache) {
      cache[0][s] = q0;
      cache[1][s] = q1;
      cache[2][s] = kv;
    }
  }
  const int kv_cap = p.pages_per_seq * p.page_size;
  if (kv < 0 || kv > kv_cap) {
    flags |= EJK_RPA_ST_KVLEN;
    kv = kv < 0 ? 0 : kv_cap;
  }
  int ql = q1 - q0;
  si.ok = true;
  if (ql < 0 || q0 < 0 || q1 > p.T) {
    flags |= EJK_RPA_ST_QLEN;
    si.ok = false;
    ql = 0;
  }
  if (ql > kv) flags |= EJK_RPA_ST_QLEN;  // rows at negative positions see no key and produce 0
  si.q_start = q0;
  si.q_len = ql;
  si.kv_len = kv;
  si.rows = ql * p.G;
  si.prefill = p.prefill_min_rows > 0 && si.rows >= p.prefill_min_rows;
  const int rpt = si.prefill ? p.prefill_item_rows : p.rows_per_tile;
  si.tiles = (si.rows + rpt - 1) / rpt;
  if (ql == 0) si.ok = false;  // _xla_impl_fwd.py:189-193: sequences without queries are skipped
  return si;
}

// Key range [lo, hi) visible to at least one row of tile t; lo is rounded down to a stage boundary.
__device__ __forceinline__ void tile_range(const Params& p, const SeqInfo& si, int t, int& lo, int& hi,
                                           int rows_per_tile) {
  const int r_first = t * rows_per_tile;
  int r_last = r_first + rows_per_tile;
  if (r_last > si.rows) r_last = si.rows;
  r_last -= 1;
  const int qt_first = r_first / p.G;
  const int qt_last = r_last / p.G;
  const int base = si.kv_len - si.q_len;  // position of the sequence's first query row
  hi = base + qt_last + 1;
  if (hi < 0) hi = 0;
  lo = 0;
  if (p.window > 0) {
    lo = base + qt_first - p.window + 1;
    if (lo < 0) lo = 0;
  }
  lo = (lo / kTileTokens) * kTileTokens;
  if (hi < lo) hi = lo;
}

__device__ __forceinline__ void chunking(int len, int chunk, int& n, int& csize) {
  n = (len + chunk - 1) / chunk;
  if (n < 1) n = 1;
  csize = (len + n - 1) / n;
  csize = ((csize + kTileTokens - 1) / kTileTokens) * kTileTokens;
  if (csize < kTileTokens) csize = kTileTokens;
}

// Work items go to scattered queue positions: three 16-byte stores per item instead of twelve 4-byte
// ones (with one item per lane every store instruction touches 32 sectors, and that store traffic was most
// of the planner's time at 2048 sequences).
__device__ __forceinline__ void store_unit(Unit* dst, const Unit& u) {
  int4* d = reinterpret_cast<int4*>(dst);
  d[0] = make_int4(u.seq, u.row0, u.kv_begin, u.kv_end);
  d[1] = make_int4(u.slot, u.q_start, u.q_len, u.kv_len);
  d[2] = make_int4(u.merge_idx, u.chunk_idx, u.n_chunks, u.pad);
}
__device__ __forceinline__ void store_merge(MergeItem* dst, const MergeItem& m) {
  static_assert(sizeof(MergeItem) == 32, "two 16-byte words");
  int4* d = reinterpret_cast<int4*>(dst);
  d[0] = make_int4(m.row0, m.slot0, m.n_chunks, m.q_start);
  d[1] = make_int4(m.q_len, m.pad[0], m.pad[1], m.pad[2]);
}

// inclusive block scan of kCnt counters; returns this thread's exclusive prefix and the block total
constexpr int kCnt = 4;
__device__ void block_scan(int (&v)[kCnt], int (&excl)[kCnt], int (&total)[kCnt], int (*s_warp)[kCnt]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc[kCnt];
#pragma unroll
  for (int k = 0; k < kCnt; ++k) {
    int x = v[k];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    inc[k] = x;
    if (lane == 31) s_warp[warp][k] = x;
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int k = 0; k < kCnt; ++k) {
      int x = s_warp[lane][k];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      s_warp[lane][k] = x;
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kCnt; ++k) {
    const int wprev = warp ? s_warp[warp - 1][k] : 0;
    excl[k] = inc[k] - v[k] + wprev;
    total[k] = s_warp[31][k];
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kPlanThreads) rpa_plan_kernel(const Params p) {
  // kernels launched as programmatic dependents may start their prologue now; they pdl_wait() for the plan
  pdl_trigger();
  // The planner itself is launched as a programmatic dependent of whatever precedes it in the stream (the previous
  // call's last kernel in a serving loop), which hides its launch latency; it touches no memory before that kernel has
  // completed.  (The kernels released above wait for this grid's completion, so they are ordered behind it as well.)
  pdl_wait();
  __shared__ int s_warp[32][kCnt];
  __shared__ unsigned long long s_keys;
  __shared__ int s_tiles;
  __shared__ int s_chunk;
  __shared__ int s_bucket[kLenBuckets];  // histogram, then write cursor, of prefill tiles per length bucket
  __shared__ int s_bdec[kLenBuckets];    // the same for the split-KV work items
  __shared__ int s_seq[3][kSeqCache];    // see load_seq
  __shared__ int s_ex[3][kPlanThreads];  // pass 2: per sequence of the round, exclusive offsets of its units / merge items / slots
  const int tid = threadIdx.x;
  unsigned flags = 0;

  int S = p.num_seqs ? p.num_seqs[0] : p.S_max;
  if (S > p.S_max) {
    flags |= EJK_RPA_ST_NUM_SEQS;
    S = p.S_max;
  }
  if (S < 0) S = 0;
  if (tid == 0) {
    s_keys = 0ull;
    s_tiles = 0;
  }
  for (int i = tid; i < kLenBuckets; i += kPlanThreads) {
    s_bucket[i] = 0;
    s_bdec[i] = 0;
  }
  // bucket = stages >> bshift, sized so the longest possible tile lands in the last bucket
  int bshift = 0;
  {
    const long long max_stages = ((long long)p.pages_per_seq * p.page_size + kTileTokens - 1) / kTileTokens;
    while ((max_stages >> bshift) >= kLenBuckets) ++bshift;
  }
  auto bucket_of = [&](int lo, int hi) {
    const int st = (hi - lo + kTileTokens - 1) / kTileTokens;
    const int b = st >> bshift;
    return b < kLenBuckets ? b : kLenBuckets - 1;
  };
  __syncthreads();

  // ---- pass 1: total number of (tile, key) pairs -> chunk size
  unsigned long long keys = 0;
  int n_tiles = 0;
  for (int s = tid; s < S; s += kPlanThreads) {
    unsigned f = 0;
    SeqInfo si = load_seq(p, s, f, s_seq, true);
    if (!si.ok) continue;
    if (si.prefill) {
      for (int t = 0; t < si.tiles; ++t) {
        int lo, hi;
        tile_range(p, si, t, lo, hi, p.prefill_item_rows);
        atomicAdd(&s_bucket[bucket_of(lo, hi)], 1);
      }
      continue;
    }
    for (int t = 0; t < si.tiles; ++t) {
      int lo, hi;
      tile_range(p, si, t, lo, hi, p.rows_per_tile);
      keys += (unsigned long long)(hi - lo);
    }
    n_tiles += si.tiles;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    keys += __shfl_xor_sync(0xffffffffu, keys, o);
    n_tiles += __shfl_xor_sync(0xffffffffu, n_tiles, o);
  }
  if ((tid & 31) == 0 && keys) atomicAdd(&s_keys, keys);
  if ((tid & 31) == 0 && n_tiles) atomicAdd(&s_tiles, n_tiles);
  __syncthreads();
  if (tid == 0) {
    const unsigned long long total = s_keys;
    unsigned long long tgt = (unsigned long long)(p.target_units > 0 ? p.target_units : 1);
    // Few row tiles, each cut into many chunks (long contexts on few kv heads): every tile is split anyway, and
    // items half as long load the CTAs more evenly -- one-of-eight head shard of 64 sequences of 33k-131k tokens
    // 0.451 -> 0.442 ms, one of four 0.864 -> 0.842, one of two 1.635 -> 1.616.  Batches of many tiles with a chunk
    // or two each (256 decode sequences of up to 8k tokens) are faster with fewer, longer items.
    if (p.target_units_max > p.target_units && (unsigned long long)s_tiles * 4ull <= tgt) tgt = (unsigned long long)p.target_units_max;
    unsigned long long c = (total + tgt - 1) / tgt;
    c = ((c + kTileTokens - 1) / kTileTokens) * kTileTokens;
    if (c < (unsigned long long)p.min_chunk) c = p.min_chunk;
    if (c < (unsigned long long)kTileTokens) c = kTileTokens;
    if (c > 0x40000000ull) c = 0x40000000ull;
    s_chunk = (int)c;
    p.header[kHdrChunk] = (int)c;
    p.header[kHdrTotalKeys] = (int)(total > 0x7fffffffull ? 0x7fffffffull : total);
    p.header[kHdrQueue] = 0;
    p.header[kHdrPrefillQueue] = 0;
    // rows of `out` from here on belong to no sequence; the split-KV kernel zero-fills them (the reference's
    // result starts as zeros, _xla_impl_fwd.py:58)
    int tail = p.query_start_loc ? p.query_start_loc[S] : S;
    p.header[kHdrTailStart] = tail < 0 ? 0 : (tail > p.T ? p.T : tail);
  }
  __syncthreads();
  const int chunk = s_chunk;

  // ---- pass 1b: histogram of the split-KV work items by length (the chunk size is known now)
  for (int s = tid; s < S && p.sort_items; s += kPlanThreads) {
    unsigned f = 0;
    SeqInfo si = load_seq(p, s, f, s_seq, false);
    if (!si.ok || si.prefill) continue;
    for (int t = 0; t < si.tiles; ++t) {
      int lo, hi, n, cs;
      tile_range(p, si, t, lo, hi, p.rows_per_tile);
      chunking(hi - lo, chunk, n, cs);
      if (n > 1) atomicAdd(&s_bdec[bucket_of(lo, lo + cs)], n - 1);
      atomicAdd(&s_bdec[bucket_of(lo + (n - 1) * cs, hi)], 1);
    }
  }
  __syncthreads();

  // histograms -> descending exclusive offsets: the longest items get the lowest queue positions, so the
  // persistent CTAs take them first (longest-processing-time order) and the kernels end on short
  // items instead of on whatever the sequence order happens to leave for last
  int n_prefill_total = 0;
  {
    static_assert(kLenBuckets == kPlanThreads, "one bucket per planner thread");
    int v[kCnt] = {s_bucket[kLenBuckets - 1 - tid], s_bdec[kLenBuckets - 1 - tid], 0, 0};
    int excl[kCnt], total[kCnt];
    block_scan(v, excl, total, s_warp);
    s_bucket[kLenBuckets - 1 - tid] = excl[0];
    s_bdec[kLenBuckets - 1 - tid] = excl[1];
    n_prefill_total = total[0];
    __syncthreads();
  }

  // ---- pass 2: per-sequence counts -> offsets -> items.  The counting is one thread per sequence; the items are
  // then written one thread per ITEM (a binary search over the sequences' offsets finds the item's sequence), so
  // that a batch of few long sequences, each cut into dozens of chunks, does not serialise on a few threads
  // (64 sequences of 33k-131k tokens on one kv head: 1184 items, 6 us of a 15 us planner when written per sequence).
  int base[kCnt] = {0, 0, 0, 0};  // units, merge items, partial slots, prefill tiles
  for (int s0 = 0; s0 < S; s0 += kPlanThreads) {
    const int s = s0 + tid;
    int cnt[kCnt] = {0, 0, 0, 0};
    SeqInfo si;
    si.ok = false;
    si.prefill = false;
    if (s < S) {
      si = load_seq(p, s, flags, s_seq, false);
      if (si.ok && si.prefill) {
        cnt[3] = si.tiles;
      } else if (si.ok) {
        for (int t = 0; t < si.tiles; ++t) {
          int lo, hi, n, cs;
          tile_range(p, si, t, lo, hi, p.rows_per_tile);
          chunking(hi - lo, chunk, n, cs);
          cnt[0] += n;
          if (n > 1) {
            cnt[1] += 1;
            cnt[2] += n;
          }
        }
      }
    }
    int excl[kCnt], total[kCnt];
    block_scan(cnt, excl, total, s_warp);
    s_ex[0][tid] = excl[0];
    s_ex[1][tid] = excl[1];
    s_ex[2][tid] = excl[2];
    __syncthreads();
    const bool fits = base[0] + total[0] <= p.max_units && base[1] + total[1] <= p.max_merge &&
                      base[2] + total[2] <= p.max_slots && base[3] + total[3] <= p.max_punits;
    if (!fits) flags |= EJK_RPA_ST_INTERNAL;
    const int n_here = (S - s0 < kPlanThreads) ? S - s0 : kPlanThreads;  // sequences of this round
    for (int j = tid; fits && j < total[0]; j += kPlanThreads) {
      // the sequence whose items include item j of this round: last i with s_ex[0][i] <= j (sequences without
      // items share their successor's offset and are skipped by taking the last)
      int a = 0, b = n_here;
      while (b - a > 1) {
        const int mid = (a + b) >> 1;
        if (s_ex[0][mid] <= j) a = mid;
        else b = mid;
      }
      const int sj = s0 + a;
      unsigned f = 0;
      const SeqInfo sq = load_seq(p, sj, f, s_seq, false);
      int left = j - s_ex[0][a];  // index of the item inside its sequence
      int m = base[1] + s_ex[1][a], sl = base[2] + s_ex[2][a];
      for (int t = 0; t < sq.tiles; ++t) {
        int lo, hi, n, cs;
        tile_range(p, sq, t, lo, hi, p.rows_per_tile);
        chunking(hi - lo, chunk, n, cs);
        if (left >= n) {
          left -= n;
          if (n > 1) {
            ++m;
            sl += n;
          }
          continue;
        }
        const int c = left;
        if (n > 1 && c == 0) {
          MergeItem mi;
          mi.row0 = t * p.rows_per_tile;
          mi.slot0 = sl;
          mi.n_chunks = n;
          mi.q_start = sq.q_start;
          mi.q_len = sq.q_len;
          mi.pad[0] = mi.pad[1] = mi.pad[2] = 0;
          store_merge(&p.merge[m], mi);
        }
        Unit un;
        un.seq = sj;
        un.row0 = t * p.rows_per_tile;
        un.kv_begin = lo + c * cs;
        const int e = lo + (c + 1) * cs;
        un.kv_end = e < hi ? e : hi;
        un.slot = (n > 1) ? sl + c : -1;
        un.q_start = sq.q_start;
        un.q_len = sq.q_len;
        un.kv_len = sq.kv_len;
        un.merge_idx = (n > 1) ? m : -1;
        un.chunk_idx = c;
        un.n_chunks = n;
        un.pad = 0;
        const int at = p.sort_items ? atomicAdd(&s_bdec[bucket_of(un.kv_begin, un.kv_end)], 1) : base[0] + j;
        if (at < p.max_units) store_unit(&p.units[at], un);
        break;
      }
    }
    __syncthreads();  // s_ex is rewritten by the next round
#pragma unroll
    for (int k = 0; k < kCnt; ++k) base[k] += total[k];
  }
  // ---- prefill items into their queue, in an order that does not depend on thread timing: the KV split
  // of the tile kernel cuts the items in queue order, so the order decides where partial sums are
  // combined and therefore the last bit of the result.  One warp walks the sequences 32 at a time;
  // lanes whose items fall into the same length bucket take consecutive positions in lane order.
  if (p.prefill_min_rows > 0 && n_prefill_total > 0 && n_prefill_total <= p.max_punits && base[3] <= p.max_punits) {
    if (tid < 32) {
      const int lane = tid;
      for (int s0 = 0; s0 < S; s0 += 32) {
        const int s = s0 + lane;
        SeqInfo si;
        si.ok = false;
        si.prefill = false;
        si.tiles = 0;
        unsigned f = 0;
        if (s < S) si = load_seq(p, s, f, s_seq, false);
        const int tiles = (si.ok && si.prefill) ? si.tiles : 0;
        int max_t = tiles;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const int other = __shfl_xor_sync(0xffffffffu, max_t, o);
          max_t = other > max_t ? other : max_t;
        }
        for (int t = 0; t < max_t; ++t) {
          const bool have = t < tiles;
          int lo = 0, hi = 0, b = -1 - lane;  // lanes without an item match nobody
          if (have) {
            tile_range(p, si, t, lo, hi, p.prefill_item_rows);
            b = bucket_of(lo, hi);
          }
          const unsigned same = __match_any_sync(0xffffffffu, b);
          if (have) {
            const int leader = __ffs(same) - 1;
            int pos = 0;
            if (lane == leader) {
              pos = s_bucket[b];
              s_bucket[b] = pos + __popc(same);
            }
            pos = __shfl_sync(same, pos, leader) + __popc(same & ((1u << lane) - 1u));
            Unit un;
            un.seq = s;
            un.row0 = t * p.prefill_item_rows;
            un.kv_begin = lo;
            un.kv_end = hi;
            un.slot = -1;
            un.q_start = si.q_start;
            un.q_len = si.q_len;
            un.kv_len = si.kv_len;
            un.merge_idx = -1;
            un.chunk_idx = 0;
            un.n_chunks = 1;
            un.pad = 0;
            store_unit(&p.punits[pos], un);
          }
          __syncwarp();  // the next round's leaders read the cursors this round's leaders moved
        }
      }
    }
    __syncthreads();
  }
  // arrival counters of the fused merge start at zero on every call
  {
    const int n_tickets = (base[1] <= p.max_merge ? base[1] : 0) * p.Hkv;
    for (int i = tid; i < n_tickets; i += kPlanThreads) p.tickets[i] = 0;
  }
  // KV split of prefill items: exclusive prefix of their stage counts in queue order (the tile kernel
  // cuts the concatenated stage sequence of all (item, kv head) pairs into equal CTA quotas), and the
  // arrival counters of the parts
  // (the stage total alone is also what the tile kernel's SM-sharing rule reads, whether or not items are split)
  int prefill_stages = 0;
  if (p.prefill_min_rows > 0) {
    const int n_items = base[3] <= p.max_punits ? base[3] : 0;
    __syncthreads();  // the items scattered above by other threads
    int running = 0;
    for (int i0 = 0; i0 < n_items; i0 += kPlanThreads) {
      const int i = i0 + tid;
      int v[kCnt] = {0, 0, 0, 0};
      if (i < n_items) {
        const int len = p.punits[i].kv_end - p.punits[i].kv_begin;
        v[0] = len > 0 ? (len + kTileTokens - 1) / kTileTokens : 1;
      }
      int excl[kCnt], total[kCnt];
      block_scan(v, excl, total, s_warp);
      if (p.prefill_split && i < n_items) p.pprefix[i] = running + excl[0];
      running += total[0];
    }
    prefill_stages = running;
    if (p.prefill_split) {
      if (tid == 0) p.pprefix[n_items] = running;
      const int nt = p.prefill_item_rows / kPrefillRows;
      const int n_pt = n_items * p.Hkv * nt * 4;
      for (int i = tid; i < n_pt; i += kPlanThreads) p.ptickets[i] = 0;
    }
  }
  if (tid == 0) {
    const bool over = base[0] > p.max_units || base[1] > p.max_merge || base[2] > p.max_slots || base[3] > p.max_punits;
    p.header[kHdrNumUnits] = over ? 0 : base[0];
    p.header[kHdrNumMerge] = over ? 0 : base[1];
    p.header[kHdrNumSlots] = over ? 0 : base[2];
    p.header[kHdrNumPrefill] = over ? 0 : base[3];
    p.header[kHdrPrefillStages] = over ? 0 : prefill_stages;
    if (over) flags |= EJK_RPA_ST_INTERNAL;
  }
  if (flags && p.status) atomicOr(reinterpret_cast<unsigned*>(p.status), flags);
}

}  // namespace

cudaError_t launch_plan(const Params& p, cudaStream_t stream, bool pdl) {
  return launch_kernel(rpa_plan_kernel, dim3(1), dim3(kPlanThreads), 0, stream, pdl, p);
}

}  // namespace ejk
