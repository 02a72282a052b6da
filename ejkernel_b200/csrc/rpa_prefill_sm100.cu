// Prefill tiles of ragged paged attention on tcgen05 + TMEM: two 128-row tiles per CTA (one at
// head_dim 256), each with its own MMA-issuing warps and softmax warps, sharing the KV stages.
//
// Per 64-token KV stage and per tile x (the two einsums of the reference's inner loop,
// _xla_impl_fwd.py:119-124,148 of ejkernel/kernels/_xla/ragged_page_attention):
//     S_x[128 x 64] = Q_x[128 x D] . K^T           D/16 tcgen05.mma, A and B from shared memory
//     O_x[128 x D] += P_x[128 x 64] . V            4 tcgen05.mma, A = P_x from TMEM, B = V MN-major
// What bounds such a tile is not the tensor pipe (measured: ~55 cycles per S MMA, ~77 per P.V MMA when
// issued back to back) but latency: a softmax warp needs ~1100 cycles per stage (one warp per scheduler
// and tile runs at a fraction of an instruction per cycle), every hand-off through an mbarrier costs
// 100+ cycles while the tensor pipe and the TMA unit stream through shared memory, and a thread
// that issues MMAs spends 50-150 cycles on each.  So the kernel is arranged for nobody to wait for
// anybody longer than necessary:
//   * S_x, P_x (two buffers) and O_x live in different TMEM columns.  As soon as the softmax warps
//     hold S_x(j) in registers (one tcgen05.ld) they release the S columns and the tile's S issuer
//     puts S_x(j+1) on the pipe while the exponentials of stage j are computed; P_x(j) goes to
//     buffer j & 1, so it never waits for P_x.V(j-1) either.
//   * S of each tile and the P.V products are issued by different warps (three single-thread issuing
//     roles), so that no role's waits delay another's MMAs.  One thread issues P.V for both tiles:
//     their P arrive in turn anyway, and with 12 warps instead of 13 a thread gets 168 registers
//     instead of 128 (each of the SM's four schedulers has its own 16 K registers and the warps
//     are dealt round to them: a thirteenth warp puts four warps on one scheduler).
//   * the two tiles' softmax warps share the schedulers and the MUFU unit (4 exponentials per cycle
//     and scheduler); they take turns at the exponentials, so that one tile's waits and TMEM
//     traffic overlap the other's MUFU phase instead of both phases running in lockstep.
//   TMEM (512 columns at head_dim 128): S_0 S_1 (64 fp32 columns each), P_0[2] P_1[2] (32 columns
//   of 16-bit pairs each), O_0 O_1 (D each).  At head_dim 256 one tile: S, P[2], O = 384 columns.
// Things measured and left out: a polynomial 2^x on the FMA pipe for part of the exponentials (no gain:
// issue slots are as scarce as MUFU slots with so few warps), two threads per row (the exchange of
// row maxima costs more than the shorter rows save), 80/96/128-token stages with P aliased on S
// (the tile's S -> softmax -> P.V chain then bounds the stage; at 128 tokens also with one thread
// issuing all MMAs in order, K and V in separate slots and the row's 128 logits fetched with a single
// TMEM wait under a register hand-over between warpgroups: level with this kernel, not faster --
// with the tiles half a stage apart one softmax warp per scheduler works at a time, and a warp
// cannot issue while one of its ex2 is dispatched to the MUFU unit).
//
// Warp roles (384 threads with two tiles, one CTA per SM, persistent over the planner's prefill queue):
//   warp 0        TMA producer: one box {64 elems, 8 tokens, D/64, (K_h, V_h)} per 8-token group,
//                 SWIZZLE_128B, 8 boxes per stage, page ids from the block table; publishes every
//                 item in a ring.  No multicast.
//   warp 1        S issuer of tile 0 (lane 0 only; the warp owns the TMEM allocation)
//   warps 2-5     softmax of tile 0, warps 6-9 of tile 1: thread = TMEM lane = tile row; the row's
//                 logits of the stage sit in registers; lazy rescaling of O (only when the maximum
//                 grows by more than 2^8), normalisation, sinks, store.
//   warps 10-11   S issuer of tile 1, P.V issuer of both tiles (one tile: warp 6 issues P.V)
//
// All hand-offs are mbarriers; every wait is bounded in wall time (Params::wait_timeout_ms): on
// expiry the warp raises the CTA's abort flag, every other wait gives up when it sees it, the status
// word gets EJK_RPA_ST_TIMEOUT and the CTA still frees its TMEM before it returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "rpa_tcgen05.cuh"
#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kBM = kPrefillRows;  // 128 rows per tile
constexpr int kRingP = 16;
constexpr float kLog2eP = 1.4426950408889634f;
constexpr float kLazyP = 8.0f;


// One piece of work of a CTA: an item (256 or 128 query rows of one sequence) of one kv head, or, with
// the KV split, the part of it that falls into the CTA's quota of KV stages.  For a part, u.kv_begin /
// u.kv_end are the part's range, u.n_chunks the number of parts of the item, u.chunk_idx this part's
// number and u.merge_idx the (item, head) index.
struct ItemDescP {
  Unit u;
  int32_t h;
  int32_t first_stage;  // index of the (item, head)'s first stage in the global stage sequence
  int32_t quota;        // stages per CTA
  int32_t pad;
};

template <int D>
struct CfgP {
  // tokens per KV stage = N of the S MMA: the largest for which TMEM holds S and two P buffers per tile
  static constexpr int BN = 64;
  static constexpr int NT = (D <= 128) ? 2 : 1;       // 128-row tiles per CTA (TMEM holds one 256-column O)
  static constexpr int SM_WARPS = 4;                  // softmax warps per tile: one thread per row
  // producer, S issuer of tile 0, softmax groups, the other issuers
  // (16 K registers per scheduler: with 12 warps, three per scheduler, a thread gets 168; with 13 only 128)
  static constexpr int THREADS = 64 + 32 * SM_WARPS * NT + 32 * NT;
  static constexpr int STAGE_BYTES = BN * 2 * D * 2;
  static constexpr int NS = (D == 64) ? 8 : (D == 128) ? 4 : 2;
  static constexpr int GROUP_BYTES = 8 * 2 * D * 2;   // one 8-token group: [K|V][D/64][8][64]
  static constexpr int V_OFF = (D / 64) * 1024;
  static constexpr int Q_BYTES = kBM * D * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + NT * Q_BYTES;
  static constexpr int OFF_RING = OFF_KV + NS * STAGE_BYTES;
  static constexpr int OFF_META = OFF_RING + kRingP * (int)sizeof(ItemDescP);
  static constexpr int OFF_BAR = OFF_META + NS * 8;
  // barriers: kv_full[NS] kv_empty[NS], then per tile: s_full s_free p_full[2] pv_done[2] q_full o_free turn
  static constexpr int BAR_PER_TILE = 9;
  static constexpr int N_BAR = 2 * NS + NT * BAR_PER_TILE;
  static constexpr int OFF_TMEM = OFF_BAR + N_BAR * 8;
  // abort flag, the published-items counter, per tile the count of items its softmax warps have skipped
  static constexpr int OFF_ABORT = OFF_TMEM + 8;
  static constexpr int SMEM_BYTES = OFF_ABORT + 8 + 4 * NT + 1024;
  static constexpr uint32_t P_COLS = BN / 2;               // one P buffer (16-bit pairs)
  static constexpr uint32_t TMEM_S = 0;                    // S_x at x*BN
  static constexpr uint32_t TMEM_P = NT * BN;              // P_x[b] at 2*BN + (2x + b)*P_COLS
  static constexpr uint32_t TMEM_O = 512 - NT * D;         // O_x at the top
  static constexpr uint32_t TMEM_COLS = 512;
  static_assert(BN % 16 == 0 && TMEM_P + NT * 2 * P_COLS <= TMEM_O, "TMEM holds 512 columns");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

template <typename T, int D>
__global__ void __launch_bounds__(CfgP<D>::THREADS, 1)
rpa_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap, const Params p) {
  using C = CfgP<D>;
  constexpr int NS = C::NS, NT = C::NT, kBN = C::BN;
  constexpr int DC = D / 64;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  ItemDescP* ring = reinterpret_cast<ItemDescP*>(smem + C::OFF_RING);
  int2* metas = reinterpret_cast<int2*>(smem + C::OFF_META);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_ABORT);
  volatile int* items_pub = reinterpret_cast<volatile int*>(smem + C::OFF_ABORT + 4);  // items in the ring so far
  // skipped[x]: one count per softmax warp of tile x and item without rows for the tile.  A counter, not an
  // mbarrier: the group is not held back by anybody while it skips items, so it can be several items
  // ahead of the role that waits for it, and a phase parity would alias.
  volatile int* skipped = reinterpret_cast<volatile int*>(smem + C::OFF_ABORT + 8);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_TMEM);
  const uint32_t bar0 = sb + C::OFF_BAR;
  auto bar_kv_full = [&](int s) { return bar0 + s * 8; };
  auto bar_kv_empty = [&](int s) { return bar0 + (NS + s) * 8; };
  auto tile_bar = [&](int x, int i) { return bar0 + (2 * NS + x * C::BAR_PER_TILE + i) * 8; };
  auto bar_s_full = [&](int x) { return tile_bar(x, 0); };    // S_x(t) complete (commit)
  auto bar_s_free = [&](int x) { return tile_bar(x, 1); };    // S_x(t) is in the 4 warps' registers
  auto bar_p_full = [&](int x, int b) { return tile_bar(x, 2 + b); };   // P_x(t) stored to buffer t&1 by the softmax warps
  auto bar_pv_done = [&](int x, int b) { return tile_bar(x, 4 + b); };  // P_x.V(t) complete (commit): buffer t&1 is free
  auto bar_q_full = [&](int x) { return tile_bar(x, 6); };
  auto bar_o_free = [&](int x) { return tile_bar(x, 7); };
  auto bar_turn = [&](int x) { return tile_bar(x, 8); };      // tile x has issued the exponentials of a stage

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Hkv = p.Hkv, G = p.G;
  const unsigned long long wait_ns = (unsigned long long)p.wait_timeout_ms * 1000000ull;
  unsigned flags = 0;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar_kv_full(s), 1);
      // released by the MMA-issuing roles, once per tile for S and once for P.V (commit, or a plain arrival
      // when the tile is idle)
      mbar_init(bar_kv_empty(s), 2 * NT);
    }
    for (int x = 0; x < NT; ++x) {
      mbar_init(bar_s_full(x), 1);
      mbar_init(bar_s_free(x), C::SM_WARPS);  // one arrival per softmax warp
      for (int b = 0; b < 2; ++b) {
        mbar_init(bar_p_full(x, b), C::SM_WARPS);
        mbar_init(bar_pv_done(x, b), 1);
      }
      mbar_init(bar_q_full(x), C::SM_WARPS);
      mbar_init(bar_o_free(x), C::SM_WARPS);
      skipped[x] = 0;
      mbar_init(bar_turn(x), C::SM_WARPS);
    }
    *abort_flag = 0;
    *items_pub = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(sb + C::OFF_TMEM), "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Launched as a programmatic dependent of the planner: everything above overlapped its tail.  The
  // split-KV kernel that follows in the stream works on other rows and may start on SMs that this
  // kernel's CTAs have left; it is released once every CTA has passed this point, i.e. after the
  // plan is complete.
  if (p.pdl & 1) pdl_wait();
  pdl_trigger();
  // Mixed batch: this kernel is compute-bound and the split-KV kernel that follows in the stream is bandwidth-bound, and
  // the two only overlap on SMs this kernel has left (a CTA of each does not fit one SM together).  With all SMs this
  // kernel finishes long before the decode rows' KV has streamed; so it keeps only as many CTAs as make it end about
  // when the split-KV kernel does, and the others exit at once and hand their SMs over: the tensor pipes of some SMs
  // and the memory system then work side by side for the whole call (64 decode sequences + four 512-token chunks:
  // 0.466 -> 0.416 ms; with 0.8 of the estimated CTAs the tile kernel becomes the long pole, 0.465; with 1.3, 0.420).
  // Estimated from the plan: T_p = stages * kStageUs / CTAs against T_d = decode bytes / kDecodeBpUs.
  int n_cta = (int)gridDim.x;
  if ((p.pdl & 1) && p.prefill_share > 0 && D <= 128) {
    const float stages = (float)p.header[kHdrPrefillStages] * (float)Hkv;           // (item, head) stages of 64 tokens
    const float dec_bytes = (float)p.header[kHdrTotalKeys] * (float)Hkv * (float)(2 * D * sizeof(T));
    // one stage of two 128-row tiles: 2460 cycles measured on evenly divisible work at head_dim 128, 0.93 of that at 64
    // (a soft cap puts a tanh on every logit: the softmax threads, which bound the stage, take about 1.6 times as long)
    const float kStageUs = (D == 64 ? 1.15f : 1.25f) * (p.cap != 0.f ? 1.6f : 1.f);
    constexpr float kDecodeBpUs = 6.6e6f;  // bytes per microsecond the split-KV kernel streams
    const float t_p = stages * kStageUs / (float)gridDim.x, t_d = dec_bytes / kDecodeBpUs;
    if (t_d > t_p && t_p > 0.f) {
      int n = (int)ceilf((float)gridDim.x * (t_p / t_d) * (float)p.prefill_share * 0.01f);
      const int floor_n = (int)gridDim.x / 8;
      n = n < floor_n ? floor_n : n;
      n_cta = n < (int)gridDim.x ? n : (int)gridDim.x;
    }
  }
  const bool idle_cta = (int)blockIdx.x >= n_cta;
  const int n_work = idle_cta ? 0 : p.header[kHdrNumPrefill] * Hkv;

  if (warp == 0) {
    // =============================== TMA producer ===============================
    constexpr int kGroups = kBN / 8;  // 8-token groups (= TMA boxes) per stage
    int gi = 0;  // stage counter of this CTA
    int k = 0;
    // Two ways to hand out work.  Dynamic: whole (item, head) pairs from the planner's longest-first
    // queue.  KV split (when the workspace has room for the parts): the stages of all (item, head)
    // pairs, in queue order, form one sequence that is cut into equal quotas, one per CTA, so that
    // every SM is busy to the end however few items there are; an item that straddles a quota
    // boundary is finished by several CTAs, whose parts the last one to arrive combines.
    // A part costs a pipeline restart, a 64-128 KB round trip of its unnormalised O through the
    // workspace and the combine (measured: 15-25 stages' worth per CTA), so the split is used only where
    // the dynamic schedule is clearly worse: rounds * average item > 1.15 * (quota + 16 stages), with a
    // quota of at least 8 stages, e.g. 160
    // equal items on 148 CTAs (0.289 -> 0.203 ms), not 128 or 256 of them, nor short items.
    const int n_items = p.header[kHdrNumPrefill];
    const long long W = idle_cta ? 0 : (long long)p.header[kHdrPrefillStages] * Hkv;
    constexpr int kMinQuota = 8;  // a part shorter than this is all overhead
    bool split = p.prefill_split && W > 0 && W < (1ll << 30);
    long long quota_ll = (W + n_cta - 1) / n_cta;
    if (quota_ll < kMinQuota) quota_ll = kMinQuota;
    if (split && p.prefill_split < 2) {  // 2 = always split (measurement aid)
      const long long U = (long long)n_items * Hkv, Cn = n_cta;
      const long long rounds = (U + Cn - 1) / Cn;
      split = rounds * W * 20 >= 23 * U * (quota_ll + 16);  // rounds * W / U >= 1.15 * (quota + 16)
    }
    const int quota = split ? (int)quota_ll : 0;
    long long g = (long long)blockIdx.x * quota;                 // next global stage of this CTA
    const long long g_end = (g + quota < W) ? g + quota : W;
    int it = 0;                                                  // item that contains stage g
    if (split && g < g_end) {
      int lo = 0, hi = n_items;  // Hkv * pprefix[lo] <= g < Hkv * pprefix[hi]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long)Hkv * __ldg(p.pprefix + mid) <= g) lo = mid;
        else hi = mid;
      }
      it = lo;
    }
    int wid = 0;
    if (!split && !idle_cta) {  // a CTA that has handed its SM over must not draw from the queue
      if (lane == 0) wid = atomicAdd(&p.header[kHdrPrefillQueue], 1);
      wid = __shfl_sync(0xffffffffu, wid, 0);
    }
    bool alive = true;
    while (alive) {
      const int s = gi % NS;
      if (split ? (g >= g_end) : (wid >= n_work)) {
        if (!mbar_wait(bar_kv_empty(s), ((gi / NS) & 1) ^ 1, abort_flag, wait_ns)) break;
        if (lane == 0) {
          metas[s] = make_int2(-1, 0);
          ring[k % kRingP].u.seq = -1;  // end of the item sequence, for the softmax groups
          __threadfence_block();
          *items_pub = k + 1;
          mbar_arrive(bar_kv_full(s));
        }
        break;
      }
      int ui, h, first_stage = 0;
      int st_b = 0, st_e = -1;  // the piece's stage range inside the item (st_e < 0: the whole item)
      int n_parts = 1, part_idx = 0;
      if (split) {
        const int p0 = __ldg(p.pprefix + it), p1 = __ldg(p.pprefix + it + 1);
        const int n_i = p1 - p0;                                  // stages of the item (per head)
        const long long rel = g - (long long)Hkv * p0;
        ui = it;
        h = (int)(rel / n_i);
        st_b = (int)(rel - (long long)h * n_i);
        const long long left = g_end - g;
        const int take = (n_i - st_b < left) ? n_i - st_b : (int)left;
        st_e = st_b + take;
        first_stage = (int)((long long)Hkv * p0 + (long long)h * n_i);
        const int c0 = first_stage / quota, c1 = (first_stage + n_i - 1) / quota;
        n_parts = c1 - c0 + 1;
        part_idx = (int)blockIdx.x - c0;
        g += take;
        if (st_e == n_i && h == Hkv - 1) ++it;
        if (st_e == n_i) st_e = -1;  // up to the item's real end (its last stage may be ragged)
      } else {
        ui = wid / Hkv;
        h = wid - ui * Hkv;
      }
      Unit u;
      {
        const int4* src = reinterpret_cast<const int4*>(p.punits + ui);
        const int4 a = __ldg(src), b = __ldg(src + 1);
        u.seq = a.x; u.row0 = a.y; u.kv_begin = a.z; u.kv_end = a.w;
        u.slot = b.x; u.q_start = b.y; u.q_len = b.z; u.kv_len = b.w;
        u.merge_idx = ui * Hkv + h; u.chunk_idx = part_idx; u.n_chunks = n_parts; u.pad = 0;
        if (st_e >= 0) u.kv_end = u.kv_begin + st_e * kBN;
        u.kv_begin += st_b * kBN;
      }
      const int ring_slot = k % kRingP;
      int wid_next = 0;
      if (!split && lane == 0) wid_next = atomicAdd(&p.header[kHdrPrefillQueue], 1);
      const int32_t* tab = p.block_tables + (size_t)u.seq * p.pages_per_seq;
      bool first = true;
      for (int pos = u.kv_begin; first || pos < u.kv_end; pos += kBN) {
        const int st = gi % NS;
        int ngrp = (u.kv_end - pos + 7) >> 3;
        if (ngrp > kGroups) ngrp = kGroups;
        if (ngrp < 0) ngrp = 0;
        // page id of this lane's 8-token group, fetched before the wait so its latency is hidden
        int page = 0, off = 0;
        if (lane < ngrp) {
          const int key = pos + lane * 8;
          int pi;
          if (p.page_shift >= 0) {
            pi = key >> p.page_shift;
            off = key & (p.page_size - 1);
          } else {
            pi = key / p.page_size;
            off = key - pi * p.page_size;
          }
          page = __ldg(tab + pi);
          if ((unsigned)page >= (unsigned)p.num_pages) {
            flags |= EJK_RPA_ST_PAGE_ID;
            page = 0;
          }
        }
        if (!mbar_wait(bar_kv_empty(st), ((gi / NS) & 1) ^ 1, abort_flag, wait_ns)) {
          alive = false;
          break;
        }
        // test hook: the stage's data is never announced (no arrival, no copies), so the waits for it must
        // run out; the item itself is published as usual, so that every role sees a valid descriptor
        const bool withhold = (p.test_withhold & 2) && first && (split ? (blockIdx.x == 0 && k == 0) : (wid == 0));
        if (withhold) ngrp = 0;
        if (lane == 0) {
          if (first) {
            // every role is within NS + 2 items of this warp (the MMA warps through the stage ring, each
            // softmax group through q_full or its skip count): slot k - kRingP is free
            ItemDescP d;
            d.u = u;
            d.h = h;
            d.first_stage = first_stage;
            d.quota = quota;
            d.pad = 0;
            ring[ring_slot] = d;
            __threadfence_block();
            *items_pub = k + 1;
          }
          // meta.x = ring slot | 0x100 on the first stage of an item | 0x200 when the item has rows for tile 1
          const bool two = NT == 2 && u.q_len * G > u.row0 + kBM;
          metas[st] = make_int2(ring_slot | (first ? 0x100 : 0) | (two ? 0x200 : 0), pos);
          const uint32_t bytes = (uint32_t)ngrp * C::GROUP_BYTES;
          if (withhold) {
          } else if (bytes > 0) {
            mbar_arrive_expect_tx(bar_kv_full(st), bytes);
          } else {
            mbar_arrive(bar_kv_full(st));
          }
        }
        __syncwarp();
        if (lane < ngrp) {
          tma_load_5d(sb + C::OFF_KV + st * C::STAGE_BYTES + lane * C::GROUP_BYTES, &tmap, bar_kv_full(st), 0, off, 0,
                      2 * h, page);
        }
        first = false;
        ++gi;
      }
      ++k;
      if (!split) wid = __shfl_sync(0xffffffffu, wid_next, 0);
    }
    // wait (bounded) until every stage this warp filled has been released, i.e. all its bulk
    // copies have landed and been consumed
    for (int i = 0; i < NS && gi > 0; ++i) {
      const int g2 = gi + i;
      if (g2 < NS) continue;  // never used
      if (!mbar_wait(bar_kv_empty(g2 % NS), ((g2 / NS) & 1) ^ 1, abort_flag, wait_ns)) break;
    }
    if (*abort_flag) {
      // giving up: nobody releases stages any more, so wait (bounded, 2 ms per stage) for the copies
      // themselves -- the "full" phase of each of the last NS announced stages
      for (int i = 1; i <= NS && i <= gi; ++i) {
        const int f = gi - i;
        mbar_wait_quiet(bar_kv_full(f % NS), (uint32_t)((f / NS) & 1), 2000000ull);
      }
    }
  } else if (warp == 1 || warp >= 2 + C::SM_WARPS * NT) {
    // =============================== MMA issuers ===============================
    // Single-thread roles: S of each tile and P.V (of both tiles) are issued by different warps.  An issuing
    // thread spends most of a stage on latency (an mbarrier poll or a shared-memory read costs it
    // 100+ cycles while the tensor pipe and the TMA unit stream through shared memory, a
    // tcgen05.mma 50-150), so one thread issuing S and P.V for a tile, or worse for both tiles,
    // becomes the bottleneck of the whole CTA.  No ordering between the roles is needed beyond the
    // barriers: S_x(t+1) only needs the S columns back (s_free), P_x.V(t) only P_x(t) (p_full).
    if (lane == 0) {
      // roles in the order S_0 .. S_{NT-1}, PV; S_0 is warp 1, the others follow the softmax warps
      const int role = (warp == 1) ? 0 : warp - (2 + C::SM_WARPS * NT) + 1;
      const bool is_s = role < NT;
      const int x = is_s ? role : 0;
      constexpr uint32_t idesc_s = instr_desc<T>(kBN, false);
      constexpr uint32_t idesc_pv = instr_desc<T>(D, true);
      // hi word of a descriptor: stride byte offset >> 4, version 1 (bit 46), SWIZZLE_128B (bits 61-63)
      constexpr uint64_t kHiAtom1024 = ((uint64_t)((1024u >> 4) | (1u << 14) | (2u << 29))) << 32;
      constexpr uint64_t kHiGroup = ((uint64_t)(((uint32_t)C::GROUP_BYTES >> 4) | (1u << 14) | (2u << 29))) << 32;
      const uint64_t q_desc = kHiAtom1024 | (uint64_t)(((sb + C::OFF_Q + x * C::Q_BYTES) >> 4) | (1u << 16));
      const uint64_t k_desc0 = kHiGroup | (uint64_t)(((sb + C::OFF_KV) >> 4) | (1u << 16));
      // V is MN-major: leading byte offset = distance between 64-element chunks of D (1024 B)
      const uint64_t v_desc0 = kHiGroup | (uint64_t)(((sb + C::OFF_KV + C::V_OFF) >> 4) | ((1024u >> 4) << 16));
      const uint32_t tm_s = tmem_base + C::TMEM_S + x * kBN;

      int gi = 0;     // KV stage counter (every role sees the same stage sequence)
      int t = 0;      // stages this tile took part in (barrier parities)
      int items = 0;  // items this tile took part in
      int skips = 0;  // items this tile had no rows for
      int tx[NT], itemsx[NT];  // the same two counters per tile, for the P.V role
#pragma unroll
      for (int y = 0; y < NT; ++y) tx[y] = itemsx[y] = 0;
      while (!is_s) {
        // ---- P.V of all tiles, tile 0 first (the order in which the tiles take their turns at the
        // exponentials, so P_0(t) is ready before P_1(t), and P_0(t+1) only after that) ----
        const int st = gi % NS;
        if (!mbar_wait_thread(bar_kv_full(st), (gi / NS) & 1, abort_flag, wait_ns)) break;
        const int mx = metas[st].x;
        if (mx < 0) break;
        const bool first = (mx & 0x100) != 0;
        bool gave_up = false;
#pragma unroll
        for (int y = 0; y < NT; ++y) {
          if (gave_up) continue;
          if (y > 0 && !(mx & 0x200)) {  // no rows for this tile: only its share of the stage's release
            mbar_arrive(bar_kv_empty(st));
            continue;
          }
          if (first) ++itemsx[y];
          const int ty = tx[y];
          // O_y (+)= P_y . V: P_y(t) must be in its TMEM buffer; the first P.V of an item overwrites
          // O_y, which the previous item's epilogue must have read
          if (!mbar_wait_thread(bar_p_full(y, ty & 1), (ty >> 1) & 1, abort_flag, wait_ns) ||
              (first && itemsx[y] > 1 && !mbar_wait_thread(bar_o_free(y), itemsx[y] & 1, abort_flag, wait_ns))) {
            gave_up = true;
            continue;
          }
          tc_fence_after();
          const uint32_t tm_p = tmem_base + C::TMEM_P + y * 2 * C::P_COLS;
          const uint32_t tm_o = tmem_base + C::TMEM_O + y * D;
          const uint64_t vd = v_desc0 + (uint64_t)((st * C::STAGE_BYTES) >> 4);
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk) {
            // V: 16 tokens = two 8-token groups per MMA; P: 16 tokens = 8 columns of 16-bit pairs
            tc_mma_ts(tm_o, tm_p + (ty & 1) * C::P_COLS + kk * 8, vd + (uint64_t)((kk * 2 * C::GROUP_BYTES) >> 4), idesc_pv,
                      !(first && kk == 0));
          }
          tc_commit(bar_pv_done(y, ty & 1));
          tc_commit(bar_kv_empty(st));  // this tile's P.V MMAs that read the stage have been issued
          ++tx[y];
        }
        if (gave_up) break;
        ++gi;
      }
      while (is_s) {
        const int st = gi % NS;
        if (!mbar_wait_thread(bar_kv_full(st), (gi / NS) & 1, abort_flag, wait_ns)) break;
        const int mx = metas[st].x;
        if (mx < 0) break;
        const bool first = (mx & 0x100) != 0;
        const bool act = (x == 0) || (mx & 0x200) != 0;
        if (!act) {  // the item has no rows for this tile: only this role's share of the stage's release
          if (first) {
            // ... once the tile's softmax group has seen the item, so that it never falls behind
            ++skips;
            bool seen = skipped[x] >= C::SM_WARPS * skips;
            if (!seen) {
              const unsigned long long t0 = global_timer_ns();
              while (!(seen = skipped[x] >= C::SM_WARPS * skips)) {
                if (*abort_flag) break;
                if (global_timer_ns() - t0 > wait_ns) {
                  *abort_flag = 1;
                  break;
                }
                __nanosleep(64);
              }
            }
            if (!seen) break;
          }
          mbar_arrive(bar_kv_empty(st));
          ++gi;
          continue;
        }
        if (first) ++items;
        {
          // the new query tile must be in shared memory, and S_x of the previous stage in the
          // softmax warps' registers
          if (first && !mbar_wait_thread(bar_q_full(x), (items - 1) & 1, abort_flag, wait_ns)) break;
          if (t > 0 && !mbar_wait_thread(bar_s_free(x), (t - 1) & 1, abort_flag, wait_ns)) break;
          tc_fence_after();
          const uint64_t kd = k_desc0 + (uint64_t)((st * C::STAGE_BYTES) >> 4);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            // K: 8-token atoms one group apart (SBO), the 64-element chunks of D 1024 bytes apart
            const uint32_t koff = (uint32_t)(((kk >> 2) * 1024 + (kk & 3) * 32) >> 4);
            const uint32_t qoff = (uint32_t)(((kk >> 2) * (kBM * 128) + (kk & 3) * 32) >> 4);
            tc_mma(tm_s, q_desc + qoff, kd + koff, idesc_s, kk > 0);
          }
          tc_commit(bar_s_full(x));
        }
        tc_commit(bar_kv_empty(st));  // this role's MMAs that read the stage have been issued
        ++t;
        ++gi;
      }
    }
    __syncwarp();
  } else {
    // =============================== softmax warps ===============================
    // One thread per tile row: warp (x, quarter) owns rows quarter*32.. of tile x (the TMEM lanes a
    // warp may touch are fixed by warp % 4), so row maxima and sums need no shuffles.
    constexpr int HB = kBN;
    const int sw = warp - 2;
    const int x = sw / C::SM_WARPS;                       // which tile of the CTA
    const int row = (warp & 3) * 32 + lane;               // TMEM lane == row within the tile
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int grp_tid = (sw % C::SM_WARPS) * 32 + lane;   // index within the tile's softmax group
    const uint32_t tm_s = tmem_base + lane_addr + C::TMEM_S + x * kBN;
    const uint32_t tm_p0 = tmem_base + lane_addr + C::TMEM_P + x * 2 * C::P_COLS;
    const uint32_t tm_o = tmem_base + lane_addr + C::TMEM_O + x * D;
    int gi = 0;   // KV stage counter (all roles see the same stage sequence)
    int ti = 0;   // stages this tile took part in
    int k = 0;    // item counter (all roles see the same item sequence)
    int pc = 0;   // stages in which both tiles took part (the tiles take turns at the exponentials)
    bool alive = true;
    // The query row of an item (K-major, 128B swizzle) goes from global to shared memory with cp.async,
    // no registers in between, so that the row of the NEXT item can be fetched under the last stage of
    // the current one: the tile's query buffer is free as soon as the item's last S has completed, and
    // with the row in place the S issuer starts the next item while this thread is still in the epilogue.
    const uint32_t q_row_smem = sb + C::OFF_Q + x * C::Q_BYTES + (uint32_t)row * 128;
    auto q_issue = [&](const Unit& uu, int hh) {
      const int R = uu.row0 + x * kBM + row;
      const bool ok = R < uu.q_len * G;
      const int qt = R / G, g = R - qt * G;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.q);
      if (ok) src += ((size_t)(uu.q_start + qt) * p.Hq + hh * G + g) * D * sizeof(T);
#pragma unroll
      for (int c = 0; c < D / 8; ++c)
        cp_async16(q_row_smem + (uint32_t)(c >> 3) * (kBM * 128) + (uint32_t)(((c & 7) ^ (row & 7)) << 4),
                   ok ? src + c * 16 : src, ok ? 16 : 0);  // rows past the item's end are zero-filled
      cp_async_commit();
    };
    auto q_finish = [&]() {
      cp_async_wait<0>();
      fence_async_smem();  // the MMA reads the tile through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_q_full(x));
    };
    bool q_ready = false;    // this item's query row was fetched during the previous item
    // The group follows the item sequence through the producer's item ring (a counter says how many
    // items have been published; an mbarrier parity could alias, because a group whose tile is idle
    // skips whole items) and counts stages itself, so that per stage it waits only for S.
    while (alive) {
      {
        bool have = *items_pub > k;
        if (!have) {
          const unsigned long long t0 = global_timer_ns();
          while (true) {
            __nanosleep(64);
            if (*items_pub > k) {
              have = true;
              break;
            }
            if (*abort_flag || global_timer_ns() - t0 > wait_ns) break;
          }
        }
        have = __all_sync(0xffffffffu, have);
        if (!have) {
          *abort_flag = 1;
          break;
        }
        __threadfence_block();  // the ring entry was written before the counter moved; read it after
      }
      const Unit u = ring[k % kRingP].u;
      const int h = ring[k % kRingP].h;
      const int first_stage = ring[k % kRingP].first_stage, quota = ring[k % kRingP].quota;
      ++k;
      if (u.seq < 0) break;
      int n_stages = (u.kv_end - u.kv_begin + kBN - 1) / kBN;
      if (n_stages < 1) n_stages = 1;
      const bool two = NT == 2 && u.q_len * G > u.row0 + kBM;  // the item has rows for both tiles
      const bool active = (x == 0) || two;
      if (!active) {  // the item has no rows for this tile
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();  // the ring entry has been read
          atomicAdd(const_cast<int*>(&skipped[x]), 1);
        }
        gi += n_stages;
        continue;
      }
      // ---- new item: row bookkeeping and the query row (K-major, 128B swizzle) ----
      const int rows_total = u.q_len * G;
      const int R = u.row0 + x * kBM + row;
      const bool row_ok = R < rows_total;
      const int qt = R / G, g = R - qt * G;
      const int out_row_q = u.q_start + qt;
      const int out_head = h * G + g;
      const int pos_row = row_ok ? (u.kv_len - u.q_len + qt) : -1;
      const int lo_row = (p.window > 0) ? pos_row - p.window : -1;
      float m_run = -INFINITY, l_run = 0.f;
      if (!q_ready) {
        // all S MMAs of this tile's previous item completed before its last s_full fired, which
        // this thread waited for, so the query tile may be overwritten
        q_issue(u, h);
        q_finish();
      }
      q_ready = false;
      for (int js = 0; js < n_stages; ++js, ++gi, ++ti) {
        const int st = gi % NS;
        const int pos = u.kv_begin + js * kBN;  // first key of the stage
        const bool first = (js == 0);
        if (!mbar_wait(bar_s_full(x), ti & 1, abort_flag, wait_ns)) { alive = false; break; }
        tc_fence_after();

        // ---- the row's logits of the stage into registers; then the S columns are free for the
        // tile's next S MMA, which runs while this stage's exponentials are computed
        uint32_t sr[HB];
#pragma unroll
        for (int c = 0; c + 32 <= HB; c += 32) tc_ld32(tm_s + c, *reinterpret_cast<uint32_t(*)[32]>(&sr[c]));
        static_assert(HB % 32 == 0, "S is read 32 columns at a time");
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s_free(x));

        // ---- logits in the log2 domain, soft cap, masks (_xla_impl_fwd.py:125-138).  The common case
        // (no cap, columns entirely visible to this row) keeps the raw dot products and folds the scale
        // into the exponent's FMA; everything else materialises the transformed, masked logits first.
        const bool full_vis = (pos + HB - 1 <= pos_row) && (pos > lo_row);
        // Without a soft cap the raw dot products stay in the registers and the scale is folded into the
        // exponent's FMA; keys the row must not see are replaced by the infinity that scales to -inf
        // (stages on the causal diagonal, window edges, the tail of the last page: common in the first
        // chunk of a prompt, where every stage is such a stage for some rows).
        const bool raw = p.cap == 0.f && p.scale_log2 != 0.f;
        float e_scale = p.scale_log2;  // p = exp2(v * e_scale - m)
        float mx;
        if (raw) {
          if (!full_vis) {
            const uint32_t gone = __float_as_uint(p.scale_log2 > 0.f ? -INFINITY : INFINITY);
            const int hi_i = pos_row - pos;  // last visible column of the stage
            const int lo_i = lo_row - pos;   // columns up to here are left of the window
#pragma unroll
            for (int i = 0; i < HB; ++i)
              if (i > hi_i || i <= lo_i) sr[i] = gone;
          }
          // max of scale*v is scale*max(v) or scale*min(v) depending on the sign of the scale
          float ext[4];
#pragma unroll
          for (int a = 0; a < 4; ++a) ext[a] = __uint_as_float(sr[a]);
          if (p.scale_log2 >= 0.f) {
#pragma unroll
            for (int i = 0; i < HB; i += 8)
#pragma unroll
              for (int a = 0; a < 4; ++a)
                ext[a] = fmax3(ext[a], __uint_as_float(sr[i + 2 * a]), __uint_as_float(sr[i + 2 * a + 1]));
            mx = fmaxf(fmaxf(ext[0], ext[1]), fmaxf(ext[2], ext[3])) * p.scale_log2;
          } else {
#pragma unroll
            for (int i = 0; i < HB; i += 8)
#pragma unroll
              for (int a = 0; a < 4; ++a)
                ext[a] = fmin3(ext[a], __uint_as_float(sr[i + 2 * a]), __uint_as_float(sr[i + 2 * a + 1]));
            mx = fminf(fminf(ext[0], ext[1]), fminf(ext[2], ext[3])) * p.scale_log2;
          }
        } else {
          mx = -INFINITY;
          e_scale = 1.f;
#pragma unroll
          for (int i = 0; i < HB; ++i) {
            float xv = __uint_as_float(sr[i]);
            xv = (p.cap != 0.f) ? p.cap_log2 * soft_cap_tanh(xv * p.inv_cap_scale) : xv * p.scale_log2;
            const int key = pos + i;
            if (!full_vis && (key > pos_row || key <= lo_row)) xv = -INFINITY;
            sr[i] = __float_as_uint(xv);
            mx = fmaxf(mx, xv);
          }
        }
        // P_x has two buffers: this stage's goes where the stage before the previous one's was, whose
        // P.V must have read it (it has, normally long ago)
        if (ti >= 2) {
          if (!mbar_wait(bar_pv_done(x, ti & 1), ((ti - 2) >> 1) & 1, abort_flag, wait_ns)) { alive = false; break; }
        }
        const uint32_t tm_p = tm_p0 + (ti & 1) * C::P_COLS;
        const bool grow = (mx > m_run + kLazyP) || (m_run == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          float alpha = 1.f;
          if (grow) {
            alpha = fast_exp2(m_run - mx);  // 0 on the first finite maximum
            m_run = mx;
            l_run *= alpha;
          }
          if (!first) {
            // O holds the sum over the earlier stages of this item: rescale the row, once the tile's
            // previous P.V has completed (O is only touched between P.Vs)
            if (!mbar_wait(bar_pv_done(x, (ti - 1) & 1), ((ti - 1) >> 1) & 1, abort_flag, wait_ns)) { alive = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 16) {
              uint32_t o[16];
              tc_ld16(tm_o + c0, o);
              tc_wait_ld();
#pragma unroll
              for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
              tc_st16(tm_o + c0, o);
            }
          }
        }
        // The MUFU unit gives 4 exponentials per cycle and scheduler, and both tiles' warps sit on the
        // same schedulers: when both tiles are at work they take turns at the exponentials (tile 0
        // first), so that one tile's waits and TMEM traffic overlap the other's MUFU phase instead of
        // both phases running in lockstep at half speed.
        if (two) {
          const bool my_turn_ok = (x == 0) ? (pc == 0 || mbar_wait(bar_turn(1), (pc - 1) & 1, abort_flag, wait_ns))
                                           : mbar_wait(bar_turn(0), pc & 1, abort_flag, wait_ns);
          if (!my_turn_ok) { alive = false; break; }
        }
        const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
        // probabilities, packed as 16-bit pairs, into the tile's P buffer of this stage
        float lsum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < HB; c += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c + 2 * j]), e_scale, -m_use));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c + 2 * j + 1]), e_scale, -m_use));
            lsum4[j & 3] += p0 + p1;
            pk[j] = Mma<T>::pack(p0, p1);
          }
          tc_st16(tm_p + (c >> 1), pk);
        }
        l_run += (lsum4[0] + lsum4[1]) + (lsum4[2] + lsum4[3]);
        if (two) {
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_turn(x));
          ++pc;
        }
        const bool tail = pos + kBN > u.kv_end;
        if (tail) {
          // Tail stage: V rows of keys >= kv_end were either never fetched (stale shared memory) or lie
          // past the sequence's length inside its last page (unowned, possibly NaN).  Their
          // probabilities are exactly 0, but 0 * NaN would poison O, so every group clears the rows
          // before its own tile's P.V can be issued (the two groups write the same zeros; zero rows are
          // invariant under the swizzle).
          int nvalid = u.kv_end - pos;
          if (nvalid < 0) nvalid = 0;
          uint8_t* vbase = smem + C::OFF_KV + st * C::STAGE_BYTES + C::V_OFF;
          const int n16 = (kBN - nvalid) * DC * 8;
          for (int idx = grp_tid; idx < n16; idx += 32 * C::SM_WARPS) {
            const int t = nvalid + idx / (DC * 8);
            const int rem = idx % (DC * 8);
            *reinterpret_cast<uint4*>(vbase + (t >> 3) * C::GROUP_BYTES + (rem >> 3) * 1024 + (t & 7) * 128 + (rem & 7) * 16) =
                make_uint4(0u, 0u, 0u, 0u);
          }
          fence_async_smem();  // the zeroed V rows are read by the async proxy
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full(x, ti & 1));

        if (pos + kBN >= u.kv_end) {
          // ---- last stage of the piece.  All S of the item completed long ago, so the tile's query
          // buffer is free: fetch the next item's query row (if the producer has published that item
          // already; it normally has, it runs stages ahead) under the wait for the last P.V ...
          bool q_pending = *items_pub > k;
          q_pending = __all_sync(0xffffffffu, q_pending);
          if (q_pending) {
            __threadfence_block();
            const Unit un = ring[k % kRingP].u;
            q_pending = un.seq >= 0 && (x == 0 || un.q_len * G > un.row0 + kBM);
            if (q_pending) q_issue(un, ring[k % kRingP].h);
          }
          // ---- ... wait for the P.V, then normalise and store, or (a part of a split item) publish the
          // unnormalised part and, if it is the last to arrive, combine ----
          if (!mbar_wait(bar_pv_done(x, ti & 1), (ti >> 1) & 1, abort_flag, wait_ns)) { alive = false; break; }
          if (q_pending) {  // the next item's first S runs while this one's epilogue does
            q_finish();
            q_ready = true;
          }
          tc_fence_after();
          if (u.n_chunks > 1) {
            // Slot of the part CTA c holds of this (item, head): a CTA has at most two parts, the item
            // its quota begins in (slot 2c) and the item its quota ends in (slot 2c + 1).
            auto slot_of = [&](int c) { return ((long long)first_stage <= (long long)c * quota) ? 2 * c : 2 * c + 1; };
            const size_t mine = ((size_t)slot_of((int)blockIdx.x) * NT + x) * kBM + row;
            if (row_ok) p.ppart_ml[mine] = make_float2(m_run, l_run);
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
              uint32_t o[32];
              tc_ld32(tm_o + c0, o);
              tc_wait_ld();
              if (row_ok) {
                float4* dst = reinterpret_cast<float4*>(p.ppart_o + mine * D + c0);
#pragma unroll
                for (int c = 0; c < 32; c += 4)
                  dst[c >> 2] = make_float4(__uint_as_float(o[c]), __uint_as_float(o[c + 1]), __uint_as_float(o[c + 2]),
                                            __uint_as_float(o[c + 3]));
              }
            }
            tc_fence_before();
            __threadfence();
            __syncwarp();
            int old = 0;
            if (lane == 0) {
              mbar_arrive(bar_o_free(x));
              // one counter per 32-row quarter of the tile: the warps of a group never wait for each other
              old = atomicAdd(&p.ptickets[((size_t)u.merge_idx * NT + x) * 4 + (warp & 3)], 1);
            }
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == u.n_chunks - 1 && row_ok) {
              // last part to arrive: combine the parts of this row, in part order (so the result does not
              // depend on which part arrived last)
              __threadfence();
              const int c_first = first_stage / quota;
              float m_tot = -INFINITY;
              for (int pi = 0; pi < u.n_chunks; ++pi)
                m_tot = fmaxf(m_tot, __ldcg(&p.ppart_ml[((size_t)slot_of(c_first + pi) * NT + x) * kBM + row]).x);
              const float mu = (m_tot == -INFINITY) ? 0.f : m_tot;
              float l_tot = 0.f;
              for (int pi = 0; pi < u.n_chunks; ++pi) {
                const float2 ml = __ldcg(&p.ppart_ml[((size_t)slot_of(c_first + pi) * NT + x) * kBM + row]);
                l_tot += ml.y * fast_exp2(ml.x - mu);
              }
              float scl = 1.f, l_fin = l_tot;
              if (p.num_sinks > 0) {
                const int srow = (p.sink_rows == p.Hq) ? out_head : (p.sink_rows == Hkv ? h : 0);
                const float* sk = p.sinks + (size_t)srow * p.num_sinks;
                float sm = -INFINITY;
                for (int i = 0; i < p.num_sinks; ++i) sm = fmaxf(sm, sk[i] * kLog2eP);
                const float m_fin = fmaxf(m_tot, sm);
                const float mf = (m_fin == -INFINITY) ? 0.f : m_fin;
                scl = fast_exp2(m_tot - mf);
                l_fin = l_tot * scl;
                for (int i = 0; i < p.num_sinks; ++i) l_fin += fast_exp2(sk[i] * kLog2eP - mf);
              }
              scl = (l_fin > 0.f) ? scl * p.out_scale / l_fin : 0.f;  // out_scale: v_scale of the v3 operator, else 1
              T* orow = reinterpret_cast<T*>(p.out) + ((size_t)out_row_q * p.Hq + out_head) * D;
#pragma unroll 1
              for (int c0 = 0; c0 < D; c0 += 32) {
                float acc[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) acc[c] = 0.f;
                for (int pi = 0; pi < u.n_chunks; ++pi) {
                  const size_t at = ((size_t)slot_of(c_first + pi) * NT + x) * kBM + row;
                  const float f = fast_exp2(__ldcg(&p.ppart_ml[at]).x - mu);
                  const float4* src = reinterpret_cast<const float4*>(p.ppart_o + at * D + c0);
#pragma unroll
                  for (int c = 0; c < 32; c += 4) {
                    const float4 v = __ldcg(src + (c >> 2));
                    acc[c] += v.x * f;
                    acc[c + 1] += v.y * f;
                    acc[c + 2] += v.z * f;
                    acc[c + 3] += v.w * f;
                  }
                }
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                  uint4 v;
                  v.x = Mma<T>::pack(acc[c] * scl, acc[c + 1] * scl);
                  v.y = Mma<T>::pack(acc[c + 2] * scl, acc[c + 3] * scl);
                  v.z = Mma<T>::pack(acc[c + 4] * scl, acc[c + 5] * scl);
                  v.w = Mma<T>::pack(acc[c + 6] * scl, acc[c + 7] * scl);
                  *reinterpret_cast<uint4*>(orow + c0 + c) = v;
                }
              }
            }
            continue;  // next stage = first stage of the next piece
          }
          const float l_row = l_run;
          float scl = 1.f, l_fin = l_row;
          if (p.num_sinks > 0 && row_ok) {
            // attention sinks join the denominator only (_xla_impl_fwd.py:161-172)
            const int srow = (p.sink_rows == p.Hq) ? out_head : (p.sink_rows == Hkv ? h : 0);
            const float* sk = p.sinks + (size_t)srow * p.num_sinks;
            float sm = -INFINITY;
            for (int i = 0; i < p.num_sinks; ++i) sm = fmaxf(sm, sk[i] * kLog2eP);
            const float m_fin = fmaxf(m_run, sm);
            const float mf = (m_fin == -INFINITY) ? 0.f : m_fin;
            scl = fast_exp2(m_run - mf);
            l_fin = l_row * scl;
            for (int i = 0; i < p.num_sinks; ++i) l_fin += fast_exp2(sk[i] * kLog2eP - mf);
          }
          scl = (l_fin > 0.f) ? scl * p.out_scale / l_fin : 0.f;  // out_scale: v_scale of the v3 operator, else 1
          T* orow = reinterpret_cast<T*>(p.out) + ((size_t)out_row_q * p.Hq + out_head) * D;
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            tc_ld32(tm_o + c0, o);
            tc_wait_ld();
            if (row_ok) {
#pragma unroll
              for (int c = 0; c < 32; c += 8) {
                uint4 v;
                v.x = Mma<T>::pack(__uint_as_float(o[c]) * scl, __uint_as_float(o[c + 1]) * scl);
                v.y = Mma<T>::pack(__uint_as_float(o[c + 2]) * scl, __uint_as_float(o[c + 3]) * scl);
                v.z = Mma<T>::pack(__uint_as_float(o[c + 4]) * scl, __uint_as_float(o[c + 5]) * scl);
                v.w = Mma<T>::pack(__uint_as_float(o[c + 6]) * scl, __uint_as_float(o[c + 7]) * scl);
                *reinterpret_cast<uint4*>(orow + c0 + c) = v;
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_o_free(x));
        }
      }
    }
  }
  cp_async_wait<0>();  // a query row fetched ahead when a wait ran out
  if (*abort_flag) flags |= EJK_RPA_ST_TIMEOUT;
  // every role has left its loop (all waits are bounded), so the TMEM can go back
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
  if (flags && p.status) atomicOr(reinterpret_cast<unsigned*>(p.status), flags);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn_p() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}

template <typename T, int D>
cudaError_t launch_one(const Params& p, const CUtensorMap& map, int n_sm, cudaStream_t stream, bool pdl) {
  using C = CfgP<D>;
  auto kern = rpa_prefill_tc_kernel<T, D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  return launch_kernel(kern, dim3(n_sm), dim3(C::THREADS), C::SMEM_BYTES, stream, pdl, map, p);
}

cudaError_t dispatch(const Params& p, int dtype, const CUtensorMap& map, int n_sm, cudaStream_t stream, bool pdl) {
  if (dtype == EJK_RPA_BF16) {
    if (p.D == 64) return launch_one<__nv_bfloat16, 64>(p, map, n_sm, stream, pdl);
    if (p.D == 128) return launch_one<__nv_bfloat16, 128>(p, map, n_sm, stream, pdl);
    if (p.D == 256) return launch_one<__nv_bfloat16, 256>(p, map, n_sm, stream, pdl);
  } else {
    if (p.D == 64) return launch_one<__half, 64>(p, map, n_sm, stream, pdl);
    if (p.D == 128) return launch_one<__half, 128>(p, map, n_sm, stream, pdl);
    if (p.D == 256) return launch_one<__half, 256>(p, map, n_sm, stream, pdl);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

int prefill_rows_per_item(int head_dim) { return head_dim <= 128 ? 2 * kPrefillRows : kPrefillRows; }

bool prefill_path_supported(const Params& p) {
  const int ps = p.page_size;
  if (ps < 8 || ps % 8 != 0) return false;  // one TMA box per 8-token group: a group must not straddle a page
  return encode_fn_p() != nullptr;
}

cudaError_t launch_prefill(const Params& p, int dtype, int n_sm, cudaStream_t stream, bool pdl) {
  EncodeFn enc = encode_fn_p();
  if (!enc) return cudaErrorNotSupported;
  const uint64_t esz = 2;
  const uint64_t D = p.D, Dkv = p.Dkv, C2 = (uint64_t)p.C2;
  cuuint64_t dims[5] = {64, (cuuint64_t)p.page_size, D / 64, C2, (cuuint64_t)p.num_pages};
  cuuint64_t strides[4] = {C2 * Dkv * esz, 64 * esz, Dkv * esz, (cuuint64_t)p.page_size * C2 * Dkv * esz};
  // one box = 8 tokens x (K_h, V_h) x all of D: per token one contiguous 2*D-element run in global memory
  cuuint32_t box[5] = {64, 8, (cuuint32_t)(D / 64), 2, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMap map;
  const CUtensorMapDataType dt = (dtype == EJK_RPA_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(&map, dt, 5, const_cast<void*>(p.kv), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  return dispatch(p, dtype, map, n_sm, stream, pdl);
}

}  // namespace ejk
