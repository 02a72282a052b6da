// Prefill tiles of ragged paged attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// A chunked-prefill sequence contributes q_len*G (query token, head-in-group) rows per kv head;
// 128 of them form one tile, the M of a tcgen05.mma.  Per 64-token KV stage the tile needs two dense
// contractions, exactly the two einsums of the reference's inner loop
// (ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:119-124,148), here as
//     S[128 x 64]  = Q[128 x D] . K^T          tcgen05.mma kind::f16, A,B from shared memory, D in TMEM
//     O[128 x D]  += P[128 x 64] . V           tcgen05.mma, A (P) from TMEM, B (V) MN-major from shared
//                                              memory, accumulator in TMEM
// with the online softmax (:125-151) in between done by one thread per row on values read from TMEM
// with tcgen05.ld, so the row maximum and row sum need no shuffles at all.
//
// One CTA works on NT = 2 such tiles at once (256 consecutive rows of the same sequence and kv head;
// NT = 1 at head_dim 256 where TMEM holds only one O accumulator): both tiles consume the same KV
// stage, which halves the L2 -> shared-memory traffic per FLOP.  That traffic, not the tensor pipe,
// is what bounds a 128-row tile: a stage of 32 KB feeds only 4.2 MFLOP.
//
// Warp roles (64 + 128*NT threads, one CTA per SM, persistent over a device work queue):
//   warp 0      TMA producer: page-table driven gather of K_h / V_h, one box
//               {64 elems, 8 tokens, D/64, (K_h,V_h)} per 8-token group, SWIZZLE_128B.  A box keeps
//               the 2*D contiguous elements of a token together (512-byte runs in global memory;
//               the TMA unit's cost is per contiguous run, so 128-byte runs are 4x slower), and lands as
//               [group of 8 tokens][K|V][D/64][8 tokens][64]: 8-row x 128-byte swizzle atoms at a uniform
//               stride, i.e. a canonical K-major (K) / MN-major (V) operand of tcgen05.mma with
//               stride-byte-offset = one group.  No cluster multicast.
//   warp 1      MMA issuer (one lane): S for stage i+1 is issued before P.V of stage i so the tensor
//               pipe works while the softmax warps exponentiate; owns the TMEM allocation.
//   warps 2-5   softmax of tile 0 (warps 6-9: tile 1): thread = TMEM lane = tile row.  Loads the tile's query rows into the
//               K-major swizzled A layout, reads S, masks, exponentiates (log2 domain, lazy
//               rescaling of O in TMEM only when a row maximum grows by more than 2^8), writes P
//               (bf16 pairs) back into the TMEM columns S came from with tcgen05.st -- the A
//               operand of the P.V MMA -- and finally normalises O and stores the rows.  The tensor
//               pipe executes MMAs in issue order, so S of stage i+2 cannot overwrite those columns
//               before P.V of stage i has read them.
//
// All hand-offs are mbarriers; tcgen05.commit signals MMA completion.  Every wait is bounded: on
// expiry the warp sets the CTA abort flag, every other wait gives up when it sees the flag, the
// status word gets EJK_RPA_ST_TIMEOUT, and the CTA still frees its TMEM before it returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "rpa_tcgen05.cuh"
#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kBM = kPrefillRows;  // 128
constexpr int kBN = kTileTokens;   // 64
constexpr int kRingP = 16;
constexpr float kLog2eP = 1.4426950408889634f;
constexpr float kLazyP = 8.0f;

struct ItemDescP {
  Unit u;
  int32_t h;
  int32_t index;  // running item number of this CTA
  int32_t pad[6];
};

template <int D>
struct CfgP {
  static constexpr int NT = (D <= 128) ? 2 : 1;                    // 128-row tiles per CTA
  static constexpr int THREADS = 64 + 128 * NT;
  static constexpr int NS = (D == 64) ? 8 : (D == 128) ? 5 : 2;    // KV stages (as many as shared memory holds)
  static constexpr int STAGE_BYTES = kBN * 2 * D * 2;
  static constexpr int GROUP_BYTES = 8 * 2 * D * 2;   // one 8-token group: [K|V][D/64][8][64]
  static constexpr int V_OFF = (D / 64) * 1024;       // V atoms follow the K atoms inside a group
  static constexpr int Q_BYTES = kBM * D * 2;         // per tile
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + NT * Q_BYTES;
  static constexpr int OFF_RING = OFF_KV + NS * STAGE_BYTES;
  static constexpr int OFF_META = OFF_RING + kRingP * (int)sizeof(ItemDescP);
  static constexpr int OFF_BAR = OFF_META + NS * 8;
  // barriers: kv_full[NS] kv_empty[NS], then per tile: s_full[2] p_full[2] pv_done[2] q_full o_free
  static constexpr int BAR_PER_TILE = 8;
  static constexpr int N_BAR = 2 * NS + NT * BAR_PER_TILE;
  static constexpr int OFF_TMEM = OFF_BAR + N_BAR * 8;
  static constexpr int OFF_ABORT = OFF_TMEM + 8;
  static constexpr int SMEM_BYTES = OFF_ABORT + 8 + 1024;
  // TMEM columns: per tile two S/P buffers of 64 columns, then per tile one O accumulator of D columns
  static constexpr uint32_t TMEM_S = 0;
  static constexpr uint32_t TMEM_O = NT * 2 * kBN;
  static constexpr uint32_t TMEM_NEED = NT * (2 * kBN + D);
  static constexpr uint32_t TMEM_COLS = TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  static_assert(TMEM_NEED <= 512, "TMEM holds 512 columns");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

template <typename T, int D>
__global__ void __launch_bounds__(CfgP<D>::THREADS, 1)
rpa_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap, const Params p) {
  using C = CfgP<D>;
  constexpr int NS = C::NS, NT = C::NT;
  constexpr int DC = D / 64;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  ItemDescP* ring = reinterpret_cast<ItemDescP*>(smem + C::OFF_RING);
  int2* metas = reinterpret_cast<int2*>(smem + C::OFF_META);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_ABORT);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_TMEM);
  const uint32_t bar0 = sb + C::OFF_BAR;
  auto bar_kv_full = [&](int s) { return bar0 + s * 8; };
  auto bar_kv_empty = [&](int s) { return bar0 + (NS + s) * 8; };
  auto tile_bar = [&](int x, int i) { return bar0 + (2 * NS + x * C::BAR_PER_TILE + i) * 8; };
  auto bar_s_full = [&](int x, int b) { return tile_bar(x, b); };        // S(t) complete (commit)
  auto bar_p_full = [&](int x, int b) { return tile_bar(x, 2 + b); };    // P(t) stored to TMEM by the 4 warps
  auto bar_pv_done = [&](int x, int b) { return tile_bar(x, 4 + b); };   // P.V(t) complete (commit)
  auto bar_q_full = [&](int x) { return tile_bar(x, 6); };
  auto bar_o_free = [&](int x) { return tile_bar(x, 7); };

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Hkv = p.Hkv, G = p.G;
  const unsigned long long wait_ns = (unsigned long long)p.wait_timeout_ms * 1000000ull;
  unsigned flags = 0;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar_kv_full(s), 1);
      // released by the MMA warp's commit and by one thread of every softmax group (after it has
      // read the stage's metadata)
      mbar_init(bar_kv_empty(s), 1 + NT);
    }
    for (int x = 0; x < NT; ++x) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(bar_s_full(x, b), 1);
        mbar_init(bar_p_full(x, b), 4);  // one arrival per softmax warp
        mbar_init(bar_pv_done(x, b), 1);
      }
      mbar_init(bar_q_full(x), 4);
      mbar_init(bar_o_free(x), 4);
    }
    *abort_flag = 0;
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
  // programmatic dependent of the planner (see rpa_prefill_pp_sm100.cu)
  if (p.pdl & 1) pdl_wait();
  pdl_trigger();
  const int n_work = p.header[kHdrNumPrefill] * Hkv;

  if (warp == 0) {
    // =============================== TMA producer ===============================
    constexpr int kGroups = kBN / 8;                          // 8-token groups (= TMA boxes) per stage
    int gi = 0;  // global stage counter of this CTA
    int k = 0;
    int wid = 0;
    if (lane == 0) wid = atomicAdd(&p.header[kHdrPrefillQueue], 1);
    wid = __shfl_sync(0xffffffffu, wid, 0);
    bool alive = true;
    while (alive) {
      const int s = gi % NS;
      const uint32_t empty_parity = ((gi / NS) & 1) ^ 1;
      if (wid >= n_work) {
        if (!mbar_wait(bar_kv_empty(s), empty_parity, abort_flag, wait_ns)) break;
        if (lane == 0) {
          metas[s] = make_int2(-1, 0);
          mbar_arrive(bar_kv_full(s));
        }
        break;
      }
      const int ui = wid / Hkv;
      const int h = wid - ui * Hkv;
      Unit u;
      {
        const int4* src = reinterpret_cast<const int4*>(p.punits + ui);
        const int4 a = __ldg(src), b = __ldg(src + 1);
        u.seq = a.x; u.row0 = a.y; u.kv_begin = a.z; u.kv_end = a.w;
        u.slot = b.x; u.q_start = b.y; u.q_len = b.z; u.kv_len = b.w;
      }
      const int ring_slot = k % kRingP;
      int wid_next = 0;
      if (lane == 0) wid_next = atomicAdd(&p.header[kHdrPrefillQueue], 1);
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
        if (lane == 0) {
          if (first) {
            // the consumers are at most NS stages (hence at most NS items) behind: slot k-kRingP is free
            ItemDescP d;
            d.u = u;
            d.h = h;
            d.index = k;
            ring[ring_slot] = d;
          }
          // meta.x = ring slot | 0x100 on the first stage of an item | 0x200 when the item has rows for tile 1
          const bool two = (NT == 2) && (u.q_len * G > u.row0 + kBM);
          metas[st] = make_int2(ring_slot | (first ? 0x100 : 0) | (two ? 0x200 : 0), pos);
          const uint32_t bytes = (uint32_t)ngrp * C::GROUP_BYTES;
          if (bytes > 0) mbar_arrive_expect_tx(bar_kv_full(st), bytes);
          else mbar_arrive(bar_kv_full(st));
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
      wid = __shfl_sync(0xffffffffu, wid_next, 0);
    }
    // wait (bounded) until every stage this warp filled has been released, i.e. all its bulk
    // copies have landed and been consumed
    for (int i = 0; i < NS && gi > 0; ++i) {
      const int g2 = gi + i;
      if (g2 < NS) continue;  // never used
      if (!mbar_wait(bar_kv_empty(g2 % NS), ((g2 / NS) & 1) ^ 1, abort_flag, wait_ns)) break;
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    constexpr uint32_t idesc_s = instr_desc<T>(kBN, false);
    constexpr uint32_t idesc_pv = instr_desc<T>(D, true);
    int gi = 0;                  // KV stage counter
    int tcount[NT];              // stages issued per tile (drives the S / P buffer parities)
    int items[NT];               // items started per tile
    int prev_t[NT];
    bool prev_act[NT];
#pragma unroll
    for (int x = 0; x < NT; ++x) {
      tcount[x] = 0;
      items[x] = 0;
      prev_t[x] = 0;
      prev_act[x] = false;
    }
    bool have_prev = false, prev_first = false;
    int prev_st = 0;
    bool ok = true;

    // Descriptors are built once; per MMA only a small constant is added to the address field
    // (the issuing thread's scalar work would otherwise cost more than the MMA itself).
    // hi word: stride byte offset >> 4, version 1 (bit 46), SWIZZLE_128B (bits 61-63).
    constexpr uint64_t kHiAtom1024 = ((uint64_t)((1024u >> 4) | (1u << 14) | (2u << 29))) << 32;
    constexpr uint64_t kHiGroup = ((uint64_t)(((uint32_t)C::GROUP_BYTES >> 4) | (1u << 14) | (2u << 29))) << 32;
    uint64_t q_desc[NT];
#pragma unroll
    for (int x = 0; x < NT; ++x) q_desc[x] = kHiAtom1024 | (uint64_t)(((sb + C::OFF_Q + x * C::Q_BYTES) >> 4) | (1u << 16));
    const uint64_t k_desc0 = kHiGroup | (uint64_t)(((sb + C::OFF_KV) >> 4) | (1u << 16));
    // V is MN-major: leading byte offset = distance between 64-element chunks of D (1024 B)
    const uint64_t v_desc0 = kHiGroup | (uint64_t)(((sb + C::OFF_KV + C::V_OFF) >> 4) | ((1024u >> 4) << 16));

    // Consecutive tcgen05.mma that accumulate into the same TMEM tile serialise on the accumulator,
    // so the two tiles' MMAs are issued alternately: every instruction is independent of the one
    // before it.  The whole role runs on lane 0: its scalar work between MMAs is on the critical
    // path of every stage, so it is kept to a few instructions (no warp votes, flags ride in the
    // stage metadata instead of being re-derived from the item descriptor).
    if (lane == 0) {
      // S_x = Q_x . K^T of stage `st` into S buffer tcount[x] & 1, for every tile in `act`.  That
      // buffer last held P of stage tcount[x]-2, which P.V of that stage -- issued earlier, and MMAs
      // execute in issue order -- has finished reading by the time this MMA writes.
      auto issue_s = [&](const bool (&act)[NT], int st) {
        tc_fence_after();
        const uint64_t kd = k_desc0 + (uint64_t)((st * C::STAGE_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          // K: 8-token atoms one group apart (SBO), the 64-element chunks of D 1024 bytes apart
          const uint64_t bd = kd + (uint64_t)(((kk >> 2) * 1024 + (kk & 3) * 32) >> 4);
#pragma unroll
          for (int x = 0; x < NT; ++x) {
            if (!act[x]) continue;
            const uint64_t ad = q_desc[x] + (uint64_t)(((kk >> 2) * (kBM * 128) + (kk & 3) * 32) >> 4);
            tc_mma(tmem_base + C::TMEM_S + (x * 2 + (tcount[x] & 1)) * kBN, ad, bd, idesc_s, kk > 0);
          }
        }
#pragma unroll
        for (int x = 0; x < NT; ++x)
          if (act[x]) tc_commit(bar_s_full(x, tcount[x] & 1));
      };
      // O_x (+)= P_x . V of the previous stage, for every tile that took part in it; P_x sits in TMEM
      auto issue_pv = [&]() -> bool {
#pragma unroll
        for (int x = 0; x < NT; ++x) {
          if (!prev_act[x]) continue;
          const int t = prev_t[x];
          if (!mbar_wait_thread(bar_p_full(x, t & 1), (t >> 1) & 1, abort_flag, wait_ns)) return false;
        }
        tc_fence_after();
        const uint64_t vd = v_desc0 + (uint64_t)((prev_st * C::STAGE_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          // V: 16 tokens = two 8-token groups per MMA
          const uint64_t bd = vd + (uint64_t)((kk * 2 * C::GROUP_BYTES) >> 4);
#pragma unroll
          for (int x = 0; x < NT; ++x) {
            if (!prev_act[x]) continue;
            // P: 16 tokens = 8 columns of bf16 pairs
            const uint32_t a_tmem = tmem_base + C::TMEM_S + (x * 2 + (prev_t[x] & 1)) * kBN + kk * 8;
            tc_mma_ts(tmem_base + C::TMEM_O + x * D, a_tmem, bd, idesc_pv, !(prev_first && kk == 0));
          }
        }
#pragma unroll
        for (int x = 0; x < NT; ++x)
          if (prev_act[x]) tc_commit(bar_pv_done(x, prev_t[x] & 1));  // O_x holds this stage
        tc_commit(bar_kv_empty(prev_st));  // every MMA that read this KV stage is complete
        have_prev = false;
        return true;
      };

      while (ok) {
        const int st = gi % NS;
        if (!mbar_wait_thread(bar_kv_full(st), (gi / NS) & 1, abort_flag, wait_ns)) break;
        const int mx = metas[st].x;
        if (mx < 0) {
          if (have_prev) issue_pv();
          break;
        }
        const bool first = (mx & 0x100) != 0;
        bool act[NT];
        act[0] = true;
        if (NT == 2) act[NT - 1] = (mx & 0x200) != 0;
        if (!first) {
          // steady state: S of this stage goes to the tensor pipe before P.V of the previous one, so
          // the pipe has work while the softmax warps exponentiate
          issue_s(act, st);
          if (have_prev) ok = issue_pv();
        } else {
          // item boundary: finish the previous item first -- its epilogue must read O before this
          // item's query tiles are loaded and before the first P.V of this item overwrites O
          if (have_prev) ok = issue_pv();
#pragma unroll
          for (int x = 0; x < NT; ++x) {
            if (!ok || !act[x]) continue;
            ok = mbar_wait_thread(bar_q_full(x), items[x] & 1, abort_flag, wait_ns);
            if (ok && items[x] > 0) ok = mbar_wait_thread(bar_o_free(x), (items[x] - 1) & 1, abort_flag, wait_ns);
            ++items[x];
          }
          if (ok) issue_s(act, st);
        }
        if (!ok) break;
        have_prev = true;
        prev_st = st;
        prev_first = first;
#pragma unroll
        for (int x = 0; x < NT; ++x) {
          prev_act[x] = act[x];
          prev_t[x] = tcount[x];
          if (act[x]) ++tcount[x];
        }
        ++gi;
      }
    }
    __syncwarp();
  } else {
    // =============================== softmax warps ===============================
    const int x = (warp - 2) >> 2;                        // which tile of the CTA
    const int row = (warp & 3) * 32 + lane;               // TMEM lane == row within the tile
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int grp_tid = (tid - 64) & 127;                 // 0..127 within the softmax group
    const bool grp_leader = (grp_tid == 0);
    const uint32_t tm_s = tmem_base + lane_addr + C::TMEM_S + x * 2 * kBN;
    const uint32_t tm_o = tmem_base + lane_addr + C::TMEM_O + x * D;
    uint8_t* q_smem = smem + C::OFF_Q + x * C::Q_BYTES;
    int gi = 0;   // KV stage counter (all roles see the same stage sequence)
    int ti = 0;   // stages this tile took part in
    float m_run = -INFINITY, l_run = 0.f;
    int pos_row = -1, lo_row = -1;
    bool row_ok = false, active = false;
    int out_row_q = 0, out_head = 0;
    Unit u;
    u.kv_begin = u.kv_end = 0;
    int h = 0;
    while (true) {
      const int st = gi % NS;
      if (!mbar_wait(bar_kv_full(st), (gi / NS) & 1, abort_flag, wait_ns)) break;
      const int2 meta = metas[st];
      if (meta.x < 0) break;
      const int pos = meta.y;
      const bool first = (meta.x & 0x100) != 0;
      if (first) {
        u = ring[meta.x & 0xff].u;
        h = ring[meta.x & 0xff].h;
        active = (x == 0) || (meta.x & 0x200) != 0;
      }
      // this group has read the stage's metadata: its share of the stage's release
      if (grp_leader) mbar_arrive(bar_kv_empty(st));
      if (!active) {  // the item has no rows for this tile
        ++gi;
        continue;
      }
      if (first) {
        // ---- new item: row bookkeeping and the query tile (K-major, 128B swizzle) ----
        const int rows_total = u.q_len * G;
        const int R = u.row0 + x * kBM + row;
        row_ok = R < rows_total;
        const int qt = R / G, g = R - qt * G;
        out_row_q = u.q_start + qt;
        out_head = h * G + g;
        pos_row = row_ok ? (u.kv_len - u.q_len + qt) : -1;
        lo_row = (p.window > 0) ? pos_row - p.window : -1;
        m_run = -INFINITY;
        l_run = 0.f;
        // all S MMAs of this tile's previous item completed before its last s_full fired, which
        // this thread waited for, so the query tile may be overwritten
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.q) +
                                                          ((size_t)out_row_q * p.Hq + out_head) * D * sizeof(T));
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (row_ok) v = __ldg(src + c);
          const uint32_t off = (uint32_t)(c >> 3) * (kBM * 128) + (uint32_t)row * 128 + (uint32_t)(((c & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(q_smem + off) = v;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_q_full(x));
      }
      const int b = ti & 1;
      if (!mbar_wait(bar_s_full(x, b), (ti >> 1) & 1, abort_flag, wait_ns)) break;
      tc_fence_after();
      uint32_t sr[2][32];
      tc_ld32(tm_s + b * kBN, sr[0]);
      tc_ld32(tm_s + b * kBN + 32, sr[1]);
      tc_wait_ld();

      // logits in the log2 domain, soft cap, masks (_xla_impl_fwd.py:125-138).  The common case (no
      // cap, stage entirely visible to this row) keeps the raw dot products and folds the scale into
      // the exponent's FMA; everything else materialises the transformed logits first.
      const bool full_vis = (pos + kBN - 1 <= pos_row) && (pos > lo_row);
      const bool plain = full_vis && p.cap == 0.f;
      float e_scale = p.scale_log2;  // p = exp2(v * e_scale - m)
      float mx;
      if (plain) {
        // max of scale*v is scale*max(v) or scale*min(v) depending on the sign of the scale
        // (four independent chains: few warps per scheduler, so latency must be hidden in-thread)
        float ext[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) ext[a] = __uint_as_float(sr[0][a]);
        if (p.scale_log2 >= 0.f) {
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf)
#pragma unroll
            for (int c = 0; c < 32; ++c) ext[c & 3] = fmaxf(ext[c & 3], __uint_as_float(sr[hlf][c]));
          mx = fmaxf(fmaxf(ext[0], ext[1]), fmaxf(ext[2], ext[3])) * p.scale_log2;
        } else {
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf)
#pragma unroll
            for (int c = 0; c < 32; ++c) ext[c & 3] = fminf(ext[c & 3], __uint_as_float(sr[hlf][c]));
          mx = fminf(fminf(ext[0], ext[1]), fminf(ext[2], ext[3])) * p.scale_log2;
        }
      } else {
        mx = -INFINITY;
        e_scale = 1.f;
        if (p.cap != 0.f) {
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf)
#pragma unroll
            for (int c = 0; c < 32; ++c)
              sr[hlf][c] = __float_as_uint(p.cap_log2 * soft_cap_tanh(__uint_as_float(sr[hlf][c]) * p.inv_cap_scale));
        } else {
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf)
#pragma unroll
            for (int c = 0; c < 32; ++c) sr[hlf][c] = __float_as_uint(__uint_as_float(sr[hlf][c]) * p.scale_log2);
        }
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            float xv = __uint_as_float(sr[hlf][c]);
            const int key = pos + hlf * 32 + c;
            if (!full_vis && (key > pos_row || key <= lo_row)) xv = -INFINITY;
            sr[hlf][c] = __float_as_uint(xv);
            mx = fmaxf(mx, xv);
          }
      }
      const bool grow = (mx > m_run + kLazyP) || (m_run == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        float alpha = 1.f;
        if (grow) {
          alpha = fast_exp2(m_run - mx);  // 0 on the first finite maximum
          m_run = mx;
          l_run *= alpha;
        }
        if (!first) {
          // O holds the sum over the earlier stages of this item: rescale this warp's 32 lanes.
          // This tile's P.V of stage ti-1 must have completed first.
          if (!mbar_wait(bar_pv_done(x, (ti - 1) & 1), ((ti - 1) >> 1) & 1, abort_flag, wait_ns)) break;
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            tc_ld32(tm_o + c0, o);
            tc_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            tc_st32(tm_o + c0, o);
          }
          tc_wait_st();
          tc_fence_before();
        }
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      // probabilities, packed as bf16 pairs, go back into the TMEM columns S came from
      float lsum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int c = 2 * j;
        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c >> 5][c & 31]), e_scale, -m_use));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]), e_scale, -m_use));
        lsum4[j & 3] += p0 + p1;
        pk[j] = Mma<T>::pack(p0, p1);
      }
      tc_st32(tm_s + b * kBN, pk);
      l_run += (lsum4[0] + lsum4[1]) + (lsum4[2] + lsum4[3]);
      if (x == 0 && pos + kBN > u.kv_end) {
        // Tail stage: V rows of keys >= kv_end were either never fetched (stale shared memory) or lie
        // past the sequence's length inside its last page (unowned, possibly NaN).  Their
        // probabilities are exactly 0, but 0 * NaN would poison O, so tile 0's group clears the rows
        // before any tensor-core read: the MMA warp issues tile 1's P.V only after it has seen tile
        // 0's p_full.  (Zero rows are invariant under the swizzle.)
        int nvalid = u.kv_end - pos;
        if (nvalid < 0) nvalid = 0;
        uint8_t* vbase = smem + C::OFF_KV + st * C::STAGE_BYTES + C::V_OFF;
        const int n16 = (kBN - nvalid) * DC * 8;
        for (int idx = grp_tid; idx < n16; idx += 128) {
          const int t = nvalid + idx / (DC * 8);
          const int rem = idx % (DC * 8);
          *reinterpret_cast<uint4*>(vbase + (t >> 3) * C::GROUP_BYTES + (rem >> 3) * 1024 + (t & 7) * 128 + (rem & 7) * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
      }
      if (x == 0 && pos + kBN > u.kv_end) fence_async_smem();  // the zeroed V rows are read by the async proxy
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full(x, b));

      if (pos + kBN >= u.kv_end) {
        // ---- last stage of the item: wait for its PV, normalise, store ----
        if (!mbar_wait(bar_pv_done(x, b), (ti >> 1) & 1, abort_flag, wait_ns)) break;
        tc_fence_after();
        float scl = 1.f, l_fin = l_run;
        if (p.num_sinks > 0 && row_ok) {
          // attention sinks join the denominator only (_xla_impl_fwd.py:161-172)
          const int srow = (p.sink_rows == p.Hq) ? out_head : (p.sink_rows == Hkv ? h : 0);
          const float* sk = p.sinks + (size_t)srow * p.num_sinks;
          float sm = -INFINITY;
          for (int i = 0; i < p.num_sinks; ++i) sm = fmaxf(sm, sk[i] * kLog2eP);
          const float m_fin = fmaxf(m_run, sm);
          const float mf = (m_fin == -INFINITY) ? 0.f : m_fin;
          scl = fast_exp2(m_run - mf);
          l_fin = l_run * scl;
          for (int i = 0; i < p.num_sinks; ++i) l_fin += fast_exp2(sk[i] * kLog2eP - mf);
        }
        scl = (l_fin > 0.f) ? scl / l_fin : 0.f;
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
      ++ti;
      ++gi;
    }
  }
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

template <typename T>
cudaError_t dispatch(const Params& p, const CUtensorMap& map, int n_sm, cudaStream_t stream, bool pdl) {
  switch (p.D) {
    case 64: return launch_one<T, 64>(p, map, n_sm, stream, pdl);
    case 128: return launch_one<T, 128>(p, map, n_sm, stream, pdl);
    case 256: return launch_one<T, 256>(p, map, n_sm, stream, pdl);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

// rpa_prefill_pp_sm100.cu
cudaError_t launch_prefill_pingpong(const Params& p, int dtype, const CUtensorMap& map, int n_sm, cudaStream_t stream, bool pdl);

int prefill_rows_per_item(int head_dim) { return head_dim <= 128 ? 2 * kPrefillRows : kPrefillRows; }

bool prefill_path_supported(const Params& p) {
  const int ps = p.page_size;
  if (ps < 8 || (ps & (ps - 1)) != 0) return false;
  return encode_fn_p() != nullptr;
}

cudaError_t launch_prefill(const Params& p, int dtype, int n_sm, cudaStream_t stream, bool pdl) {
  EncodeFn enc = encode_fn_p();
  if (!enc) return cudaErrorNotSupported;
  const uint64_t esz = 2;
  const uint64_t D = p.D, C2 = 2ull * p.Hkv;
  cuuint64_t dims[5] = {64, (cuuint64_t)p.page_size, D / 64, C2, (cuuint64_t)p.num_pages};
  cuuint64_t strides[4] = {C2 * D * esz, 64 * esz, D * esz, (cuuint64_t)p.page_size * C2 * D * esz};
  // one box = 8 tokens x (K_h, V_h) x all of D: per token one contiguous 2*D-element run in global memory
  cuuint32_t box[5] = {64, 8, (cuuint32_t)(D / 64), 2, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMap map;
  const CUtensorMapDataType dt = (dtype == EJK_RPA_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(&map, dt, 5, const_cast<void*>(p.kv), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  if (p.D <= 128 && p.prefill_kernel == 0) return launch_prefill_pingpong(p, dtype, map, n_sm, stream, pdl);
  if (dtype == EJK_RPA_BF16) return dispatch<__nv_bfloat16>(p, map, n_sm, stream, pdl);
  return dispatch<__half>(p, map, n_sm, stream, pdl);
}

}  // namespace ejk
