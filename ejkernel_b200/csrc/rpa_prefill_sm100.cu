// Prefill tiles of ragged paged attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// A chunked-prefill sequence contributes q_len*G (query token, head-in-group) rows per kv head;
// 128 of them form one tile, the M of a tcgen05.mma.  Per 64-token KV stage the tile needs two dense
// contractions, exactly the two einsums of the reference's inner loop
// (ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:119-124,148), here as
//     S[128 x 64]  = Q[128 x D] . K^T          tcgen05.mma kind::f16, A,B from shared memory, D in TMEM
//     O[128 x D]  += P[128 x 64] . V           tcgen05.mma, B operand MN-major, accumulator in TMEM
// with the online softmax (:125-151) in between done by one thread per row on values read from TMEM
// with tcgen05.ld, so the row maximum and row sum need no shuffles at all.
//
// Warp roles (192 threads, one CTA per SM, persistent over a device work queue):
//   warp 0      TMA producer: page-table driven gather of K_h / V_h, one box {64 elems, PB tokens}
//               per (K|V, 64-element chunk of D, page block), SWIZZLE_128B, into a stage laid out
//               [K|V][D/64][64 tokens][64] = the canonical K-major (for K) / MN-major (for V)
//               128B-swizzled operand layout of tcgen05.mma.  No cluster multicast.
//   warp 1      MMA issuer (one lane): S for stage i+1 is issued before P.V of stage i so the tensor
//               pipe works while the softmax warps exponentiate; owns the TMEM allocation.
//   warps 2-5   softmax: thread = TMEM lane = tile row.  Loads the tile's query rows into the
//               K-major swizzled A layout, reads S, masks, exponentiates (log2 domain, lazy
//               rescaling of O in TMEM only when a row maximum grows by more than 2^8), writes P
//               (bf16) as the next A operand, and finally normalises O and stores the rows.
//
// All hand-offs are mbarriers; tcgen05.commit signals MMA completion.  Every wait is bounded: on
// expiry the warp sets the CTA abort flag, every other wait gives up when it sees the flag, the
// status word gets EJK_RPA_ST_TIMEOUT, and the CTA still frees its TMEM before it returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "rpa_device.cuh"
#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kBM = kPrefillRows;  // 128
constexpr int kBN = kTileTokens;   // 64
constexpr int kThreadsP = 192;
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
  static constexpr int NS = (D == 64) ? 8 : (D == 128) ? 5 : 2;  // KV stages (as many as shared memory holds)
  static constexpr int NP = (D <= 128) ? 2 : 1;   // P buffers
  static constexpr int STAGE_BYTES = kBN * 2 * D * 2;
  static constexpr int KV_HALF = kBN * D * 2;     // bytes of the K (or V) part of a stage
  static constexpr int Q_BYTES = kBM * D * 2;
  static constexpr int P_BYTES = kBM * kBN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + Q_BYTES;
  static constexpr int OFF_P = OFF_KV + NS * STAGE_BYTES;
  static constexpr int OFF_RING = OFF_P + NP * P_BYTES;
  static constexpr int OFF_META = OFF_RING + kRingP * (int)sizeof(ItemDescP);
  static constexpr int OFF_BAR = OFF_META + NS * 8;
  // barriers: kv_full[NS] kv_empty[NS] s_full[2] s_free[2] p_full[NP] p_free[NP] q_full o_free
  static constexpr int N_BAR = 2 * NS + 4 + 2 * NP + 2;
  static constexpr int OFF_TMEM = OFF_BAR + N_BAR * 8;
  static constexpr int OFF_ABORT = OFF_TMEM + 8;
  static constexpr int SMEM_BYTES = OFF_ABORT + 8 + 1024;
  static constexpr uint32_t TMEM_S = 0;       // two S buffers of 64 columns
  static constexpr uint32_t TMEM_O = 2 * kBN; // O accumulator, D columns
  static constexpr uint32_t TMEM_COLS = (2 * kBN + D <= 256) ? 256 : 512;  // power of two >= 128 + D
};

// ---- PTX wrappers (mbarrier helpers live in rpa_device.cuh) ----
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t addr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t addr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(addr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 encoding: start>>4 at [0,14),
// leading byte offset>>4 at [16,30), stride byte offset>>4 at [32,46), version 1 at [46,48),
// layout type 2 (SWIZZLE_128B) at [61,64).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor of kind::f16: D fp32, A/B bf16 or f16, M = 128.
template <typename T>
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn_major) {
  const uint32_t fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kBM >> 4) << 24);
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreadsP, 1)
rpa_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap, const Params p) {
  using C = CfgP<D>;
  constexpr int NS = C::NS, NP = C::NP;
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
  auto bar_s_full = [&](int b) { return bar0 + (2 * NS + b) * 8; };
  auto bar_s_free = [&](int b) { return bar0 + (2 * NS + 2 + b) * 8; };
  auto bar_p_full = [&](int b) { return bar0 + (2 * NS + 4 + b) * 8; };
  auto bar_p_free = [&](int b) { return bar0 + (2 * NS + 4 + NP + b) * 8; };
  const uint32_t bar_q_full = bar0 + (2 * NS + 4 + 2 * NP) * 8;
  const uint32_t bar_o_free = bar_q_full + 8;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Hkv = p.Hkv, G = p.G;
  const int n_work = p.header[kHdrNumPrefill] * Hkv;
  const int pb = p.tma_block_tokens, pb_shift = p.tma_block_shift;
  const unsigned long long wait_ns = (unsigned long long)p.wait_timeout_ms * 1000000ull;
  unsigned flags = 0;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_s_full(b), 1);
      mbar_init(bar_s_free(b), 4);  // one arrival per softmax warp
    }
    for (int b = 0; b < NP; ++b) {
      mbar_init(bar_p_full(b), 4);
      mbar_init(bar_p_free(b), 1);
    }
    mbar_init(bar_q_full, 4);
    mbar_init(bar_o_free, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    // TMEM: two S buffers (2 x 64 columns) + O (D columns)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(sb + C::OFF_TMEM), "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =============================== TMA producer ===============================
    const int blocks_per_stage = kBN >> pb_shift;
    const int boxes_per_block = 2 * DC;                      // (K|V) x 64-element chunks of D
    const uint32_t box_bytes = (uint32_t)pb * 128;
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
        if (!mbar_wait(bar_kv_empty(st), ((gi / NS) & 1) ^ 1, abort_flag, wait_ns)) {
          alive = false;
          break;
        }
        int nblk = (u.kv_end - pos + pb - 1) >> pb_shift;
        if (nblk > blocks_per_stage) nblk = blocks_per_stage;
        if (nblk < 0) nblk = 0;
        if (lane == 0) {
          if (first) {
            // The ring slot of item k was last used by item k-4, whose stages are long consumed:
            // the consumers are at most NS stages behind, and every item has at least one stage.
            ItemDescP d;
            d.u = u;
            d.h = h;
            d.index = k;
            ring[ring_slot] = d;
          }
          metas[st] = make_int2(ring_slot, pos);
          const uint32_t bytes = (uint32_t)nblk * boxes_per_block * box_bytes;
          if (bytes > 0) mbar_arrive_expect_tx(bar_kv_full(st), bytes);
          else mbar_arrive(bar_kv_full(st));
        }
        __syncwarp();
        // one box per (page block j, K|V, chunk dc): lane -> (j, kv, dc)
        const int nbox = nblk * boxes_per_block;
        for (int bi = lane; bi < nbox; bi += 32) {
          const int j = bi / boxes_per_block;
          const int rem = bi - j * boxes_per_block;
          const int kv = rem / DC, dc = rem - kv * DC;
          const int key = pos + (j << pb_shift);
          int pi, off;
          if (p.page_shift >= 0) {
            pi = key >> p.page_shift;
            off = key & (p.page_size - 1);
          } else {
            pi = key / p.page_size;
            off = key - pi * p.page_size;
          }
          int page = __ldg(tab + pi);
          if ((unsigned)page >= (unsigned)p.num_pages) {
            flags |= EJK_RPA_ST_PAGE_ID;
            page = 0;
          }
          const uint32_t dst = sb + C::OFF_KV + st * C::STAGE_BYTES + (uint32_t)(kv * DC + dc) * (kBN * 128) +
                               (uint32_t)(j << pb_shift) * 128;
          tma_load_5d(dst, &tmap, bar_kv_full(st), 0, off, dc, 2 * h + kv, page);
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
    int gi = 0;       // stage whose S is issued next
    int k_items = 0;  // items started
    bool have_prev = false, prev_first = false;
    int prev_st = 0, prev_gi = 0;
    bool ok = true;

    // S(gi) = Q . K^T of stage `st` into S buffer gi & 1
    auto issue_s = [&](int st) -> bool {
      const int b = gi & 1;
      // the softmax warps must have drained the previous use of this S buffer
      if (!mbar_wait(bar_s_free(b), ((gi >> 1) & 1) ^ 1, abort_flag, wait_ns)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t q_base = sb + C::OFF_Q;
        const uint32_t k_base = sb + C::OFF_KV + st * C::STAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t coff = (uint32_t)(kk >> 2), koff = (uint32_t)(kk & 3) * 32;
          const uint64_t ad = smem_desc(q_base + coff * (kBM * 128) + koff, 16, 1024);
          const uint64_t bd = smem_desc(k_base + coff * (kBN * 128) + koff, 16, 1024);
          tc_mma(tmem_base + C::TMEM_S + b * kBN, ad, bd, idesc_s, kk > 0);
        }
        tc_commit(bar_s_full(b));
      }
      __syncwarp();
      return true;
    };
    // O (+)= P . V of the previous stage
    auto issue_pv = [&]() -> bool {
      const int pbuf = prev_gi % NP;
      if (!mbar_wait(bar_p_full(pbuf), (prev_gi / NP) & 1, abort_flag, wait_ns)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t p_base = sb + C::OFF_P + pbuf * C::P_BYTES;
        const uint32_t v_base = sb + C::OFF_KV + prev_st * C::STAGE_BYTES + C::KV_HALF;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          const uint64_t ad = smem_desc(p_base + kk * 32, 16, 1024);
          // V: MN-major, 64-element chunks of D are kBN*128 bytes apart (LBO), 8-token groups 1024 (SBO)
          const uint64_t bd = smem_desc(v_base + kk * (16 * 128), kBN * 128, 1024);
          tc_mma(tmem_base + C::TMEM_O, ad, bd, idesc_pv, !(prev_first && kk == 0));
        }
        tc_commit(bar_p_free(pbuf));       // P buffer reusable; O holds this stage
        tc_commit(bar_kv_empty(prev_st));  // both MMAs that read this KV stage are complete
      }
      __syncwarp();
      have_prev = false;
      return true;
    };

    while (ok) {
      const int st = gi % NS;
      if (!mbar_wait(bar_kv_full(st), (gi / NS) & 1, abort_flag, wait_ns)) break;
      const int2 meta = metas[st];
      if (meta.x < 0) {
        if (have_prev) issue_pv();
        break;
      }
      const bool first = (meta.y == ring[meta.x].u.kv_begin);
      if (!first) {
        // steady state: S of this stage goes to the tensor pipe before P.V of the previous one, so
        // the pipe has work while the softmax warps exponentiate
        ok = issue_s(st);
        if (ok && have_prev) ok = issue_pv();
      } else {
        // item boundary: finish the previous item first -- its epilogue must read O before this
        // item's query tile is loaded and before the first P.V of this item overwrites O
        if (have_prev) ok = issue_pv();
        if (ok) ok = mbar_wait(bar_q_full, k_items & 1, abort_flag, wait_ns);
        if (ok && k_items > 0) ok = mbar_wait(bar_o_free, (k_items - 1) & 1, abort_flag, wait_ns);
        ++k_items;
        if (ok) ok = issue_s(st);
      }
      if (!ok) break;
      have_prev = true;
      prev_st = st;
      prev_gi = gi;
      prev_first = first;
      ++gi;
    }
  } else {
    // =============================== softmax warps ===============================
    const int row = (warp & 3) * 32 + lane;             // TMEM lane == tile row
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int st_tid = tid - 64;                         // 0..127
    int gi = 0;
    float m_run = -INFINITY, l_run = 0.f;
    int pos_row = -1, lo_row = -1;
    bool row_ok = false;
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
      if (pos == ring[meta.x].u.kv_begin) {
        // ---- new item: row bookkeeping and the query tile (K-major, 128B swizzle) ----
        u = ring[meta.x].u;
        h = ring[meta.x].h;
        const int rows_total = u.q_len * G;
        const int R = u.row0 + row;
        row_ok = R < rows_total;
        const int qt = R / G, g = R - qt * G;
        out_row_q = u.q_start + qt;
        out_head = h * G + g;
        pos_row = row_ok ? (u.kv_len - u.q_len + qt) : -1;
        lo_row = (p.window > 0) ? pos_row - p.window : -1;
        m_run = -INFINITY;
        l_run = 0.f;
        // all S MMAs of the previous item completed before its last s_full fired, which this
        // thread waited for, so the Q tile may be overwritten
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.q) +
                                                          ((size_t)out_row_q * p.Hq + out_head) * D * sizeof(T));
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (row_ok) v = __ldg(src + c);
          const uint32_t off = (uint32_t)(c >> 3) * (kBM * 128) + (uint32_t)row * 128 + (uint32_t)(((c & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(smem + C::OFF_Q + off) = v;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_q_full);
      }
      const int b = gi & 1;
      if (!mbar_wait(bar_s_full(b), (gi >> 1) & 1, abort_flag, wait_ns)) break;
      tc_fence_after();
      uint32_t sr[2][32];
      tc_ld32(tmem_base + lane_addr + C::TMEM_S + b * kBN, sr[0]);
      tc_ld32(tmem_base + lane_addr + C::TMEM_S + b * kBN + 32, sr[1]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_s_free(b));

      // logits in the log2 domain, soft cap, masks (_xla_impl_fwd.py:125-138).  The common case (no
      // cap, stage entirely visible to this row) keeps the raw dot products and folds the scale into
      // the exponent's FMA; everything else materialises the transformed logits first.
      const bool full_vis = (pos + kBN - 1 <= pos_row) && (pos > lo_row);
      const bool plain = full_vis && p.cap == 0.f;
      float e_scale = p.scale_log2;  // p = exp2(v * e_scale - m)
      float mx;
      if (plain) {
        // max of scale*v is scale*max(v) or scale*min(v) depending on the sign of the scale
        // (four independent chains: one warp per scheduler has nothing else to hide latency with)
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
            float x = __uint_as_float(sr[hlf][c]);
            const int key = pos + hlf * 32 + c;
            if (!full_vis && (key > pos_row || key <= lo_row)) x = -INFINITY;
            sr[hlf][c] = __float_as_uint(x);
            mx = fmaxf(mx, x);
          }
      }
      const bool first_stage = (pos == u.kv_begin);
      const bool grow = (mx > m_run + kLazyP) || (m_run == -INFINITY && mx > -INFINITY);
      const int pbuf = gi % NP;
      // P buffer pbuf was last read by PV(gi - NP)
      if (!mbar_wait(bar_p_free(pbuf), ((gi / NP) & 1) ^ 1, abort_flag, wait_ns)) break;
      if (__any_sync(0xffffffffu, grow)) {
        float alpha = 1.f;
        if (grow) {
          alpha = fast_exp2(m_run - mx);  // 0 on the first finite maximum
          m_run = mx;
          l_run *= alpha;
        }
        if (!first_stage) {
          // O holds the sum over the earlier stages of this item: rescale this warp's 32 lanes.
          // PV(gi-1) must have completed first.
          if (NP == 2) {
            const int pprev = (gi - 1) % NP;
            if (!mbar_wait(bar_p_free(pprev), ((gi - 1) / NP) & 1, abort_flag, wait_ns)) break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            tc_ld32(tmem_base + lane_addr + C::TMEM_O + c0, o);
            tc_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            tc_st32(tmem_base + lane_addr + C::TMEM_O + c0, o);
          }
          tc_wait_st();
          tc_fence_before();
        }
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      float lsum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* prow = smem + C::OFF_P + pbuf * C::P_BYTES + row * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = c8 * 8 + e * 2;
          const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c >> 5][c & 31]), e_scale, -m_use));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]), e_scale, -m_use));
          lsum4[e] += p0 + p1;
          pk[e] = Mma<T>::pack(p0, p1);
        }
        *reinterpret_cast<uint4*>(prow + ((c8 ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l_run += (lsum4[0] + lsum4[1]) + (lsum4[2] + lsum4[3]);
      if (pos + kBN > u.kv_end) {
        // Tail stage: V rows of keys >= kv_end were either never fetched (stale shared memory) or lie
        // past the sequence's length inside its last page (unowned, possibly NaN).  Their
        // probabilities are exactly 0, but 0 * NaN would poison O, so the rows are cleared before
        // the tensor core reads them.  (Zero rows are invariant under the swizzle.)
        int nvalid = u.kv_end - pos;
        if (nvalid < 0) nvalid = 0;
        uint8_t* vbase = smem + C::OFF_KV + st * C::STAGE_BYTES + C::KV_HALF;
        const int n16 = (kBN - nvalid) * DC * 8;
        for (int idx = st_tid; idx < n16; idx += 128) {
          const int t = nvalid + idx / (DC * 8);
          const int rem = idx % (DC * 8);
          *reinterpret_cast<uint4*>(vbase + (rem >> 3) * (kBN * 128) + t * 128 + (rem & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full(pbuf));

      if (pos + kBN >= u.kv_end) {
        // ---- last stage of the item: wait for its PV, normalise, store ----
        if (!mbar_wait(bar_p_free(pbuf), (gi / NP) & 1, abort_flag, wait_ns)) break;
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
          tc_ld32(tmem_base + lane_addr + C::TMEM_O + c0, o);
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
        if (lane == 0) mbar_arrive(bar_o_free);
      }
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
cudaError_t launch_one(const Params& p, const CUtensorMap& map, int n_sm, cudaStream_t stream) {
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
  kern<<<n_sm, kThreadsP, C::SMEM_BYTES, stream>>>(map, p);
  return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch(const Params& p, const CUtensorMap& map, int n_sm, cudaStream_t stream) {
  switch (p.D) {
    case 64: return launch_one<T, 64>(p, map, n_sm, stream);
    case 128: return launch_one<T, 128>(p, map, n_sm, stream);
    case 256: return launch_one<T, 256>(p, map, n_sm, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

bool prefill_path_supported(const Params& p) {
  const int ps = p.page_size;
  if (ps < 8 || (ps & (ps - 1)) != 0) return false;
  return encode_fn_p() != nullptr;
}

cudaError_t launch_prefill(const Params& p, int dtype, int n_sm, cudaStream_t stream) {
  EncodeFn enc = encode_fn_p();
  if (!enc) return cudaErrorNotSupported;
  const uint64_t esz = 2;
  const uint64_t D = p.D, C2 = 2ull * p.Hkv;
  cuuint64_t dims[5] = {64, (cuuint64_t)p.page_size, D / 64, C2, (cuuint64_t)p.num_pages};
  cuuint64_t strides[4] = {C2 * D * esz, 64 * esz, D * esz, (cuuint64_t)p.page_size * C2 * D * esz};
  // one box = PB tokens x 64 elements of one (K|V head, chunk of D): rows of 128 bytes
  cuuint32_t box[5] = {64, (cuuint32_t)p.tma_block_tokens, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMap map;
  const CUtensorMapDataType dt = (dtype == EJK_RPA_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(&map, dt, 5, const_cast<void*>(p.kv), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  if (dtype == EJK_RPA_BF16) return dispatch<__nv_bfloat16>(p, map, n_sm, stream);
  return dispatch<__half>(p, map, n_sm, stream);
}

}  // namespace ejk
