// Split-KV ragged paged attention, TMA variant: the page-table driven gather is issued by one
// producer warp as bulk tensor copies (cp.async.bulk.tensor, one box per KV page block, mbarrier
// tracked), four consumer warps do the math.  Same work items, same shared-memory tile layout and
// the same transposed mma formulation as rpa_splitkv.cu; what changes is who moves the bytes:
//
//   producer warp : pulls work items from a device queue, looks up page ids, issues one 5-D TMA
//                   box {64 elems, PB tokens, D/64, (K_h,V_h), 1 page} per page block of the
//                   64-token stage with SWIZZLE_128B, stages the item's query tile, publishes
//                   per-stage metadata, and runs up to NS stages ahead across item boundaries.
//   consumer warps: wait on the stage's "full" mbarrier, take 16 tokens each, release the stage
//                   through the "empty" mbarrier; at the end of an item they combine through
//                   shared memory and write final rows or a split-KV partial.
//
// Replaces ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:99-159 of the reference
// (page gather + two einsums + online softmax).  No cluster multicast is used anywhere.
//
// Every wait on an mbarrier is bounded in wall time (option "wait_ms"): on expiry the warp raises
// EJK_RPA_ST_TIMEOUT, sets the CTA's abort flag and returns, and every other wait of the CTA
// gives up as soon as it sees the flag, so a protocol error can never hang the device.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "rpa_device.cuh"
#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kConsumerWarps = 4;
constexpr int kThreadsTma = (kConsumerWarps + 1) * 32;
constexpr int kRingTma = 8;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMergeInFlight = 8;      // partials whose loads the last-arriver merge keeps in flight per row
constexpr float kLazyRescale = 8.0f;  // rescale the accumulators only when the max grows by 2^8

struct ItemDesc {
  Unit u;
  int32_t h;
  int32_t pad[3];
};

// KV8: 0 = the cache has the 16-bit dtype of the queries; 1 = e4m3 cache, queries kept at 16 bits (K is widened to
// f16 in registers for Q.K^T); 2 = e4m3 cache and queries quantised to e4m3 as they are staged (q_scale of the v3
// operator).  With an e4m3 cache a stage holds 128 tokens -- the same bytes as 64 tokens at 16 bits -- and every
// consumer warp takes 32 of them, the K extent of one e4m3 mma.
template <int D, int NT, int NS, int KV8 = 0>
struct CfgT {
  static constexpr int ESZ = KV8 ? 1 : 2;                 // bytes per cache element
  static constexpr int TK = KV8 ? 2 * kTileTokens : kTileTokens;
  static constexpr int TW = TK / kConsumerWarps;          // tokens of a stage per consumer warp
  static constexpr int DC = D * ESZ / 128;                // 128-byte columns per token and K or V
  static constexpr int RT = 8 * NT;
  static constexpr int STAGE_BYTES = TK * 2 * D * ESZ;
  static constexpr int Q_ROW_BYTES = (KV8 == 2 ? D : D * 2) + 16;
  static constexpr int Q_BYTES = RT * Q_ROW_BYTES;
  static constexpr int OFF_Q = NS * STAGE_BYTES;
  static constexpr int OFF_OBUF = OFF_Q + NS * Q_BYTES;
  static constexpr int OFF_MBUF = OFF_OBUF + RT * D * 4;
  static constexpr int OFF_LBUF = OFF_MBUF + kConsumerWarps * RT * 4;
  static constexpr int OFF_FBUF = OFF_LBUF + kConsumerWarps * RT * 4;
  static constexpr int OFF_ROWSCALE = OFF_FBUF + kConsumerWarps * RT * 4;
  static constexpr int OFF_ROWM = OFF_ROWSCALE + RT * 4;
  static constexpr int OFF_ROWL = OFF_ROWM + RT * 4;
  static constexpr int OFF_RING = (OFF_ROWL + RT * 4 + 63) / 64 * 64;
  static constexpr int OFF_META = OFF_RING + kRingTma * (int)sizeof(ItemDesc);
  static constexpr int OFF_BAR = OFF_META + NS * 8;        // full[NS], empty[NS], cbar
  static constexpr int OFF_ABORT = OFF_BAR + (2 * NS + 1) * 8;
  static constexpr int SMEM_BYTES = OFF_ABORT + 16 + 1024;  // + alignment slack
  static_assert(DC >= 1, "an e4m3 cache needs head_dim >= 128 (one 128-byte swizzle row per token)");
};

// ---- TMA wrapper (mbarrier helpers live in rpa_device.cuh) ----
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// ---- e4m3 helpers ----
// D(16x8,f32) += A(16x32,row,e4m3) * B(32x8,col,e4m3)
__device__ __forceinline__ void mma_e4m3(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two floats -> two e4m3 (round to nearest even, saturating at +-448) in 16 bits: `lo` in the low byte
__device__ __forceinline__ uint32_t e4m3x2_from_f32(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// two e4m3 (16 bits) -> two f16 (exact): low byte -> low half
__device__ __forceinline__ uint32_t f16x2_from_e4m3x2(uint32_t two) {
  uint32_t r;
  const uint16_t h = (uint16_t)two;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(r) : "h"(h));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
// In an e4m3 kernel the probabilities go to the P.V mma as e4m3 (the reference casts them to the cache dtype,
// ragged_page_attention_v3/_kernel.py:281).  They are exp2(s - m) with a reference m that lags the true
// maximum by at most 2^kLazyRescale, i.e. values up to 2^8 = 256 < 448; a new reference is set kRefBelowMax
// below the maximum it was chosen for, which moves the values into the upper, normal range of e4m3.
constexpr float kRefBelowMax = 4.0f;

template <typename T, int D, int NT, int NS, int KV8>
__global__ void __launch_bounds__(kThreadsTma, (CfgT<D, NT, NS, KV8>::SMEM_BYTES <= 112 * 1024) ? 2 : 1)
rpa_splitkv_tma_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_v,
                       const Params p) {
  using C = CfgT<D, NT, NS, KV8>;
  constexpr int TK = C::TK, RT = C::RT, TW = C::TW;
  constexpr int KT = D / 16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  float* obuf = reinterpret_cast<float*>(smem + C::OFF_OBUF);
  float* mbuf = reinterpret_cast<float*>(smem + C::OFF_MBUF);
  float* lbuf = reinterpret_cast<float*>(smem + C::OFF_LBUF);
  float* row_scale = reinterpret_cast<float*>(smem + C::OFF_ROWSCALE);
  float* row_m = reinterpret_cast<float*>(smem + C::OFF_ROWM);
  float* row_l = reinterpret_cast<float*>(smem + C::OFF_ROWL);
  ItemDesc* ring = reinterpret_cast<ItemDesc*>(smem + C::OFF_RING);
  int2* metas = reinterpret_cast<int2*>(smem + C::OFF_META);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_ABORT);
  const uint32_t bar_full = smem_base + C::OFF_BAR;
  const uint32_t bar_empty = bar_full + NS * 8;
  const uint32_t bar_c = bar_empty + NS * 8;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Hkv = p.Hkv, G = p.G;
  const int pb = p.tma_block_tokens;       // tokens per TMA box (power of two, >= 8)
  const int pb_shift = p.tma_block_shift;
  const unsigned long long wait_ns = (unsigned long long)p.wait_timeout_ms * 1000000ull;
  unsigned flags = 0;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, kConsumerWarps);
    }
    mbar_init(bar_c, kConsumerWarps);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();
  // launched as a programmatic dependent of the planner: everything above overlapped its tail
  if (p.pdl & 2) pdl_wait();
  const int n_work = p.header[kHdrNumUnits] * Hkv;

  if (warp == kConsumerWarps) {
    // =============================== producer warp ===============================
    const int blocks_per_stage = TK >> pb_shift;
    const uint32_t box_bytes = (uint32_t)pb * 2 * D * C::ESZ;
    int s = 0;
    uint32_t empty_parity = 1;  // a fresh barrier passes a wait on parity 1: all stages start empty
    int k = 0;
    int fills = 0;  // stages announced so far
    int wid = 0;
    if (lane == 0) wid = atomicAdd(&p.header[kHdrQueue], 1);
    wid = __shfl_sync(0xffffffffu, wid, 0);
    bool alive = true;
    while (alive) {
      if (wid >= n_work) {
        // end-of-stream marker for the consumers
        if (!mbar_wait(bar_empty + s * 8, empty_parity, abort_flag, wait_ns)) break;
        if (lane == 0) {
          metas[s] = make_int2(-1, 0);
          mbar_arrive(bar_full + s * 8);
        }
        ++fills;
        break;
      }
      const int ui = wid / Hkv;
      const int h = wid - ui * Hkv;
      Unit u;
      {
        const int4* src = reinterpret_cast<const int4*>(p.units + ui);
        const int4 a = __ldg(src), b = __ldg(src + 1), c3 = __ldg(src + 2);
        u.seq = a.x; u.row0 = a.y; u.kv_begin = a.z; u.kv_end = a.w;
        u.slot = b.x; u.q_start = b.y; u.q_len = b.z; u.kv_len = b.w;
        u.merge_idx = c3.x; u.chunk_idx = c3.y; u.n_chunks = c3.z; u.pad = 0;
      }
      const int ring_slot = k % kRingTma;
      int wid_next = 0;
      if (lane == 0) wid_next = atomicAdd(&p.header[kHdrQueue], 1);  // consumed only at the next item
      const int32_t* tab = p.block_tables + (size_t)u.seq * p.pages_per_seq;
      bool first = true;
      for (int pos = u.kv_begin; first || pos < u.kv_end; pos += TK) {
        if (!mbar_wait(bar_empty + s * 8, empty_parity, abort_flag, wait_ns)) {
          alive = false;
          break;
        }
        if (first) {
          // the item's descriptor and query tile travel with its first stage
          if (lane == 0) {
            ItemDesc d;
            d.u = u;
            d.h = h;
            ring[ring_slot] = d;
          }
          constexpr int QCH = D / 8;
          uint8_t* qdst = smem + C::OFF_Q + s * C::Q_BYTES;
          const int rows_total = u.q_len * G;
          for (int cidx = lane; cidx < RT * QCH; cidx += 32) {
            const int r = cidx / QCH, ch = cidx % QCH;
            const int R = u.row0 + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (R < rows_total && ch * 8 < p.Dq) {  // p.Dq < D: a row of queries is narrower than the cache row, the rest is 0
              const int qt = R / G, g = R - qt * G;
              v = __ldg(reinterpret_cast<const uint4*>(
                  reinterpret_cast<const uint8_t*>(p.q) +
                  ((size_t)(u.q_start + qt) * p.Hq + h * G + g) * p.Dq * sizeof(T) + ch * 16));
            }
            if constexpr (KV8 == 2) {
              // queries / q_scale, saturated to the e4m3 range and rounded to e4m3 (_kernel.py:249-254): 8 bytes
              const uint32_t w[4] = {v.x, v.y, v.z, v.w};
              uint32_t o[2];
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                // the reference divides in the queries' dtype first (one rounding to 16 bits), then casts
                float2 a = unpack2<T>(w[2 * i]), b = unpack2<T>(w[2 * i + 1]);
                a = unpack2<T>(Mma<T>::pack(a.x * p.inv_q_scale, a.y * p.inv_q_scale));
                b = unpack2<T>(Mma<T>::pack(b.x * p.inv_q_scale, b.y * p.inv_q_scale));
                o[i] = e4m3x2_from_f32(a.x, a.y) | (e4m3x2_from_f32(b.x, b.y) << 16);
              }
              *reinterpret_cast<uint2*>(qdst + r * C::Q_ROW_BYTES + ch * 8) = make_uint2(o[0], o[1]);
            } else if constexpr (KV8 == 1 && !std::is_same<T, __half>::value) {
              // the e4m3 keys are widened to f16 (exact), so the queries go to f16 too (values beyond +-65504 saturate)
              uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 a = unpack2<T>(w[i]);
                w[i] = Mma<__half>::pack(fminf(fmaxf(a.x, -65504.f), 65504.f), fminf(fmaxf(a.y, -65504.f), 65504.f));
              }
              *reinterpret_cast<uint4*>(qdst + r * C::Q_ROW_BYTES + ch * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
              if (KV8 == 0 && p.inv_q_scale != 0.f) {
                // 16-bit cache with q_scale: queries / q_scale, clipped to the finite range of the cache dtype and
                // rounded to it (_kernel.py:249-254); the logits are multiplied back through softmax_scale
                constexpr float kMaxT = std::is_same<T, __half>::value ? 65504.f : 3.3895313892515355e38f;
                uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 a = unpack2<T>(w[i]);
                  w[i] = Mma<T>::pack(fminf(fmaxf(a.x * p.inv_q_scale, -kMaxT), kMaxT),
                                      fminf(fmaxf(a.y * p.inv_q_scale, -kMaxT), kMaxT));
                }
                v = make_uint4(w[0], w[1], w[2], w[3]);
              }
              *reinterpret_cast<uint4*>(qdst + r * C::Q_ROW_BYTES + ch * 16) = v;
            }
          }
        }
        int nblk = (u.kv_end - pos + pb - 1) >> pb_shift;
        if (nblk > blocks_per_stage) nblk = blocks_per_stage;
        if (nblk < 0) nblk = 0;
        __syncwarp();
        // test hook: the stage is never announced, the consumers' wait for it must run out
        const bool withhold = (p.test_withhold & 1) && wid == 0 && first;
        ++fills;
        if (withhold) nblk = 0;
        if (lane == 0 && !withhold) {
          metas[s] = make_int2(ring_slot, pos);
          if (nblk > 0) mbar_arrive_expect_tx(bar_full + s * 8, (uint32_t)nblk * box_bytes);
          else mbar_arrive(bar_full + s * 8);
        }
        __syncwarp();
        if (lane < nblk) {
          const int key = pos + (lane << pb_shift);
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
          const uint32_t dst = smem_base + s * C::STAGE_BYTES + lane * box_bytes;
          if (p.v_cache == nullptr) {
            tma_load_5d(dst, &tmap, bar_full + s * 8, 0, off, 0, 2 * h, page);
          } else {
            // separate caches [P, Hkv, page, D]: one box each for K and V, landing where the
            // interleaved box would have put them ([K|V][D/64][PB tokens][64])
            tma_load_5d(dst, &tmap, bar_full + s * 8, 0, off, 0, h, page);
            tma_load_5d(dst + box_bytes / 2, &tmap_v, bar_full + s * 8, 0, off, 0, h, page);
          }
        }
        first = false;
        if (++s == NS) {
          s = 0;
          empty_parity ^= 1u;
        }
      }
      ++k;
      wid = __shfl_sync(0xffffffffu, wid_next, 0);
    }
    // Leave only after every bulk copy this warp issued has landed: wait (bounded) for the
    // consumers to drain all stages, which implies all "full" phases completed.
    for (int i = 0; i < NS; ++i) {
      if (!mbar_wait(bar_empty + s * 8, empty_parity, abort_flag, wait_ns)) break;
      if (++s == NS) {
        s = 0;
        empty_parity ^= 1u;
      }
    }
    if (*abort_flag) {
      // Giving up: the consumers no longer release stages, so wait (bounded, 2 ms per stage) for the
      // copies themselves -- the "full" phase of each of the last NS announced stages -- before this
      // CTA's shared memory can go to another CTA.
      flags |= EJK_RPA_ST_TIMEOUT;
      for (int i = 1; i <= NS && i <= fills; ++i) {
        const int f = fills - i;
        mbar_wait_quiet(bar_full + (f % NS) * 8, (uint32_t)((f / NS) & 1), 2000000ull);
      }
    }
  } else {
    // =============================== consumer warps ===============================
    // per-thread shared-memory offsets of the ldmatrix rows (constant for the whole kernel)
    const uint32_t swz = (uint32_t)(lane & 7) << 4;
    const uint32_t dc_stride = (uint32_t)pb * 128;
    // token tl of the stage sits in box tl / pb at row tl % pb; a box is [K|V][DC columns][pb rows][128 bytes]
    auto row_off = [&](int tl, int kv) {
      const int j = tl >> pb_shift, tp = tl & (pb - 1);
      return (uint32_t)((j * 2 + kv) * C::DC) * dc_stride + (uint32_t)tp * 128;
    };
    uint32_t k_off, v_off, k_off1 = 0;
    if constexpr (KV8 == 0) {
      k_off = row_off(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 0);  // K: second matrix = tokens 8..15
      v_off = row_off(warp * 16 + (lane & 7) + (lane >> 4) * 8, 1);        // V: third/fourth matrix = tokens 8..15
    } else {
      // K: two 16-token blocks, in each the matrices (tokens 0-7 | 8-15) x (16-byte chunk c | c + 1);
      // V: four transposed matrices of one chunk, tokens 8j .. 8j+7
      k_off = row_off(warp * TW + (lane & 7) + ((lane >> 3) & 1) * 8, 0);
      k_off1 = row_off(warp * TW + 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 0);
      v_off = row_off(warp * TW + (lane & 7) + (lane >> 3) * 8, 1);
    }
    const int k_dhalf = lane >> 4, v_dhalf = (lane >> 3) & 1;

    // query fragments (B operands of Q.K^T), per 8-row tile and k step:
    //   16-bit cache: D/16 steps x 2 registers; e4m3 queries: D/32 steps x 2; f16 queries against e4m3 keys:
    //   D/32 steps x 4 (two f16 mmas per 32-byte chunk of K)
    constexpr int QK_STEPS = KV8 ? D / 32 : D / 16;
    constexpr int QREGS = KV8 == 1 ? 4 : 2;
    uint32_t qf[NT][QK_STEPS][QREGS];
    float acc[NT][KT][4];
    float m_run[NT][2], l_run[NT][2];
    int pos_r[NT][2], lo_r[NT][2];
    int pos_min = 0, lo_max = 0;
    int s = 0;
    uint32_t full_parity = 0, c_parity = 0;

    auto consumer_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_c);
      const bool ok = mbar_wait(bar_c, c_parity, abort_flag, wait_ns);
      c_parity ^= 1u;
      return ok;
    };

    while (true) {
      if (!mbar_wait(bar_full + s * 8, full_parity, abort_flag, wait_ns)) break;
      const int2 meta = metas[s];
      if (meta.x < 0) break;
      const ItemDesc& it = ring[meta.x];
      const Unit u = it.u;
      const int h = it.h;
      const int pos = meta.y;
      const uint32_t sbase = smem_base + s * C::STAGE_BYTES;
      const int rows_total = u.q_len * G;
      int n_rows = rows_total - u.row0;
      if (n_rows > RT) n_rows = RT;

      if (pos == u.kv_begin) {
        const uint8_t* qs = smem + C::OFF_Q + s * C::Q_BYTES;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if constexpr (KV8 == 1) {
            // f16 queries: elements 32kt + 4t .. +3 (first mma of the chunk) and 32kt + 16 + 4t .. +3 (second)
            const uint8_t* qrow = qs + (nt * 8 + (lane >> 2)) * C::Q_ROW_BYTES + (lane & 3) * 8;
#pragma unroll
            for (int kt = 0; kt < QK_STEPS; ++kt) {
              const uint2 a = *reinterpret_cast<const uint2*>(qrow + kt * 64);
              const uint2 b = *reinterpret_cast<const uint2*>(qrow + kt * 64 + 32);
              qf[nt][kt][0] = a.x;
              qf[nt][kt][1] = a.y;
              qf[nt][kt][2] = b.x;
              qf[nt][kt][3] = b.y;
            }
          } else {
            // 16-bit: elements 16kt + 2t, +1 and 16kt + 8 + 2t, +1; e4m3: bytes 32kt + 4t .. +3 and 32kt + 16 + 4t .. +3
            const uint8_t* qrow = qs + (nt * 8 + (lane >> 2)) * C::Q_ROW_BYTES + (lane & 3) * 4;
#pragma unroll
            for (int kt = 0; kt < QK_STEPS; ++kt) {
              qf[nt][kt][0] = *reinterpret_cast<const uint32_t*>(qrow + kt * 32);
              qf[nt][kt][1] = *reinterpret_cast<const uint32_t*>(qrow + kt * 32 + 16);
            }
          }
        }
        const int base = u.kv_len - u.q_len;
        pos_min = base + u.row0 / G;
        lo_max = (p.window > 0) ? (base + (u.row0 + n_rows - 1) / G - p.window) : -1;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int R = u.row0 + nt * 8 + (lane & 3) * 2 + j;
            const int ps = (R < rows_total) ? base + R / G : -1;
            pos_r[nt][j] = ps;
            lo_r[nt][j] = (p.window > 0) ? ps - p.window : -1;
            m_run[nt][j] = -INFINITY;
            l_run[nt][j] = 0.f;
          }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int kt = 0; kt < KT; ++kt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][kt][e] = 0.f;
      }

      if constexpr (KV8 == 0) {
        const int key0 = pos + warp * 16;
        if (key0 < u.kv_end) {
          float sc[NT][4];
  #pragma unroll
          for (int nt = 0; nt < NT; ++nt)
  #pragma unroll
            for (int e = 0; e < 4; ++e) sc[nt][e] = 0.f;
  #pragma unroll
          for (int kt = 0; kt < KT; ++kt) {
            const int d16 = kt * 2;  // + k_dhalf at run time; both fold into one XOR below
            uint32_t a[4];
            ldmatrix_x4(a, sbase + k_off + (uint32_t)(d16 >> 3) * dc_stride +
                               ((((uint32_t)(d16 & 7) | (uint32_t)k_dhalf) << 4) ^ swz));
  #pragma unroll
            for (int nt = 0; nt < NT; ++nt) Mma<T>::run(sc[nt], a, qf[nt][kt][0], qf[nt][kt][1]);
          }
          const bool tail = key0 + 16 > u.kv_end;  // tokens past the chunk end: stale or unowned bytes
          const bool need_mask = tail || (key0 + 15 > pos_min) || (key0 <= lo_max);
          uint32_t pbf[NT][2];
          bool grow = false;
          float mx[NT][2];
  #pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
  #pragma unroll
            for (int e = 0; e < 4; ++e) {
              float x = sc[nt][e];
              if (p.cap != 0.f) x = p.cap_log2 * soft_cap_tanh(x * p.inv_cap_scale);
              else x *= p.scale_log2;
              if (need_mask) {
                const int key = key0 + (lane >> 2) + (e >> 1) * 8;
                const int j = e & 1;
                if (key > pos_r[nt][j] || key <= lo_r[nt][j]) x = -INFINITY;
              }
              sc[nt][e] = x;
            }
  #pragma unroll
            for (int j = 0; j < 2; ++j) {
              float v = fmaxf(sc[nt][j], sc[nt][j + 2]);
              v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
              v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
              v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
              mx[nt][j] = v;
              // lazy rescaling: keep the old reference maximum unless the new one is 2^8 larger
              grow |= (v > m_run[nt][j] + kLazyRescale) || (m_run[nt][j] == -INFINITY && v > -INFINITY);
            }
          }
          if (__any_sync(0xffffffffu, grow)) {
  #pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              float alpha[2];
  #pragma unroll
              for (int j = 0; j < 2; ++j) {
                const bool g = (mx[nt][j] > m_run[nt][j] + kLazyRescale) || (m_run[nt][j] == -INFINITY && mx[nt][j] > -INFINITY);
                const float m_new = g ? mx[nt][j] : m_run[nt][j];
                alpha[j] = g ? fast_exp2(m_run[nt][j] - m_new) : 1.f;  // exp2(-inf) = 0 on the first tile
                m_run[nt][j] = m_new;
                l_run[nt][j] *= alpha[j];
              }
  #pragma unroll
              for (int kt = 0; kt < KT; ++kt) {
                acc[nt][kt][0] *= alpha[0];
                acc[nt][kt][1] *= alpha[1];
                acc[nt][kt][2] *= alpha[0];
                acc[nt][kt][3] *= alpha[1];
              }
            }
          }
  #pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
  #pragma unroll
            for (int j = 0; j < 2; ++j) {
              const float m_use = (m_run[nt][j] == -INFINITY) ? 0.f : m_run[nt][j];
              const float p0 = fast_exp2(sc[nt][j] - m_use);
              const float p1 = fast_exp2(sc[nt][j + 2] - m_use);
              sc[nt][j] = p0;
              sc[nt][j + 2] = p1;
              l_run[nt][j] += p0 + p1;
            }
            pbf[nt][0] = movmatrix_trans(Mma<T>::pack(sc[nt][0], sc[nt][1]));
            pbf[nt][1] = movmatrix_trans(Mma<T>::pack(sc[nt][2], sc[nt][3]));
          }
          // V^T fragments; in a tail tile the registers of tokens >= kv_end are cleared so that
          // 0 * (stale NaN) can never reach the accumulators
          uint32_t vmask_lo = 0xffffffffu, vmask_hi = 0xffffffffu;
          if (tail) {
            const int t0 = key0 + (lane & 3) * 2;
            vmask_lo = (t0 < u.kv_end ? 0x0000ffffu : 0u) | (t0 + 1 < u.kv_end ? 0xffff0000u : 0u);
            vmask_hi = (t0 + 8 < u.kv_end ? 0x0000ffffu : 0u) | (t0 + 9 < u.kv_end ? 0xffff0000u : 0u);
          }
  #pragma unroll
          for (int mt = 0; mt < KT; ++mt) {
            const int d16 = mt * 2;
            uint32_t a[4];
            ldmatrix_x4_trans(a, sbase + v_off + (uint32_t)(d16 >> 3) * dc_stride +
                                     ((((uint32_t)(d16 & 7) | (uint32_t)v_dhalf) << 4) ^ swz));
            if (tail) {
              a[0] &= vmask_lo;
              a[1] &= vmask_lo;
              a[2] &= vmask_hi;
              a[3] &= vmask_hi;
            }
  #pragma unroll
            for (int nt = 0; nt < NT; ++nt) Mma<T>::run(acc[nt][mt], a, pbf[nt][0], pbf[nt][1]);
          }
        }
      } else {
        // ---------------- e4m3 cache: this warp's 32 tokens of the stage ----------------
        const int key0 = pos + warp * TW;
        if (key0 < u.kv_end) {
          // S^T[32 tokens x 8 rows] = K . Q^T as two 16-token blocks
          float sc[NT][2][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
              for (int e = 0; e < 4; ++e) sc[nt][b][e] = 0.f;
#pragma unroll
          for (int kt = 0; kt < QK_STEPS; ++kt) {
            const int c16 = kt * 2;  // 16-byte chunk of the token row; + k_dhalf at run time
            const uint32_t coff = (uint32_t)(c16 >> 3) * dc_stride + ((((uint32_t)(c16 & 7) | (uint32_t)k_dhalf) << 4) ^ swz);
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              // a[0] = (token g, bytes 4t..4t+3 of the chunk), a[1] = token g+8, a[2] / a[3] = the next chunk
              uint32_t a[4];
              ldmatrix_x4(a, sbase + (b ? k_off1 : k_off) + coff);
              if constexpr (KV8 == 2) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_e4m3(sc[nt][b], a, qf[nt][kt][0], qf[nt][kt][1]);
              } else {
                // widen to f16: the low two bytes of a register become k slots 2t, 2t+1, the high two k slots
                // 8+2t, 8+2t+1 of one f16 mma -- the query fragments were loaded in the same order
                const uint32_t l0 = f16x2_from_e4m3x2(a[0]), h0 = f16x2_from_e4m3x2(a[0] >> 16);
                const uint32_t l1 = f16x2_from_e4m3x2(a[1]), h1 = f16x2_from_e4m3x2(a[1] >> 16);
                const uint32_t l2 = f16x2_from_e4m3x2(a[2]), h2 = f16x2_from_e4m3x2(a[2] >> 16);
                const uint32_t l3 = f16x2_from_e4m3x2(a[3]), h3 = f16x2_from_e4m3x2(a[3] >> 16);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                  mma_f16(sc[nt][b], l0, l1, h0, h1, qf[nt][kt][0], qf[nt][kt][1]);
                  mma_f16(sc[nt][b], l2, l3, h2, h3, qf[nt][kt][2], qf[nt][kt][3]);
                }
              }
            }
          }
          const bool tail = key0 + TW > u.kv_end;  // tokens past the chunk end: stale or unowned bytes
          const bool need_mask = tail || (key0 + TW - 1 > pos_min) || (key0 <= lo_max);
          bool grow = false;
          float mx[NT][2];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float x = sc[nt][b][e];
                if (p.cap != 0.f) x = p.cap_log2 * soft_cap_tanh(x * p.inv_cap_scale);
                else x *= p.scale_log2;
                if (need_mask) {
                  // a 128-token stage can straddle the end of a chunk (chunks are cut at multiples of 64): keys from
                  // kv_end on belong to the next chunk, or to nobody
                  const int key = key0 + b * 16 + (lane >> 2) + (e >> 1) * 8;
                  const int j = e & 1;
                  if (key > pos_r[nt][j] || key <= lo_r[nt][j] || key >= u.kv_end) x = -INFINITY;
                }
                sc[nt][b][e] = x;
              }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              float v = fmaxf(fmaxf(sc[nt][0][j], sc[nt][0][j + 2]), fmaxf(sc[nt][1][j], sc[nt][1][j + 2]));
              v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
              v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
              v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
              mx[nt][j] = v;
              // the reference sits kRefBelowMax below the maximum it was chosen for and is kept until the
              // maximum has grown 2^8 beyond it, so exp2(s - m) never exceeds 256 (e4m3 holds 448)
              grow |= (v > m_run[nt][j] + kLazyRescale) || (m_run[nt][j] == -INFINITY && v > -INFINITY);
            }
          }
          if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              float alpha[2];
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const bool g = (mx[nt][j] > m_run[nt][j] + kLazyRescale) || (m_run[nt][j] == -INFINITY && mx[nt][j] > -INFINITY);
                const float m_new = g ? mx[nt][j] - kRefBelowMax : m_run[nt][j];
                alpha[j] = g ? fast_exp2(m_run[nt][j] - m_new) : 1.f;  // exp2(-inf) = 0 on the first tile
                m_run[nt][j] = m_new;
                l_run[nt][j] *= alpha[j];
              }
#pragma unroll
              for (int mt = 0; mt < KT; ++mt) {
                acc[nt][mt][0] *= alpha[0];
                acc[nt][mt][1] *= alpha[1];
                acc[nt][mt][2] *= alpha[0];
                acc[nt][mt][3] *= alpha[1];
              }
            }
          }
          // probabilities -> e4m3, transposed into the B fragments of P.V: after the transpose the four bytes of
          // pb[nt][b] belong to query row g and tokens 16b + {2t, 2t+8, 2t+1, 2t+9}
          uint32_t pb8[NT][2];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const float m_use = (m_run[nt][j] == -INFINITY) ? 0.f : m_run[nt][j];
                const float p0 = fast_exp2(sc[nt][b][j] - m_use);
                const float p1 = fast_exp2(sc[nt][b][j + 2] - m_use);
                sc[nt][b][j] = p0;
                sc[nt][b][j + 2] = p1;
                l_run[nt][j] += p0 + p1;
              }
              // element (token g, row 2t) pairs with (token g+8, row 2t) in the low half, rows 2t+1 in the high half
              const uint32_t w = e4m3x2_from_f32(sc[nt][b][0], sc[nt][b][2]) | (e4m3x2_from_f32(sc[nt][b][1], sc[nt][b][3]) << 16);
              pb8[nt][b] = movmatrix_trans(w);
            }
          }
          // V^T fragments: four transposed 8-token matrices of one 16-byte chunk; register j holds, for the
          // two head-dim lanes 2g and 2g+1, tokens 8j + 2t (low half) and 8j + 2t + 1 (high half).  In a tail
          // tile the bytes of tokens >= kv_end are cleared, so that 0 * (stale NaN) cannot reach the accumulators.
          uint32_t vmask[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
          if (tail) {
            const int t0 = key0 + (lane & 3) * 2;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              vmask[j] = (t0 + 8 * j < u.kv_end ? 0x0000ffffu : 0u) | (t0 + 8 * j + 1 < u.kv_end ? 0xffff0000u : 0u);
          }
#pragma unroll
          for (int mt = 0; mt < KT; ++mt) {
            uint32_t r[4];
            ldmatrix_x4_trans(r, sbase + v_off + (uint32_t)(mt >> 3) * dc_stride + (((uint32_t)(mt & 7) << 4) ^ swz));
            if (tail) {
#pragma unroll
              for (int j = 0; j < 4; ++j) r[j] &= vmask[j];
            }
            // rows of the mma: g <-> head-dim lane 16mt + 2g, g+8 <-> lane 16mt + 2g + 1; k slots in the token
            // order of pb8
            uint32_t a[4];
            a[0] = prmt(r[0], r[1], 0x6240u);
            a[1] = prmt(r[0], r[1], 0x7351u);
            a[2] = prmt(r[2], r[3], 0x6240u);
            a[3] = prmt(r[2], r[3], 0x7351u);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma_e4m3(acc[nt][mt], a, pb8[nt][0], pb8[nt][1]);
          }
        }
      }
      // this warp is done with the stage's bytes (query fragments are in registers by now)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + s * 8);

      if (pos + TK >= u.kv_end) {
        // ---- end of item: combine the four warps ----
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            float l = l_run[nt][j];
            l += __shfl_xor_sync(0xffffffffu, l, 4);
            l += __shfl_xor_sync(0xffffffffu, l, 8);
            l += __shfl_xor_sync(0xffffffffu, l, 16);
            if (lane < 4) {
              const int r = nt * 8 + lane * 2 + j;
              mbuf[warp * RT + r] = m_run[nt][j];
              lbuf[warp * RT + r] = l;
            }
          }
        if (!consumer_sync()) break;
        // Every lane derives the rescale factors of its own rows from the four (m, l) pairs; the
        // accumulators are then added into obuf in four rounds, warp w handling the d-slice
        // (w + round) % 4, so each address receives its four contributions in a fixed order and
        // the result does not depend on warp timing (no floating-point atomics).
        float f_own[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int r = nt * 8 + (lane & 3) * 2 + j;
            float mt = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) mt = fmaxf(mt, mbuf[w * RT + r]);
            const float mu = (mt == -INFINITY) ? 0.f : mt;
            f_own[nt][j] = fast_exp2(m_run[nt][j] - mu);
          }
        if (tid < RT) {
          const int r = tid;
          float mt = -INFINITY;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) mt = fmaxf(mt, mbuf[w * RT + r]);
          const float mu = (mt == -INFINITY) ? 0.f : mt;
          float lt = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) lt += lbuf[w * RT + r] * fast_exp2(mbuf[w * RT + r] - mu);
          float scl = 1.f;
          if (u.slot < 0) {
            float l_fin = lt;
            if (p.num_sinks > 0 && r < n_rows) {
              // attention sinks join the denominator only (_xla_impl_fwd.py:161-172)
              const int R = u.row0 + r;
              const int hq = h * G + (R % G);
              const int srow = (p.sink_rows == p.Hq) ? hq : (p.sink_rows == Hkv ? h : 0);
              const float* sk = p.sinks + (size_t)srow * p.num_sinks;
              float sm = -INFINITY;
              for (int i = 0; i < p.num_sinks; ++i) sm = fmaxf(sm, sk[i] * kLog2e);
              const float m_fin = fmaxf(mt, sm);
              const float mf = (m_fin == -INFINITY) ? 0.f : m_fin;
              scl = fast_exp2(mt - mf);
              l_fin = lt * scl;
              for (int i = 0; i < p.num_sinks; ++i) l_fin += fast_exp2(sk[i] * kLog2e - mf);
            }
            scl = (l_fin > 0.f) ? scl * p.out_scale / l_fin : 0.f;  // out_scale: v_scale of the v3 operator, else 1
          }
          row_scale[r] = scl;
          row_m[r] = mt;
          row_l[r] = lt;
        }
        bool alive_c = true;
#pragma unroll
        for (int round = 0; round < kConsumerWarps; ++round) {
          const int slice = (warp + round) % kConsumerWarps;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const int r0 = nt * 8 + (lane & 3) * 2;
            const float f0 = f_own[nt][0], f1 = f_own[nt][1];
#pragma unroll
            for (int mi = 0; mi < KT / kConsumerWarps; ++mi) {
              // compile-time accumulator index in every branch keeps acc[] in registers
#pragma unroll
              for (int sl = 0; sl < kConsumerWarps; ++sl) {
                if (sl == slice) {
                  const int mt = sl * (KT / kConsumerWarps) + mi;
                  // accumulator rows g / g+8 of block mt are head-dim lanes 16mt + g / + 8, or, in the e4m3
                  // kernels (see the V fragments), 16mt + 2g / + 1
                  constexpr int HI = KV8 ? 1 : 8;
                  const int d = mt * 16 + (lane >> 2) * (KV8 ? 2 : 1);
                  float* o0 = &obuf[r0 * D + d];
                  float* o1 = &obuf[(r0 + 1) * D + d];
                  if (round == 0) {
                    o0[0] = acc[nt][mt][0] * f0;
                    o0[HI] = acc[nt][mt][2] * f0;
                    o1[0] = acc[nt][mt][1] * f1;
                    o1[HI] = acc[nt][mt][3] * f1;
                  } else {
                    o0[0] += acc[nt][mt][0] * f0;
                    o0[HI] += acc[nt][mt][2] * f0;
                    o1[0] += acc[nt][mt][1] * f1;
                    o1[HI] += acc[nt][mt][3] * f1;
                  }
                }
              }
            }
          }
          if (!consumer_sync()) {
            alive_c = false;
            break;
          }
        }
        if (!alive_c) break;
        constexpr int kCT = kConsumerWarps * 32;
        if (u.slot < 0) {
          T* out = reinterpret_cast<T*>(p.out);
          for (int i = tid; i < n_rows * (D / 2); i += kCT) {
            const int r = i / (D / 2), d = (i % (D / 2)) * 2;
            const int R = u.row0 + r;
            const int qt = R / G, g = R - qt * G;
            const float scl = row_scale[r];
            const float2 v = *reinterpret_cast<float2*>(&obuf[r * D + d]);
            if (d < p.Dq)
              *reinterpret_cast<uint32_t*>(out + ((size_t)(u.q_start + qt) * p.Hq + h * G + g) * p.Dq + d) =
                  Mma<T>::pack(v.x * scl, v.y * scl);
          }
        } else {
          float* po = p.part_o + ((size_t)u.slot * Hkv + h) * RT * D;
          float2* pml = p.part_ml + ((size_t)u.slot * Hkv + h) * RT;
          for (int i = tid; i < n_rows * (D / 4); i += kCT) {
            const int r = i / (D / 4), d = (i % (D / 4)) * 4;
            const float4 v = *reinterpret_cast<float4*>(&obuf[r * D + d]);
            *reinterpret_cast<float4*>(po + r * D + d) = v;
          }
          if (tid < n_rows) pml[tid] = make_float2(row_m[tid], row_l[tid]);
          if (p.fused_merge) {
            // Last-arriver merge: publish this chunk's partial, take a ticket for (tile, kv head); the
            // chunk that draws the last ticket combines all of them, in chunk order, so the result
            // does not depend on which chunk finished last.  No CTA ever waits for another.
            __threadfence();
            if (!consumer_sync()) break;
            if (tid == 0) {
              const int old = atomicAdd(&p.tickets[(size_t)u.merge_idx * Hkv + h], 1);
              row_l[0] = (old == u.n_chunks - 1) ? 1.f : 0.f;  // row_l/row_m were consumed above
            }
            if (!consumer_sync()) break;
            const bool last = row_l[0] != 0.f;
            if (last) {
              __threadfence();
              constexpr int VPL = D / 32;
              const int slot0 = u.slot - u.chunk_idx;
              T* out = reinterpret_cast<T*>(p.out);
              for (int r = warp; r < n_rows; r += kConsumerWarps) {
                float m_tot = -INFINITY;
                for (int c = lane; c < u.n_chunks; c += 32)
                  m_tot = fmaxf(m_tot, __ldcg(&p.part_ml[((size_t)(slot0 + c) * Hkv + h) * RT + r]).x);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m_tot = fmaxf(m_tot, __shfl_xor_sync(0xffffffffu, m_tot, o));
                const float mu = (m_tot == -INFINITY) ? 0.f : m_tot;
                float accm[VPL];
#pragma unroll
                for (int i = 0; i < VPL; ++i) accm[i] = 0.f;
                float l_tot = 0.f;
                // kMergeInFlight chunks' loads in flight at a time (each is an L2 round trip); the sums still run in
                // chunk order
                for (int c0 = 0; c0 < u.n_chunks; c0 += kMergeInFlight) {
                  float2 ml[kMergeInFlight];
                  float vv[kMergeInFlight][VPL];
#pragma unroll
                  for (int j = 0; j < kMergeInFlight; ++j) {
                    const int c = min(c0 + j, u.n_chunks - 1);
                    const size_t base = ((size_t)(slot0 + c) * Hkv + h) * RT + r;
                    ml[j] = __ldcg(&p.part_ml[base]);
                    const float* src = p.part_o + base * D + lane * VPL;
                    if constexpr (VPL == 2) {
                      const float2 v = __ldcg(reinterpret_cast<const float2*>(src));
                      vv[j][0] = v.x;
                      vv[j][1] = v.y;
                    } else {
#pragma unroll
                      for (int i = 0; i < VPL; i += 4) {
                        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + i));
                        vv[j][i] = v.x;
                        vv[j][i + 1] = v.y;
                        vv[j][i + 2] = v.z;
                        vv[j][i + 3] = v.w;
                      }
                    }
                  }
#pragma unroll
                  for (int j = 0; j < kMergeInFlight; ++j) {
                    if (c0 + j < u.n_chunks) {
                      const float f = fast_exp2(ml[j].x - mu);
                      l_tot += ml[j].y * f;
#pragma unroll
                      for (int i = 0; i < VPL; ++i) accm[i] += vv[j][i] * f;
                    }
                  }
                }
                const int R = u.row0 + r;
                const int qt = R / G, g = R - qt * G;
                const int hq = h * G + g;
                float scl = 1.f, l_fin = l_tot;
                if (p.num_sinks > 0) {
                  const int srow = (p.sink_rows == p.Hq) ? hq : (p.sink_rows == Hkv ? h : 0);
                  const float* sk = p.sinks + (size_t)srow * p.num_sinks;
                  float sm = -INFINITY;
                  for (int i = 0; i < p.num_sinks; ++i) sm = fmaxf(sm, sk[i] * kLog2e);
                  const float m_fin = fmaxf(m_tot, sm);
                  const float mf = (m_fin == -INFINITY) ? 0.f : m_fin;
                  scl = fast_exp2(m_tot - mf);
                  l_fin = l_tot * scl;
                  for (int i = 0; i < p.num_sinks; ++i) l_fin += fast_exp2(sk[i] * kLog2e - mf);
                }
                scl = (l_fin > 0.f) ? scl * p.out_scale / l_fin : 0.f;  // out_scale: v_scale of the v3 operator, else 1
                T* dst = out + ((size_t)(u.q_start + qt) * p.Hq + hq) * p.Dq + lane * VPL;
                if (lane * VPL < p.Dq) {
#pragma unroll
                  for (int i = 0; i < VPL; i += 2)
                    *reinterpret_cast<uint32_t*>(dst + i) = Mma<T>::pack(accm[i] * scl, accm[i + 1] * scl);
                }
              }
            }
          }
        }
        // The next item's writes to mbuf/lbuf come before its first consumer_sync, but they only
        // race with readers of mbuf/lbuf, and those finished before the first combine step's sync above; its
        // writes to obuf/row_* come after its first consumer_sync, which every warp reaches only
        // after finishing the loops above.
      }
      if (++s == NS) {
        s = 0;
        full_parity ^= 1u;
      }
    }
    if (*abort_flag) flags |= EJK_RPA_ST_TIMEOUT;
  }
  if (flags && p.status) atomicOr(reinterpret_cast<unsigned*>(p.status), flags);
  zero_tail_rows(p.out, p.header[kHdrTailStart], p.T, (size_t)p.Hq * p.Dq * sizeof(T));
  // In a mixed batch this grid is a programmatic dependent of the prefill-tile grid and never waited for it
  // (the two write different rows).  Whatever follows in the stream, though, is only ordered after THIS grid:
  // one thread per CTA now waits for the prefill grid, so this grid cannot complete before it, and a later
  // kernel (a reader of `out`, the next call's planner) is ordered after both.  All prefill CTAs are resident
  // before this grid starts (it is released when each of them has seen the plan), so the wait cannot starve them.
  if ((p.pdl & 1) && tid == 0) pdl_wait();
}

// ---- host side: tensor map over kv_pages ----
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
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

template <typename T, int D, int NT, int NS, int KV8>
cudaError_t launch_one(const Params& p, const CUtensorMap& map, const CUtensorMap& map_v, int n_sm, cudaStream_t stream, bool pdl) {
  using C = CfgT<D, NT, NS, KV8>;
  auto kern = rpa_splitkv_tma_kernel<T, D, NT, NS, KV8>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int per_sm = (C::SMEM_BYTES <= 112 * 1024) ? 2 : 1;
  return launch_kernel(kern, dim3(n_sm * per_sm), dim3(kThreadsTma), C::SMEM_BYTES, stream, pdl, map, map_v, p);
}

template <typename T, int KV8>
cudaError_t dispatch(const Params& p, const CUtensorMap& map, const CUtensorMap& map_v, int n_sm, cudaStream_t stream, bool pdl) {
  const bool wide = p.rows_per_tile == 16;
  if constexpr (KV8 == 0) {
    switch (p.D) {
      case 64:
        return wide ? launch_one<T, 64, 2, 4, 0>(p, map, map_v, n_sm, stream, pdl) : launch_one<T, 64, 1, 4, 0>(p, map, map_v, n_sm, stream, pdl);
      case 128:
        return wide ? launch_one<T, 128, 2, 3, 0>(p, map, map_v, n_sm, stream, pdl) : launch_one<T, 128, 1, 3, 0>(p, map, map_v, n_sm, stream, pdl);
      case 256:
        return wide ? launch_one<T, 256, 2, 2, 0>(p, map, map_v, n_sm, stream, pdl) : launch_one<T, 256, 1, 3, 0>(p, map, map_v, n_sm, stream, pdl);
    }
  } else {
    // an e4m3 stage of 128 tokens has the bytes of a 16-bit stage of 64 tokens: same stage counts
    switch (p.D) {
      case 128:
        return wide ? launch_one<T, 128, 2, 3, KV8>(p, map, map_v, n_sm, stream, pdl) : launch_one<T, 128, 1, 3, KV8>(p, map, map_v, n_sm, stream, pdl);
      case 256:
        return wide ? launch_one<T, 256, 2, 2, KV8>(p, map, map_v, n_sm, stream, pdl) : launch_one<T, 256, 1, 3, KV8>(p, map, map_v, n_sm, stream, pdl);
    }
  }
  return cudaErrorInvalidValue;
}

}  // namespace

bool tma_path_supported(const Params& p) {
  const int ps = p.page_size;
  if (ps < 8 || ps % 8 != 0) return false;  // boxes are whole 8-token (1024-byte) swizzle atoms inside one page
  return encode_fn() != nullptr;
}

cudaError_t launch_splitkv_tma(const Params& p, int dtype, int n_sm, cudaStream_t stream, bool pdl) {
  EncodeFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  // elements of the innermost dimension: one 128-byte swizzle row = 64 16-bit or 128 e4m3 values
  const bool kv8 = p.kv8 != 0;
  const uint64_t esz = kv8 ? 1 : 2, inner = 128 / esz;
  const uint64_t D = p.D, Dkv = p.Dkv, C2 = (uint64_t)p.C2;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = kv8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                     : (dtype == EJK_RPA_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap map, map_v;
  if (p.v_cache == nullptr) {
    // dims, innermost first: one swizzle row of elements | token in page | column of D | combined head | page
    cuuint64_t dims[5] = {inner, (cuuint64_t)p.page_size, D / inner, C2, (cuuint64_t)p.num_pages};
    cuuint64_t strides[4] = {C2 * Dkv * esz, inner * esz, Dkv * esz, (cuuint64_t)p.page_size * C2 * Dkv * esz};
    cuuint32_t box[5] = {(cuuint32_t)inner, (cuuint32_t)p.tma_block_tokens, (cuuint32_t)(D / inner), 2, 1};
    CUresult r = enc(&map, dt, 5, const_cast<void*>(p.kv), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    map_v = map;
  } else {
    if (kv8) return cudaErrorInvalidValue;  // separate key / value caches: 16-bit only
    // key_cache / value_cache [P, Hkv, page, D]: 64 elements | token in page | chunk of D | kv head | page
    cuuint64_t dims[5] = {64, (cuuint64_t)p.page_size, D / 64, (cuuint64_t)p.Hkv, (cuuint64_t)p.num_pages};
    cuuint64_t strides[4] = {D * esz, 64 * esz, (cuuint64_t)p.page_size * D * esz,
                             (cuuint64_t)p.Hkv * p.page_size * D * esz};
    cuuint32_t box[5] = {64, (cuuint32_t)p.tma_block_tokens, (cuuint32_t)(D / 64), 1, 1};
    CUresult r = enc(&map, dt, 5, const_cast<void*>(p.kv), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    r = enc(&map_v, dt, 5, const_cast<void*>(p.v_cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  }
  if (kv8) {
    // queries quantised to e4m3 (q_scale given) or kept at 16 bits
    if (p.inv_q_scale != 0.f)
      return dtype == EJK_RPA_BF16 ? dispatch<__nv_bfloat16, 2>(p, map, map_v, n_sm, stream, pdl)
                                   : dispatch<__half, 2>(p, map, map_v, n_sm, stream, pdl);
    return dtype == EJK_RPA_BF16 ? dispatch<__nv_bfloat16, 1>(p, map, map_v, n_sm, stream, pdl)
                                 : dispatch<__half, 1>(p, map, map_v, n_sm, stream, pdl);
  }
  if (dtype == EJK_RPA_BF16) return dispatch<__nv_bfloat16, 0>(p, map, map_v, n_sm, stream, pdl);
  return dispatch<__half, 0>(p, map, map_v, n_sm, stream, pdl);
}

}  // namespace ejk
