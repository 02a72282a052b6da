// Split-KV ragged paged attention for small query tiles (decode rows, short speculative or
// chunk tails): one work item = (sequence, row tile of 8*NT (token,head-in-group) rows, KV chunk,
// kv head).  HBM-bound: every K_h/V_h row of the chunk is read exactly once and serves the whole
// GQA group.
//
// Replaces the inner loops of the reference
//   ejkernel/kernels/_xla/ragged_page_attention/_xla_impl_fwd.py:99-159
// (page-table slice, page gather, QK^T, soft cap, masks, online softmax, PV) without ever
// materialising gathered K/V copies in HBM.
//
// Data movement: persistent CTAs walk their work items as ONE continuous stream of 64-token
// stages, so the cp.async pipeline never drains between items.  A stage holds K_h and V_h of 64
// tokens as 128-byte rows [kv][d/64][token][64] with the 16-byte chunk index XOR-ed by (token & 7)
// (the 128B swizzle pattern), which makes every ldmatrix below bank-conflict free.
//
// Math (transposed so the tiny query tile is the N operand and no tensor-core rows are wasted):
//   S^T[16 tok x 8 rows]  = K[16 tok x D] * Q^T[D x 8 rows]        mma.m16n8k16, K via ldmatrix
//   O^T[D x 8 rows]      += V^T[D x 16 tok] * P^T[16 tok x 8 rows]  V via ldmatrix.trans,
//                                                                   P^T via movmatrix.trans
// Each of the 4 warps takes 16 of the stage's 64 tokens and keeps its own (m, l, O^T); the warps
// are combined at the end of the item, then the item writes either the final rows or one
// (m, l, O) partial for the merge kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "rpa_device.cuh"
#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kRing = 8;
constexpr float kLog2e = 1.4426950408889634f;

template <int D, int NT, int NS>
struct Cfg {
  static constexpr int TK = kTileTokens;
  static constexpr int RT = 8 * NT;
  static constexpr int STAGE_BYTES = TK * 2 * D * 2;
  static constexpr int Q_ROW_BYTES = D * 2 + 16;
  static constexpr int Q_BYTES = RT * Q_ROW_BYTES;
  static constexpr int OFF_Q = NS * STAGE_BYTES;
  static constexpr int OFF_OBUF = OFF_Q + NS * Q_BYTES;
  static constexpr int OFF_MBUF = OFF_OBUF + RT * D * 4;
  static constexpr int OFF_LBUF = OFF_MBUF + kWarps * RT * 4;
  static constexpr int OFF_FBUF = OFF_LBUF + kWarps * RT * 4;
  static constexpr int OFF_ROWSCALE = OFF_FBUF + kWarps * RT * 4;
  static constexpr int OFF_ROWM = OFF_ROWSCALE + RT * 4;
  static constexpr int OFF_ROWL = OFF_ROWM + RT * 4;
  static constexpr int OFF_RING = (OFF_ROWL + RT * 4 + 31) / 32 * 32;
  static constexpr int SMEM_BYTES = OFF_RING + kRing * (int)sizeof(Unit) + 1024;  // + alignment slack
};

struct Cursor {
  Unit u;
  int wid;    // flattened work id = unit index * Hkv + kv head
  int k;      // how many items this CTA has started before this one
  int pos;    // first key of the current stage
  int h;      // kv head
  bool valid;
};

__device__ __forceinline__ Unit load_unit_global(const Unit* units, int idx) {
  const int4* src = reinterpret_cast<const int4*>(units + idx);
  int4 a = __ldg(src), b = __ldg(src + 1);
  Unit u;
  u.seq = a.x; u.row0 = a.y; u.kv_begin = a.z; u.kv_end = a.w;
  u.slot = b.x; u.q_start = b.y; u.q_len = b.z; u.kv_len = b.w;
  return u;
}

template <typename T, int D, int NT, int NS>
__global__ void __launch_bounds__(kThreads, (Cfg<D, NT, NS>::SMEM_BYTES <= 112 * 1024) ? 2 : 1)
rpa_splitkv_kernel(const Params p) {
  using C = Cfg<D, NT, NS>;
  constexpr int TK = C::TK, RT = C::RT;
  constexpr int KT = D / 16;  // k-steps of QK^T == m-tiles of O^T

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  float* obuf = reinterpret_cast<float*>(smem + C::OFF_OBUF);
  float* mbuf = reinterpret_cast<float*>(smem + C::OFF_MBUF);
  float* lbuf = reinterpret_cast<float*>(smem + C::OFF_LBUF);
  float* row_scale = reinterpret_cast<float*>(smem + C::OFF_ROWSCALE);
  float* row_m = reinterpret_cast<float*>(smem + C::OFF_ROWM);
  float* row_l = reinterpret_cast<float*>(smem + C::OFF_ROWL);
  Unit* ring = reinterpret_cast<Unit*>(smem + C::OFF_RING);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_work = p.header[kHdrNumUnits] * p.Hkv;
  const int Hkv = p.Hkv, G = p.G;
  unsigned flags = 0;

  auto load_cursor = [&](Cursor& c) {
    c.valid = c.wid < n_work;
    if (c.valid) {
      const int ui = c.wid / Hkv;
      c.h = c.wid - ui * Hkv;
      c.u = load_unit_global(p.units, ui);
      c.pos = c.u.kv_begin;
      if (tid == 0) ring[c.k % kRing] = c.u;
    }
  };
  auto advance_pref = [&](Cursor& c) {
    if (!c.valid) return;
    c.pos += TK;
    if (c.pos >= c.u.kv_end) {
      c.wid += gridDim.x;
      c.k += 1;
      load_cursor(c);
    }
  };

  // ---- stage producer: page-table driven gather of 64 tokens of (K_h, V_h) ----
  auto issue_stage = [&](const Cursor& c, int slot) {
    if (!c.valid) return;
    constexpr int CPT = D / 4;                 // 16-byte chunks per token (K_h then V_h)
    constexpr int ITERS = TK * CPT / kThreads;
    const uint32_t sbase = smem_base + slot * C::STAGE_BYTES;
    const int32_t* tab = p.block_tables + (size_t)c.u.seq * p.pages_per_seq;
    const size_t head_stride = (size_t)p.Dkv * sizeof(T);  // K_h and V_h are one (possibly padded) row apart
    const size_t tok_stride = (size_t)p.C2 * head_stride;
    const uint8_t* kvb = reinterpret_cast<const uint8_t*>(p.kv) + (size_t)(2 * c.h) * head_stride;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int cidx = tid + i * kThreads;
      const int tok = cidx / CPT, within = cidx % CPT;
      const int key = c.pos + tok;
      const bool ok = key < c.u.kv_end;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.kv);
      if (ok) {
        int pi, sl;
        if (p.page_shift >= 0) {
          pi = key >> p.page_shift;
          sl = key & (p.page_size - 1);
        } else {
          pi = key / p.page_size;
          sl = key - pi * p.page_size;
        }
        int page = __ldg(tab + pi);
        if ((unsigned)page >= (unsigned)p.num_pages) {
          flags |= EJK_RPA_ST_PAGE_ID;
          page = 0;
        }
        if (p.v_cache == nullptr) {
          src = kvb + ((size_t)page * p.page_size + sl) * tok_stride + (within / (D / 8)) * head_stride +
                (within % (D / 8)) * 16;
        } else {
          // separate caches [blocks, Hkv, block_size, D] (page_attention): K from one, V from the other
          const uint8_t* base = reinterpret_cast<const uint8_t*>((within / (D / 8)) ? p.v_cache : p.kv);
          src = base + ((((size_t)page * Hkv + c.h) * p.page_size + sl) * D) * sizeof(T) + (within % (D / 8)) * 16;
        }
      }
      const int kvsel = within / (D / 8), d16 = within % (D / 8);
      const int row = (kvsel * (D / 64) + (d16 >> 3)) * TK + tok;
      const uint32_t dst = sbase + row * 128 + (((d16 & 7) ^ (row & 7)) << 4);
      cp_async16(dst, src, ok ? 16 : 0);
    }
    if (c.pos == c.u.kv_begin) {  // first stage of an item also brings its query tile
      constexpr int QCH = D / 8;  // 16-byte chunks per query row
      const uint32_t qbase = smem_base + C::OFF_Q + slot * C::Q_BYTES;
      const int rows_total = c.u.q_len * G;
      for (int cidx = tid; cidx < RT * QCH; cidx += kThreads) {
        const int r = cidx / QCH, ch = cidx % QCH;
        const int R = c.u.row0 + r;
        const bool ok = R < rows_total;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.q);
        if (ok) {
          const int qt = R / G, g = R - qt * G;
          src += ((size_t)(c.u.q_start + qt) * p.Hq + c.h * G + g) * D * sizeof(T) + ch * 16;
        }
        cp_async16(qbase + r * C::Q_ROW_BYTES + ch * 16, src, ok ? 16 : 0);
      }
    }
  };

  // ---- per-item consumer state ----
  uint32_t qf[NT][KT][2];   // Q^T fragments (B operand)
  float acc[NT][KT][4];     // O^T accumulators
  float m_run[NT][2], l_run[NT][2];
  int pos_r[NT][2], lo_r[NT][2];
  int pos_min = 0, lo_max = 0;

  Cursor pf;
  pf.wid = blockIdx.x;
  pf.k = 0;
  load_cursor(pf);
  Cursor cc = pf;  // the consumer starts on the same item

#pragma unroll
  for (int s = 0; s < NS - 1; ++s) {
    issue_stage(pf, s);
    cp_async_commit();
    advance_pref(pf);
  }

  int it = 0;
  while (cc.valid) {
    cp_async_wait<NS - 2>();
    __syncthreads();
    issue_stage(pf, (it + NS - 1) % NS);
    cp_async_commit();
    advance_pref(pf);

    const int slot = it % NS;
    const uint32_t sbase = smem_base + slot * C::STAGE_BYTES;

    if (cc.pos == cc.u.kv_begin) {
      // new item: query fragments from the slot's query tile, row metadata, fresh state
      const uint8_t* qs = smem + C::OFF_Q + slot * C::Q_BYTES;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint8_t* qrow = qs + (nt * 8 + (lane >> 2)) * C::Q_ROW_BYTES + (lane & 3) * 4;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          qf[nt][kt][0] = *reinterpret_cast<const uint32_t*>(qrow + kt * 32);
          qf[nt][kt][1] = *reinterpret_cast<const uint32_t*>(qrow + kt * 32 + 16);
        }
      }
      const int rows_total = cc.u.q_len * G;
      const int base = cc.u.kv_len - cc.u.q_len;
      int n_rows = rows_total - cc.u.row0;
      if (n_rows > RT) n_rows = RT;
      pos_min = base + cc.u.row0 / G;
      lo_max = (p.window > 0) ? (base + (cc.u.row0 + n_rows - 1) / G - p.window) : -1;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int R = cc.u.row0 + nt * 8 + (lane & 3) * 2 + j;
          const bool ok = R < rows_total;
          const int ps = ok ? base + R / G : -1;
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

    // ---- this warp's 16 tokens of the stage ----
    const int key0 = cc.pos + warp * 16;
    if (key0 < cc.u.kv_end) {
      float s[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
      {
        // K rows: matrices (tok 0-7,d 0-7) (tok 8-15,d 0-7) (tok 0-7,d 8-15) (tok 8-15,d 8-15)
        const int tok = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int dhalf = lane >> 4;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          const int d16 = kt * 2 + dhalf;
          const int row = (d16 >> 3) * TK + tok;
          uint32_t a[4];
          ldmatrix_x4(a, sbase + row * 128 + (((d16 & 7) ^ (row & 7)) << 4));
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) Mma<T>::run(s[nt], a, qf[nt][kt][0], qf[nt][kt][1]);
        }
      }
      // logits in the log2 domain, soft cap, masks (_xla_impl_fwd.py:125-138)
      const bool need_mask = (key0 + 15 > pos_min) || (key0 <= lo_max);
      uint32_t pb[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = s[nt][e];
          if (p.cap != 0.f) x = p.cap_log2 * soft_cap_tanh(x * p.inv_cap_scale);
          else x *= p.scale_log2;
          if (need_mask) {
            const int key = key0 + (lane >> 2) + (e >> 1) * 8;
            const int j = e & 1;
            if (key > pos_r[nt][j] || key <= lo_r[nt][j]) x = -INFINITY;
          }
          s[nt][e] = x;
        }
        float alpha[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float mx = fmaxf(s[nt][j], s[nt][j + 2]);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m_run[nt][j], mx);
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
          alpha[j] = fast_exp2(m_run[nt][j] - m_use);
          m_run[nt][j] = m_new;
          const float p0 = fast_exp2(s[nt][j] - m_use);
          const float p1 = fast_exp2(s[nt][j + 2] - m_use);
          s[nt][j] = p0;
          s[nt][j + 2] = p1;
          l_run[nt][j] = l_run[nt][j] * alpha[j] + p0 + p1;
        }
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          acc[nt][kt][0] *= alpha[0];
          acc[nt][kt][1] *= alpha[1];
          acc[nt][kt][2] *= alpha[0];
          acc[nt][kt][3] *= alpha[1];
        }
        // P^T as the B operand: transpose the two 8x8 (token x row) blocks
        pb[nt][0] = movmatrix_trans(Mma<T>::pack(s[nt][0], s[nt][1]));
        pb[nt][1] = movmatrix_trans(Mma<T>::pack(s[nt][2], s[nt][3]));
      }
      {
        // V^T tiles: matrices (tok 0-7,d 0-7) (tok 0-7,d 8-15) (tok 8-15,d 0-7) (tok 8-15,d 8-15), transposed
        const int tok = warp * 16 + (lane & 7) + (lane >> 4) * 8;
        const int dhalf = (lane >> 3) & 1;
#pragma unroll
        for (int mt = 0; mt < KT; ++mt) {
          const int d16 = mt * 2 + dhalf;
          const int row = ((D / 64) + (d16 >> 3)) * TK + tok;
          uint32_t a[4];
          ldmatrix_x4_trans(a, sbase + row * 128 + (((d16 & 7) ^ (row & 7)) << 4));
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) Mma<T>::run(acc[nt][mt], a, pb[nt][0], pb[nt][1]);
        }
      }
    }

    // ---- end of item: combine the warps, write rows or a partial ----
    if (cc.pos + TK >= cc.u.kv_end) {
      const int rows_total = cc.u.q_len * G;
      int n_rows = rows_total - cc.u.row0;
      if (n_rows > RT) n_rows = RT;
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
      __syncthreads();
      // Every lane derives the rescale factors of its own rows; the accumulators are then added
      // into obuf in four rounds, warp w handling d-slice (w + round) % 4, so each address gets
      // its four contributions in a fixed order (deterministic, no floating-point atomics).
      float f_own[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int r = nt * 8 + (lane & 3) * 2 + j;
          float mt = -INFINITY;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) mt = fmaxf(mt, mbuf[w * RT + r]);
          const float mu = (mt == -INFINITY) ? 0.f : mt;
          f_own[nt][j] = fast_exp2(m_run[nt][j] - mu);
        }
      if (tid < RT) {
        const int r = tid;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mt = fmaxf(mt, mbuf[w * RT + r]);
        const float mu = (mt == -INFINITY) ? 0.f : mt;
        float lt = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) lt += lbuf[w * RT + r] * fast_exp2(mbuf[w * RT + r] - mu);
        float sc = 1.f;
        if (cc.u.slot < 0) {
          float l_fin = lt;
          if (p.num_sinks > 0 && r < n_rows) {
            // attention sinks join the denominator only (_xla_impl_fwd.py:161-172)
            const int R = cc.u.row0 + r;
            const int hq = cc.h * G + (R % G);
            const int srow = (p.sink_rows == p.Hq) ? hq : (p.sink_rows == Hkv ? cc.h : 0);
            const float* sk = p.sinks + (size_t)srow * p.num_sinks;
            float sm = -INFINITY;
            for (int i = 0; i < p.num_sinks; ++i) sm = fmaxf(sm, sk[i] * kLog2e);
            const float m_fin = fmaxf(mt, sm);
            const float mf = (m_fin == -INFINITY) ? 0.f : m_fin;
            sc = fast_exp2(mt - mf);
            l_fin = lt * sc;
            for (int i = 0; i < p.num_sinks; ++i) l_fin += fast_exp2(sk[i] * kLog2e - mf);
          }
          sc = (l_fin > 0.f) ? sc * p.out_scale / l_fin : 0.f;  // out_scale: v_scale of the v3 operator, else 1
        }
        row_scale[r] = sc;
        row_m[r] = mt;
        row_l[r] = lt;
      }
#pragma unroll
      for (int round = 0; round < kWarps; ++round) {
        const int slice = (warp + round) % kWarps;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int r0 = nt * 8 + (lane & 3) * 2;
          const float f0 = f_own[nt][0], f1 = f_own[nt][1];
#pragma unroll
          for (int mi = 0; mi < KT / kWarps; ++mi) {
#pragma unroll
            for (int sl = 0; sl < kWarps; ++sl) {
              if (sl == slice) {  // compile-time accumulator index in every branch
                const int mt = sl * (KT / kWarps) + mi;
                const int d = mt * 16 + (lane >> 2);
                float* o0 = &obuf[r0 * D + d];
                float* o1 = &obuf[(r0 + 1) * D + d];
                if (round == 0) {
                  o0[0] = acc[nt][mt][0] * f0;
                  o0[8] = acc[nt][mt][2] * f0;
                  o1[0] = acc[nt][mt][1] * f1;
                  o1[8] = acc[nt][mt][3] * f1;
                } else {
                  o0[0] += acc[nt][mt][0] * f0;
                  o0[8] += acc[nt][mt][2] * f0;
                  o1[0] += acc[nt][mt][1] * f1;
                  o1[8] += acc[nt][mt][3] * f1;
                }
              }
            }
          }
        }
        __syncthreads();
      }
      if (cc.u.slot < 0) {
        T* out = reinterpret_cast<T*>(p.out);
        for (int i = tid; i < n_rows * (D / 2); i += kThreads) {
          const int r = i / (D / 2), d = (i % (D / 2)) * 2;
          const int R = cc.u.row0 + r;
          const int qt = R / G, g = R - qt * G;
          const float sc = row_scale[r];
          const float2 v = *reinterpret_cast<float2*>(&obuf[r * D + d]);
          const uint32_t pk = Mma<T>::pack(v.x * sc, v.y * sc);
          *reinterpret_cast<uint32_t*>(out + ((size_t)(cc.u.q_start + qt) * p.Hq + cc.h * G + g) * D + d) = pk;
        }
      } else {
        float* po = p.part_o + ((size_t)cc.u.slot * Hkv + cc.h) * RT * D;
        float2* pml = p.part_ml + ((size_t)cc.u.slot * Hkv + cc.h) * RT;
        for (int i = tid; i < n_rows * (D / 4); i += kThreads) {
          const int r = i / (D / 4), d = (i % (D / 4)) * 4;
          const float4 v = *reinterpret_cast<float4*>(&obuf[r * D + d]);
          *reinterpret_cast<float4*>(po + r * D + d) = v;
        }
        if (tid < n_rows) pml[tid] = make_float2(row_m[tid], row_l[tid]);
      }
      // the next item's writes to mbuf/obuf/row_* are separated from these reads by the stage barrier
    }

    // advance the consumer
    cc.pos += TK;
    if (cc.pos >= cc.u.kv_end) {
      cc.wid += gridDim.x;
      cc.k += 1;
      cc.valid = cc.wid < n_work;
      if (cc.valid) {
        const int ui = cc.wid / Hkv;
        cc.h = cc.wid - ui * Hkv;
        cc.u = ring[cc.k % kRing];
        cc.pos = cc.u.kv_begin;
      }
    }
    ++it;
  }
  cp_async_wait<0>();
  if (flags && p.status) atomicOr(reinterpret_cast<unsigned*>(p.status), flags);
  zero_tail_rows(p.out, p.header[kHdrTailStart], p.T, (size_t)p.Hq * D * sizeof(T));
}

template <typename T, int D, int NT, int NS>
cudaError_t launch_one(const Params& p, int n_sm, cudaStream_t stream) {
  using C = Cfg<D, NT, NS>;
  auto kern = rpa_splitkv_kernel<T, D, NT, NS>;
  static bool configured[64] = {};  // the attribute is per function and per device
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int per_sm = (C::SMEM_BYTES <= 112 * 1024) ? 2 : 1;
  kern<<<n_sm * per_sm, kThreads, C::SMEM_BYTES, stream>>>(p);
  return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch(const Params& p, int n_sm, cudaStream_t stream) {
  const bool wide = p.rows_per_tile == 16;
  switch (p.D) {
    case 64:
      return wide ? launch_one<T, 64, 2, 4>(p, n_sm, stream) : launch_one<T, 64, 1, 4>(p, n_sm, stream);
    case 128:
      return wide ? launch_one<T, 128, 2, 3>(p, n_sm, stream) : launch_one<T, 128, 1, 3>(p, n_sm, stream);
    case 256:
      return wide ? launch_one<T, 256, 2, 2>(p, n_sm, stream) : launch_one<T, 256, 1, 3>(p, n_sm, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_splitkv(const Params& p, int dtype, int n_sm, cudaStream_t stream) {
  if (dtype == EJK_RPA_BF16) return dispatch<__nv_bfloat16>(p, n_sm, stream);
  return dispatch<__half>(p, n_sm, stream);
}

}  // namespace ejk
