// Combines the split-KV partials of one row tile: the online-softmax carry
// (_xla_impl_fwd.py:140-151 of the reference: rescale by exp(m_old - m_new), add) applied across KV
// chunks instead of across loop iterations, then the final normalisation (:173-177) and the
// optional attention sinks (:161-172).  One warp owns one output row; chunk maxima are reduced with
// warp shuffles, the D-wide accumulation is lane-parallel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "rpa_device.cuh"
#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kMergeWarps = 8;
constexpr float kLog2e = 1.4426950408889634f;

template <typename T, int D>
__global__ void __launch_bounds__(kMergeWarps * 32) rpa_merge_kernel(const Params p) {
  constexpr int VPL = D / 32;  // floats per lane
  const int lane = threadIdx.x & 31;
  const int gwarp = blockIdx.x * kMergeWarps + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * kMergeWarps;
  const int RT = p.rows_per_tile, Hkv = p.Hkv, G = p.G;
  const int n_items = p.header[kHdrNumMerge];
  const long long total = (long long)n_items * Hkv * RT;
  T* out = reinterpret_cast<T*>(p.out);

  for (long long w = gwarp; w < total; w += n_warps) {
    const int r = (int)(w % RT);
    const int h = (int)((w / RT) % Hkv);
    const int item = (int)(w / ((long long)RT * Hkv));
    const MergeItem mi = p.merge[item];
    const int R = mi.row0 + r;
    if (R >= mi.q_len * G) continue;
    const int n = mi.n_chunks;

    // pass 1: global maximum over chunks
    float m_tot = -INFINITY;
    for (int c = lane; c < n; c += 32) {
      const float2 ml = p.part_ml[((size_t)(mi.slot0 + c) * Hkv + h) * RT + r];
      m_tot = fmaxf(m_tot, ml.x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m_tot = fmaxf(m_tot, __shfl_xor_sync(0xffffffffu, m_tot, o));
    const float mu = (m_tot == -INFINITY) ? 0.f : m_tot;

    // pass 2: rescaled sums
    float acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[i] = 0.f;
    float l_tot = 0.f;
    // eight chunks' loads in flight at a time (each is an L2 round trip, and a row of a long context has
    // dozens of chunks); the sums still run in chunk order
    constexpr int kInFlight = 8;
    for (int c0 = 0; c0 < n; c0 += kInFlight) {
      float2 ml[kInFlight];
      float vv[kInFlight][VPL];
#pragma unroll
      for (int j = 0; j < kInFlight; ++j) {
        const int c = min(c0 + j, n - 1);
        const size_t base = ((size_t)(mi.slot0 + c) * Hkv + h) * RT + r;
        ml[j] = p.part_ml[base];
        const float* po = p.part_o + base * D + lane * VPL;
        if constexpr (VPL == 2) {
          const float2 v = *reinterpret_cast<const float2*>(po);
          vv[j][0] = v.x;
          vv[j][1] = v.y;
        } else {
#pragma unroll
          for (int i = 0; i < VPL; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(po + i);
            vv[j][i] = v.x;
            vv[j][i + 1] = v.y;
            vv[j][i + 2] = v.z;
            vv[j][i + 3] = v.w;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < kInFlight; ++j) {
        if (c0 + j < n) {
          const float f = fast_exp2(ml[j].x - mu);
          l_tot += ml[j].y * f;
#pragma unroll
          for (int i = 0; i < VPL; ++i) acc[i] += vv[j][i] * f;
        }
      }
    }
    const int qt = R / G, g = R - qt * G;
    const int hq = h * G + g;
    float sc = 1.f, l_fin = l_tot;
    if (p.num_sinks > 0) {
      const int srow = (p.sink_rows == p.Hq) ? hq : (p.sink_rows == Hkv ? h : 0);
      const float* sk = p.sinks + (size_t)srow * p.num_sinks;
      float sm = -INFINITY;
      for (int i = 0; i < p.num_sinks; ++i) sm = fmaxf(sm, sk[i] * kLog2e);
      const float m_fin = fmaxf(m_tot, sm);
      const float mf = (m_fin == -INFINITY) ? 0.f : m_fin;
      sc = fast_exp2(m_tot - mf);
      l_fin = l_tot * sc;
      for (int i = 0; i < p.num_sinks; ++i) l_fin += fast_exp2(sk[i] * kLog2e - mf);
    }
    sc = (l_fin > 0.f) ? sc * p.out_scale / l_fin : 0.f;  // out_scale: v_scale of the v3 operator, else 1
    T* dst = out + ((size_t)(mi.q_start + qt) * p.Hq + hq) * D + lane * VPL;
#pragma unroll
    for (int i = 0; i < VPL; i += 2) {
      *reinterpret_cast<uint32_t*>(dst + i) = Mma<T>::pack(acc[i] * sc, acc[i + 1] * sc);
    }
  }
}

template <typename T>
cudaError_t dispatch(const Params& p, int n_sm, cudaStream_t stream) {
  const int blocks = n_sm * 2;
  switch (p.D) {
    case 64:
      rpa_merge_kernel<T, 64><<<blocks, kMergeWarps * 32, 0, stream>>>(p);
      break;
    case 128:
      rpa_merge_kernel<T, 128><<<blocks, kMergeWarps * 32, 0, stream>>>(p);
      break;
    case 256:
      rpa_merge_kernel<T, 256><<<blocks, kMergeWarps * 32, 0, stream>>>(p);
      break;
    default:
      return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_merge(const Params& p, int dtype, int n_sm, cudaStream_t stream) {
  if (dtype == EJK_RPA_BF16) return dispatch<__nv_bfloat16>(p, n_sm, stream);
  return dispatch<__half>(p, n_sm, stream);
}

}  // namespace ejk
