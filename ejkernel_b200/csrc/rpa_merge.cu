// Combines the split-KV partials of one row tile: the online-softmax carry
// (_xla_impl_fwd.py:140-151 of the reference: rescale by exp(m_old - m_new), add) applied across KV
// chunks instead of across loop iterations, then the final normalisation (:173-177) and the
// optional attention sinks (:161-172).  One warp owns one output row (several share it when rows are few and chunks
// many); chunk maxima are reduced with warp shuffles, the D-wide accumulation is lane-parallel.
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
  __shared__ float s_acc[kMergeWarps][D];
  __shared__ float s_l[kMergeWarps];
  // launched as a programmatic dependent of the split-KV kernel (its launch latency then lies under that kernel's
  // tail): nothing of the plan or the partials may be read before that kernel has completed
  pdl_wait();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int n_warps = gridDim.x * kMergeWarps;
  const int RT = p.rows_per_tile, Hkv = p.Hkv, G = p.G;
  const int n_items = p.header[kHdrNumMerge];
  const long long total = (long long)n_items * Hkv * RT;
  T* out = reinterpret_cast<T*>(p.out);
  // K warps share one row when there are few rows for the grid (a head shard of a long-context batch: 64 tiles of
  // dozens of chunks each): every chunk is an L2 round trip, and K warps make K times fewer of them one after
  // another.  All K compute the row's maximum (a pass over 8 bytes per chunk), each sums every K-th chunk relative
  // to it, and the sums are added in warp order in shared memory.  K is the same for every block of a launch.
  int K = 1;
  while (K < kMergeWarps && total * (2 * K) <= (long long)n_warps) K *= 2;
  const int rows_per_block = kMergeWarps / K;
  const int sub = wid % K, rib = wid / K;

  for (long long base = (long long)blockIdx.x * rows_per_block; base < total; base += (long long)gridDim.x * rows_per_block) {
    const long long w = base + rib;
    bool valid = w < total;
    int r = 0, h = 0, R = 0, n = 0;
    MergeItem mi = {};
    if (valid) {
      r = (int)(w % RT);
      h = (int)((w / RT) % Hkv);
      mi = p.merge[(int)(w / ((long long)RT * Hkv))];
      R = mi.row0 + r;
      n = mi.n_chunks;
      valid = R < mi.q_len * G;
    }
    float acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[i] = 0.f;
    float l_tot = 0.f, m_tot = -INFINITY;
    if (valid) {
      // pass 1: global maximum over chunks
      for (int c = lane; c < n; c += 32) {
        const float2 ml = p.part_ml[((size_t)(mi.slot0 + c) * Hkv + h) * RT + r];
        m_tot = fmaxf(m_tot, ml.x);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m_tot = fmaxf(m_tot, __shfl_xor_sync(0xffffffffu, m_tot, o));
      const float mu = (m_tot == -INFINITY) ? 0.f : m_tot;

      // pass 2: rescaled sums over this warp's chunks (sub, sub + K, ...).  Eight chunks' loads in flight at a time
      // (a row of a long context has dozens of chunks); the sums still run in chunk order
      constexpr int kInFlight = 8;
      for (int c0 = sub; c0 < n; c0 += kInFlight * K) {
        float2 ml[kInFlight];
        float vv[kInFlight][VPL];
#pragma unroll
        for (int j = 0; j < kInFlight; ++j) {
          const int c = min(c0 + j * K, n - 1);
          const size_t at = ((size_t)(mi.slot0 + c) * Hkv + h) * RT + r;
          ml[j] = p.part_ml[at];
          const float* po = p.part_o + at * D + lane * VPL;
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
          if (c0 + j * K < n) {
            const float f = fast_exp2(ml[j].x - mu);
            l_tot += ml[j].y * f;
#pragma unroll
            for (int i = 0; i < VPL; ++i) acc[i] += vv[j][i] * f;
          }
        }
      }
    }
    if (K > 1) {  // the same for every thread of the launch: the barriers are reached by all
      if (sub > 0) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) s_acc[wid][lane * VPL + i] = acc[i];
        if (lane == 0) s_l[wid] = l_tot;
      }
      __syncthreads();
      if (sub == 0) {
        for (int k = 1; k < K; ++k) {
#pragma unroll
          for (int i = 0; i < VPL; ++i) acc[i] += s_acc[wid + k][lane * VPL + i];
          l_tot += s_l[wid + k];
        }
      }
      __syncthreads();
    }
    if (!valid || sub > 0) continue;
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
    T* dst = out + ((size_t)(mi.q_start + qt) * p.Hq + hq) * p.Dq + lane * VPL;
    if (lane * VPL < p.Dq) {  // p.Dq < D: the output row is narrower than the partials (see Params::Dq)
#pragma unroll
      for (int i = 0; i < VPL; i += 2) {
        *reinterpret_cast<uint32_t*>(dst + i) = Mma<T>::pack(acc[i] * sc, acc[i + 1] * sc);
      }
    }
  }
}

template <typename T>
cudaError_t dispatch(const Params& p, int n_sm, cudaStream_t stream, bool pdl) {
  const dim3 grid(n_sm * 2), block(kMergeWarps * 32);
  switch (p.D) {
    case 64:
      return launch_kernel(rpa_merge_kernel<T, 64>, grid, block, 0, stream, pdl, p);
    case 128:
      return launch_kernel(rpa_merge_kernel<T, 128>, grid, block, 0, stream, pdl, p);
    case 256:
      return launch_kernel(rpa_merge_kernel<T, 256>, grid, block, 0, stream, pdl, p);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_merge(const Params& p, int dtype, int n_sm, cudaStream_t stream, bool pdl) {
  if (dtype == EJK_RPA_BF16) return dispatch<__nv_bfloat16>(p, n_sm, stream, pdl);
  return dispatch<__half>(p, n_sm, stream, pdl);
}

}  // namespace ejk
