// KV-cache page write of the v3 operator: the new key/value rows of this step are scattered
// into the paged cache before attention reads it.
//
// The reference does this per sequence by gathering all of the sequence's pages, blending the new
// rows in with a mask, and scattering every page back
// (ejkernel/kernels/_xla/ragged_page_attention_v3/_kernel.py:227-240); its cache layout
// [P, page, 2*Hkv/pack, pack, D_aligned] with `merge_kv` (:45-57) putting K_h at combined index 2h
// and V_h at 2h+1 is byte-identical to the [P, page, 2*Hkv, D_aligned] layout the attention kernels
// read (with the combined heads padded to a multiple of `pack`: [P, page, C2, D_aligned], C2 >= 2*Hkv).  Here one CTA moves one token: its 2*Hkv*D new elements go to one contiguous row of one page,
// so the update costs exactly the bytes of the new rows (read once, written once).
#include <cuda_bf16.h>

#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kUpdThreads = 128;

// token t of the batch belongs to the sequence s with query_start_loc[s] <= t < query_start_loc[s+1]
__device__ __forceinline__ int find_seq(const int32_t* cu, int S, int t) {
  int lo = 0, hi = S;  // answer in [lo, hi)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu[mid] <= t) lo = mid;
    else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(kUpdThreads)
rpa_kv_update_kernel(const uint4* __restrict__ k_new, const uint4* __restrict__ v_new, uint4* __restrict__ cache,
                     const int32_t* __restrict__ kv_lens, const int32_t* __restrict__ block_tables,
                     const int32_t* __restrict__ query_start_loc, const int32_t* __restrict__ num_seqs,
                     int32_t* status, int T, int S_max, int pages_per_seq, int num_pages, int page_size, int Hkv,
                     int C2, int d16, int dalign16) {
  // d16 / dalign16: head_dim and padded head_dim in 16-byte units; C2: combined heads per row in memory (>= 2 * Hkv)
  const int t = blockIdx.x;
  int S = num_seqs[0];
  unsigned flags = 0;
  if (S > S_max) {
    S = S_max;
    flags |= EJK_RPA_ST_NUM_SEQS;
  }
  if (S <= 0 || t >= query_start_loc[S] || t < query_start_loc[0]) return;  // row belongs to no sequence
  const int s = find_seq(query_start_loc, S, t);
  const int q0 = query_start_loc[s], q_len = query_start_loc[s + 1] - q0;
  const int kv_len = kv_lens[s];
  const int pos = kv_len - q_len + (t - q0);
  const int pi = pos / page_size;
  if (pos < 0 || kv_len > pages_per_seq * page_size || pi >= pages_per_seq) {
    if (threadIdx.x == 0 && status) atomicOr(reinterpret_cast<unsigned*>(status), flags | EJK_RPA_ST_QLEN);
    return;
  }
  int page = block_tables[(size_t)s * pages_per_seq + pi];
  if ((unsigned)page >= (unsigned)num_pages) {
    if (threadIdx.x == 0 && status) atomicOr(reinterpret_cast<unsigned*>(status), flags | EJK_RPA_ST_PAGE_ID);
    return;  // never write through a bad page id
  }
  uint4* dst = cache + ((size_t)page * page_size + (pos - pi * page_size)) * C2 * dalign16;
  const uint4* ks = k_new + (size_t)t * Hkv * d16;
  const uint4* vs = v_new + (size_t)t * Hkv * d16;
  const int per_row = C2 * dalign16;
  for (int i = threadIdx.x; i < per_row; i += kUpdThreads) {
    const int c = i / dalign16, e = i - c * dalign16;  // combined head, 16-byte chunk
    uint4 v = make_uint4(0u, 0u, 0u, 0u);              // the padding lanes and padding heads of merge_kv are zeros
    if (e < d16 && c < 2 * Hkv) v = (c & 1) ? vs[(c >> 1) * d16 + e] : ks[(c >> 1) * d16 + e];
    dst[i] = v;
  }
  if (flags && threadIdx.x == 0 && status) atomicOr(reinterpret_cast<unsigned*>(status), flags);
}

}  // namespace

cudaError_t launch_kv_update(const void* k_new, const void* v_new, void* cache, const int32_t* kv_lens,
                             const int32_t* block_tables, const int32_t* query_start_loc, const int32_t* num_seqs,
                             int32_t* status, int T, int S_max, int pages_per_seq, int num_pages, int page_size, int Hkv,
                             int C2, int D, int Dalign, int elem_bytes, cudaStream_t stream) {
  // rows move as 16-byte words: 8 elements of a 16-bit cache, 16 of an e4m3 cache
  rpa_kv_update_kernel<<<T, kUpdThreads, 0, stream>>>(
      static_cast<const uint4*>(k_new), static_cast<const uint4*>(v_new), static_cast<uint4*>(cache), kv_lens,
      block_tables, query_start_loc, num_seqs, status, T, S_max, pages_per_seq, num_pages, page_size, Hkv, C2,
      D * elem_bytes / 16, Dalign * elem_bytes / 16);
  return cudaGetLastError();
}

}  // namespace ejk
