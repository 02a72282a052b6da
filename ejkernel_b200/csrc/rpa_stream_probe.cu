// Read-only streaming probe: how fast this GPU moves bytes from HBM into shared memory with bulk asynchronous
// copies -- the mechanism the split-KV kernel gathers KV pages with -- when nothing else is done with them.  It is the
// practical ceiling for that kernel (a copy benchmark reads AND writes, so a read-only stream can be faster than it),
// measured on the device the library runs on and with the same 2 CTAs per SM and ring depth.
//
// One warp per CTA: lane 0 issues 32 KB copies into a ring of slots, each completing on its slot's mbarrier; the warp
// waits for a slot (bounded, like every wait in this library), touches one word of it and reissues.  CTA b takes
// chunks b, b + grid, b + 2 grid, ... so neighbouring CTAs read neighbouring addresses.  No multicast.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rpa_device.cuh"
#include "rpa_types.h"

namespace ejk {
namespace {

constexpr int kProbeMaxSlots = 12;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__global__ void __launch_bounds__(32) rpa_stream_probe_kernel(const uint8_t* src, unsigned long long n_chunks,
                                                              unsigned* sink, unsigned long long wait_ns, int chunk,
                                                              int slots) {
  extern __shared__ uint8_t probe_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(probe_raw) + 127) & ~uintptr_t(127));
  __shared__ __align__(8) unsigned long long bars[kProbeMaxSlots];
  const uint32_t sb = smem_u32(smem), bar0 = smem_u32(bars);
  const int lane = threadIdx.x;
  if (lane == 0) {
    for (int s = 0; s < slots; ++s) mbar_init(bar0 + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  unsigned long long mine = 0;  // chunks of this CTA
  if (blockIdx.x < n_chunks) mine = (n_chunks - blockIdx.x + gridDim.x - 1) / gridDim.x;
  auto issue = [&](unsigned long long k) {
    const int s = (int)(k % slots);
    if (lane == 0) {
      mbar_arrive_expect_tx(bar0 + s * 8, chunk);
      bulk_load(sb + s * chunk, src + (blockIdx.x + k * gridDim.x) * (unsigned long long)chunk, chunk,
                bar0 + s * 8);
    }
  };
  unsigned long long issued = 0;
  for (; issued < mine && issued < slots; ++issued) issue(issued);
  unsigned acc = 0;
  unsigned long long done = 0;
  bool ok = true;
  for (; done < mine; ++done) {
    const int s = (int)(done % slots);
    // the outcome is made warp-uniform, so the lanes never part ways on it
    ok = __all_sync(0xffffffffu, mbar_wait_quiet(bar0 + s * 8, (uint32_t)((done / slots) & 1), wait_ns));
    if (!ok) break;
    acc ^= *reinterpret_cast<volatile unsigned*>(smem + s * chunk + lane * 4);
    __syncwarp();
    if (issued < mine) {
      // the slot was read through the generic proxy; order that before the next asynchronous write into it
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      issue(issued);
      ++issued;
    }
  }
  if (!ok) {
    // giving up: let the copies that are still in flight land (bounded) before the shared memory goes back
    for (unsigned long long k = done; k < issued; ++k)
      mbar_wait_quiet(bar0 + (int)(k % slots) * 8, (uint32_t)((k / slots) & 1), 2000000ull);
    if (lane == 0) atomicOr(sink + 1, 1u);
  }
  if (acc == 0x9e3779b9u && lane == 0) atomicAdd(sink, 1u);  // keeps the reads alive; practically never true
}

}  // namespace

cudaError_t launch_stream_probe(const void* src, size_t bytes, unsigned* sink, int n_sm, int wait_ms, int chunk_kb, int slots,
                                int ctas_per_sm, cudaStream_t stream) {
  // defaults: 32 KB copies, 3 slots (96 KB of shared memory), two CTAs per SM -- as the split-KV kernel runs
  const int chunk = (chunk_kb > 0 ? chunk_kb : 32) * 1024;
  if (slots <= 0) slots = 3;
  if (ctas_per_sm <= 0) ctas_per_sm = 2;
  if (slots > kProbeMaxSlots || (size_t)slots * chunk > 220 * 1024) return cudaErrorInvalidValue;
  const unsigned long long n_chunks = bytes / chunk;  // whole copies only
  const size_t smem = (size_t)slots * chunk + 128;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(rpa_stream_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 221 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  rpa_stream_probe_kernel<<<ctas_per_sm * n_sm, 32, smem, stream>>>(static_cast<const uint8_t*>(src), n_chunks, sink,
                                                                     (unsigned long long)wait_ms * 1000000ull, chunk, slots);
  return cudaGetLastError();
}

}  // namespace ejk
