// Thin inline-PTX wrappers used by the attention kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace ejk {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global->shared copy; src_bytes == 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// transpose an 8x8 matrix of 16-bit elements held one row-pair per thread
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}

template <typename T>
struct Mma;
template <>
struct Mma<__nv_bfloat16> {
  // D(16x8,f32) += A(16x16,row) * B(16x8,col)
  __device__ static __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct Mma<__half> {
  __device__ static __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
};

// ---- mbarrier helpers shared by the TMA kernels ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that lets the hardware park the thread for up to `hint_ns` while the phase is incomplete
// (it wakes as soon as the phase completes): a waiting warp then issues almost no instructions,
// which matters when it shares a scheduler with warps that do the arithmetic.
__device__ __forceinline__ bool mbar_try_wait_park(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
constexpr uint32_t kParkNs = 4000;
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
// Bounded wait, executed by all 32 lanes of a warp.  Gives up when `timeout_ns` of wall time have
// passed or when another warp of the CTA has raised `abort_flag`; the outcome is made
// warp-uniform so the lanes never part ways on it.  false = gave up (the flag is then set).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long timeout_ns) {
  bool ok = mbar_try_wait(bar, parity);
  if (!ok) {
    const unsigned long long t0 = global_timer_ns();
    while (true) {
      if (mbar_try_wait_park(bar, parity, kParkNs)) {
        ok = true;
        break;
      }
      if (*abort_flag) break;
      if (global_timer_ns() - t0 > timeout_ns) break;
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) *abort_flag = 1;
  return ok;
}

// Bounded wait that ignores the abort flag: used on the way out of a kernel, to give bulk copies that
// are still in flight time to land before the CTA's shared memory is released.
__device__ __forceinline__ bool mbar_wait_quiet(uint32_t bar, uint32_t parity, unsigned long long timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  while (global_timer_ns() - t0 <= timeout_ns)
    if (mbar_try_wait_park(bar, parity, kParkNs)) return true;
  return false;
}

// Same bounded wait for a role that runs on a single thread (no warp vote).
__device__ __forceinline__ bool mbar_wait_thread(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                 unsigned long long timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  while (true) {
    if (mbar_try_wait_park(bar, parity, kParkNs)) return true;
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > timeout_ns) break;
  }
  *abort_flag = 1;
  return false;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while its predecessor in the stream is still running.  pdl_wait() blocks until that
// predecessor has completed and its memory is visible; pdl_trigger() lets this kernel's own
// dependents start (they are released once every CTA has called it or exited).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// Zero-fills rows [row0, T) of a dense [T, row_bytes] output, spread over all threads of the grid.
// row_bytes is a multiple of 16 and `out` is 16-byte aligned (both checked on the host).
__device__ __forceinline__ void zero_tail_rows(void* out, int row0, int T, size_t row_bytes) {
  if (row0 >= T) return;
  uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(out) + (size_t)row0 * row_bytes);
  const size_t n16 = (size_t)(T - row0) * row_bytes / 16;
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) dst[i] = z;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// logits_soft_cap: cap * tanh(x / cap), with tanh from one ex2 and one division:
// tanh(t) = 1 - 2 / (exp(2t) + 1); exact at +-inf, relative error ~1e-6.
__device__ __forceinline__ float soft_cap_tanh(float t) {
  float e = fast_exp2(t * 2.885390081777927f);  // exp(2t)
  return 1.0f - __fdividef(2.0f, e + 1.0f);
}

}  // namespace ejk
