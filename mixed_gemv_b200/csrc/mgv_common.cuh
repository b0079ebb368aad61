// Shared host/device helpers of the library: status plumbing and the PTX wrappers the
// kernels use (mbarrier, bulk asynchronous copy, cp.async, warp-level MMA).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mixed_gemv_b200.h"

namespace mgv {

// ---- status plumbing (host) ----

mgv_status fail(mgv_status st, const char *fmt, ...);
mgv_status cuda_fail(cudaError_t err, const char *what);

#define MGV_CUDA_TRY(expr)                                        \
  do {                                                            \
    cudaError_t mgv_err__ = (expr);                               \
    if (mgv_err__ != cudaSuccess) return cuda_fail(mgv_err__, #expr); \
  } while (0)

// Device-side error word: kernels OR a code into it when a bounded wait gives up.
enum : int {
  DEVERR_FULL_WAIT = 1,   // a consumer warp gave up waiting for a stage to fill
  DEVERR_EMPTY_WAIT = 2,  // the producer gave up waiting for a stage to drain
  DEVERR_DRAIN_WAIT = 4   // the producer gave up waiting for its own copies at exit
};
int *device_error_word();  // device address of the word on the current device

#if defined(__CUDACC__)

// ---- mbarrier ----

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Waits for the phase with the given parity to complete, for at most about one second.
// Returns false when it gave up; the caller records the failure and unwinds.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > 1000000000ull) return false;
  }
}

// ---- asynchronous copies ----

// 1-D bulk copy global -> shared of `bytes` (multiple of 16; both addresses 16-byte aligned),
// completion counted in bytes on `bar`.  No multicast.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src, uint32_t bytes,
                                         uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst_smem)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

template <int BYTES>
__device__ __forceinline__ void cp_async_small(void *dst_smem, const void *src) {
  static_assert(BYTES == 4 || BYTES == 8 || BYTES == 16, "cp.async size");
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(smem_u32(dst_smem)), "l"(src),
               "n"(BYTES)
               : "memory");
}

// Makes `bar` receive one arrival (already counted at init) once all of this thread's
// earlier cp.async copies have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t *bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint4 lds128(const void *p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(smem_u32(p)));
  return v;
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- integer -> fp16 converters for the preprocessed layouts ----
// Same arithmetic as gemv/interleaved_numeric_conversion.h:225-298 (u4) and :55-88 (u8):
// splice the unsigned field into the mantissa of 1024.0 and subtract the offset in fp16.
// Both are exact, so any ordering of these steps gives the reference's values.

// One word of the int4 layout -> 8 signed values as 4 half2 in natural k order.
__device__ __forceinline__ void cvt_u4x8(uint32_t w, uint32_t (&h)[4]) {
  const uint32_t top = w >> 8;
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(h[0]) : "r"(w));
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(h[1]) : "r"(w));
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(h[2]) : "r"(top));
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(h[3]) : "r"(top));
  const uint32_t k1032 = 0x64086408u, k16th = 0x2c002c00u, kneg72 = 0xd480d480u;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(h[0]) : "r"(h[0]), "r"(k1032));
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(h[1]) : "r"(h[1]), "r"(k16th), "r"(kneg72));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(h[2]) : "r"(h[2]), "r"(k1032));
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(h[3]) : "r"(h[3]), "r"(k16th), "r"(kneg72));
}

// One word of the int8 layout (bytes e0 e2 e1 e3) -> 4 signed values as 2 half2, natural order.
__device__ __forceinline__ void cvt_u8x4(uint32_t w, uint32_t (&h)[2]) {
  asm("prmt.b32 %0, %1, 0x64646464, 0x5250;" : "=r"(h[0]) : "r"(w));
  asm("prmt.b32 %0, %1, 0x64646464, 0x5351;" : "=r"(h[1]) : "r"(w));
  const uint32_t k1152 = 0x64806480u;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(h[0]) : "r"(h[0]), "r"(k1152));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(h[1]) : "r"(h[1]), "r"(k1152));
}

#endif  // __CUDACC__

}  // namespace mgv
