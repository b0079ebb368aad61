// Shared host/device helpers of the library: status plumbing and the PTX wrappers the
// kernels use (shared-memory addresses, the global timer, warp-level MMA, the integer converters).
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
int *device_error_word();  // device address of the word on the current device

#if defined(__CUDACC__)

// ---- PTX wrappers ----

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
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
