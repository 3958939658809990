// Shared helpers for the q40b200 kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/q40b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "q40b200 kernels are written for sm_100a only"
#endif

#define Q40_LAUNCH_CHECK()                          \
  do {                                              \
    cudaError_t e__ = cudaGetLastError();           \
    if (e__ != cudaSuccess) return (int)e__;        \
  } while (0)

static inline bool q40_aligned(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }

namespace q40 {

__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t mask, uint32_t x) {
  uint32_t r;
  // (a & mask) ^ x : immLut = (0xF0 & 0xCC) ^ 0xAA
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(mask), "r"(x));
  return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) {
  return *reinterpret_cast<__half2*>(&v);
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) {
  return *reinterpret_cast<uint32_t*>(&v);
}

// Two signed 4-bit codes sitting in the LOW nibbles of bytes 0 and 2 of `p` -> exact half2.
// (nib ^ 8) | 0x6400 is the half 1024 + (code + 8); subtracting 1032 is exact.
__device__ __forceinline__ __half2 codes_lo_to_h2(uint32_t p) {
  uint32_t v = lop3_and_xor(p, 0x000F000Fu, 0x64086408u);
  return __hsub2(u32_as_h2(v), u32_as_h2(0x64086408u));
}
// Same for the HIGH nibbles of bytes 0 and 2: the half is 1024 + 16*(code + 8);
// fma(v, 1/16, -72) is exact.
__device__ __forceinline__ __half2 codes_hi_to_h2(uint32_t p) {
  uint32_t v = lop3_and_xor(p, 0x00F000F0u, 0x64806480u);
  return __hfma2(u32_as_h2(v), u32_as_h2(0x2C002C00u) /* 1/16 */, u32_as_h2(0xD480D480u) /* -72 */);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace q40
