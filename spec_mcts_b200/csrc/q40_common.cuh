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

// Launch with programmatic stream serialization.  Kernels launched this way execute griddepcontrol.wait
// before their first access to global memory, so for the caller the launch orders exactly like a plain
// one; what changes is that the CTAs may become resident while the previous launch on the stream drains
// (and, where that launch triggered early, while it runs), which takes the launch latency off the
// critical path of a chain of small dependent launches.
template <typename... KArgs, typename... Args>
static inline cudaError_t q40_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Optional stage timestamps (builds with -DQ40_TRACE only; compiled out otherwise): thread 0 of a CTA
// reads the global nanosecond timer at up to 8 points and appends one record of 10 words
// {kind, linear CTA id, t0..t7} to the buffer given to q40_debug_trace (word 0 = record counter,
// word 1 = capacity in records, records from word 16).
#ifdef Q40_TRACE
extern void* q40_trace_ptr;
#define Q40_TRACE_DECL unsigned long long q40_ts_[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define Q40_STAMP(i) \
  do { if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(q40_ts_[i])::"memory"); } while (0)
#define Q40_STAMP_DEP(i, v) /* not before the float v is available */ \
  do { if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(q40_ts_[i]) : "f"(v) : "memory"); } while (0)
#define Q40_TRACE_FLUSH(buf, kind)                                                                   \
  do {                                                                                               \
    unsigned long long* tb_ = (unsigned long long*)(buf);                                            \
    if (threadIdx.x == 0 && tb_) {                                                                   \
      const unsigned long long slot_ = atomicAdd(tb_, 1ull);                                         \
      if (slot_ < tb_[1]) {                                                                          \
        unsigned long long* r_ = tb_ + 16 + slot_ * 10;                                              \
        r_[0] = (kind);                                                                              \
        r_[1] = (unsigned long long)blockIdx.x + (unsigned long long)gridDim.x * blockIdx.y;         \
        for (int i_ = 0; i_ < 8; ++i_) r_[2 + i_] = q40_ts_[i_];                                     \
      }                                                                                              \
    }                                                                                                \
  } while (0)
#else
#define Q40_TRACE_DECL
#define Q40_STAMP(i) do { } while (0)
#define Q40_STAMP_DEP(i, v) do { } while (0)
#define Q40_TRACE_FLUSH(buf, kind) do { } while (0)
#endif

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
