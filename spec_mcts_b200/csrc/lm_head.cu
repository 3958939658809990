// Tail of a decode step in one launch: final RMSNorm, the fp16 lm_head product, and (optionally)
// greedy feedback — arg-max of every row written as the next input token and the position advanced.
//
// Reference: `h = self.norm(h); output = self.output(h).to(DTYPE)` (hf_model_q40_kv_shared.py:508-510);
// the lm_head is an fp16 nn.Linear (not quantised), 32016 x 4096 for the 7B model = 262 MB per step,
// HBM-bound.  RMSNorm keeps the reference's rounding points (fp32 inside, fp16, times fp16 weight); the
// product accumulates in fp32 like the library GEMM the reference calls and rounds once to fp16.
//
// Work split: a CTA takes pairs of 16-row vocabulary tiles; its eight warps are (tile of the pair) x
// (quarter of K).  A lane streams 16 bytes of its two vocabulary rows per 32-wide k chunk straight from
// global memory into the A fragments of two mma.m16n8k16 (the k order inside a chunk is permuted the
// same way for both operands, which a dot product does not notice), the activations come from shared
// memory, the four K quarters are added in a fixed order.
#include "q40_common.cuh"

namespace q40 {
namespace lmhead {

constexpr int THREADS = 256;
constexpr int XS_PAD = 32;          // halfs: row pitch = K + 32, i.e. 64 bytes past a multiple of 128

struct Params {
  const __half* h;        // [M, ldh] residual stream before the final norm
  int64_t ldh;
  const float* ss_in;     // [M, ss_count] partial sums of squares of h, or nullptr (computed here)
  int ss_count;
  const __half* norm_w;
  float eps;
  const __half* w;        // [V, K] lm_head weight
  __half* logits;         // [M, ldl]
  int64_t ldl;
  int M, V, K;
  int64_t* tok_out;       // [M] or nullptr
  int32_t* pos;           // [M] or nullptr: advanced by one together with tok_out
  unsigned long long* best;   // [16] running arg-max keys, zero between launches
  unsigned int* counter;      // CTAs finished, zero between launches
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ld_stream(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }

// fp16 bits -> unsigned key with the same order as the values (negative zero below positive zero)
__device__ __forceinline__ uint32_t order_key(__half v) {
  const uint32_t b = __half_as_ushort(v);
  return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
}

template <int MT>
__global__ void __launch_bounds__(THREADS, 2) lm_head_kernel(const Params p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int xs_ld = p.K + XS_PAD;
  __half* xs = reinterpret_cast<__half*>(smem);                                          // [M][xs_ld]
  float* red = reinterpret_cast<float*>(smem + (size_t)p.M * xs_ld * 2);                 // [2][4][16][8 * MT]
  float* s_inv = red + 2 * 4 * 16 * 8 * MT;                                              // [16]
  unsigned long long* s_best = reinterpret_cast<unsigned long long*>(s_inv + 16);        // [16]
  __shared__ int s_last;
  asm volatile("griddepcontrol.launch_dependents;");
  if (tid < 16) s_best[tid] = 0ull;
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- final RMSNorm of the M rows into shared memory ----
  for (int m = warp; m < p.M; m += THREADS / 32) {
    float s = 0.f;
    if (p.ss_in) {
      for (int i = lane; i < p.ss_count; i += 32) s += __ldcg(p.ss_in + (int64_t)m * p.ss_count + i);
    } else {
      for (int i = lane * 8; i < p.K; i += 256) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.h + (int64_t)m * p.ldh + i);
        const __half2* vh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(vh[j]);
          s = fmaf(f.x, f.x, s);
          s = fmaf(f.y, f.y, s);
        }
      }
    }
    s = warp_sum(s);
    if (lane == 0) s_inv[m] = rsqrtf(s / (float)p.K + p.eps);
  }
  __syncthreads();
  for (int idx = tid; idx < p.M * (p.K / 8); idx += THREADS) {
    const int m = idx / (p.K / 8), k = (idx % (p.K / 8)) * 8;
    uint4 v = *reinterpret_cast<const uint4*>(p.h + (int64_t)m * p.ldh + k);
    const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + k);
    const float inv = s_inv[m];
    __half2* vh = reinterpret_cast<__half2*>(&v);
    const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(vh[j]);
      vh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);
    }
    *reinterpret_cast<uint4*>(xs + (int64_t)m * xs_ld + k) = v;
  }
  __syncthreads();

  const int ntiles = (p.V + 15) / 16, npairs = (ntiles + 1) / 2;
  const int tl = warp >> 2, kq = warp & 3;
  const int kq_len = p.K / 4;
  // of the outputs this thread finishes: pass j of the output loop belongs to batch row tid / 32 + 8 * j
  unsigned long long my_best[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) my_best[j] = 0ull;
  for (int pair = blockIdx.x; pair < npairs; pair += gridDim.x) {
    const int tile = 2 * pair + tl;
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[mt][j] = 0.f;
    if (tile < ntiles) {
      const int ra = min(tile * 16 + g, p.V - 1), rb = min(tile * 16 + g + 8, p.V - 1);
      const __half* wa = p.w + (int64_t)ra * p.K + kq * kq_len + 8 * t;
      const __half* wb = p.w + (int64_t)rb * p.K + kq * kq_len + 8 * t;
      const __half* xr = xs + kq * kq_len + 8 * t;
      // the weights of the next 128 k are requested before the MMAs of the current ones (two batches of eight
      // 16-byte loads in flight per lane)
      uint4 na[4], nb[4];
      auto fetch = [&](int k0, uint4 (&a4)[4], uint4 (&b4)[4]) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const bool ok = k0 + 32 * u < kq_len;
          a4[u] = ok ? ld_stream(wa + k0 + 32 * u) : make_uint4(0, 0, 0, 0);
          b4[u] = ok ? ld_stream(wb + k0 + 32 * u) : make_uint4(0, 0, 0, 0);
        }
      };
      fetch(0, na, nb);
      for (int k0 = 0; k0 < kq_len; k0 += 128) {
        uint4 va[4], vb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { va[u] = na[u]; vb[u] = nb[u]; }
        if (k0 + 128 < kq_len) fetch(k0 + 128, na, nb);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (k0 + 32 * u >= kq_len) break;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const int row = mt * 8 + g;
            const uint4 xb = (row < p.M) ? *reinterpret_cast<const uint4*>(xr + (int64_t)row * xs_ld + k0 + 32 * u)
                                         : make_uint4(0, 0, 0, 0);
            mma16816(acc[mt], va[u].x, vb[u].x, va[u].y, vb[u].y, xb.x, xb.y);
            mma16816(acc[mt], va[u].z, vb[u].z, va[u].w, vb[u].w, xb.z, xb.w);
          }
        }
      }
    }
    // fragment -> red[tl][kq][row][batch]: c0 (row g, batch 2t), c1 (g, 2t+1), c2 (g+8, 2t), c3 (g+8, 2t+1)
    float* rw = red + ((tl * 4 + kq) * 16) * (8 * MT);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      rw[(g) * (8 * MT) + mt * 8 + 2 * t] = acc[mt][0];
      rw[(g) * (8 * MT) + mt * 8 + 2 * t + 1] = acc[mt][1];
      rw[(g + 8) * (8 * MT) + mt * 8 + 2 * t] = acc[mt][2];
      rw[(g + 8) * (8 * MT) + mt * 8 + 2 * t + 1] = acc[mt][3];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int idx = tid + j * THREADS;
      if (idx >= 2 * 16 * p.M) break;
      const int m = idx / 32, r32 = idx % 32, tl2 = r32 >> 4, r = r32 & 15;
      const int row = (2 * pair + tl2) * 16 + r;
      if (row < p.V) {
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) v += red[((tl2 * 4 + q) * 16 + r) * (8 * MT) + m];
        const __half hv = __float2half_rn(v);
        p.logits[(int64_t)m * p.ldl + row] = hv;
        const unsigned long long key = ((unsigned long long)order_key(hv) << 32) | (0xFFFFFFFFu - (uint32_t)row);
        my_best[j] = key > my_best[j] ? key : my_best[j];
      }
    }
    __syncthreads();
  }
  if (p.tok_out == nullptr) return;

  // ---- arg-max: CTA -> global running maximum (larger value wins, then the smaller index), the CTA
  // that finishes last publishes tokens and positions and leaves the scratch zeroed ----
#pragma unroll
  for (int j = 0; j < MT; ++j)
    if (my_best[j]) atomicMax(&s_best[tid / 32 + 8 * j], my_best[j]);
  __syncthreads();
  if (tid < p.M && s_best[tid]) atomicMax(p.best + tid, s_best[tid]);
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(p.counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {
    __threadfence();
    if (tid < p.M) {
      const unsigned long long k = __ldcg(p.best + tid);
      p.tok_out[tid] = (int64_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
      if (p.pos) p.pos[tid] += 1;
      p.best[tid] = 0ull;
    }
    if (tid == 0) *p.counter = 0u;
  }
}

}  // namespace lmhead
}  // namespace q40

// logits[M, V] = RMSNorm(h) @ w^T (fp16), optionally followed by greedy feedback.  See include/q40b200.h.
extern "C" int q40_lm_head(const void* h, int64_t ldh, const float* ss_in, int ss_count, const void* norm_w, float eps,
                           const void* w, int V, int K, void* logits, int64_t ldl, int M, int64_t* tok_out,
                           int32_t* pos, void* scratch, int use_pdl, void* stream) {
  using namespace q40::lmhead;
  if (!h || !norm_w || !w || !logits) return Q40_E_NULL;
  if (tok_out && !scratch) return Q40_E_WORKSPACE;
  if (M < 1 || M > 16 || V < 1 || K < 128 || K % 128 != 0 || ldh < K || ldl < V || ldh % 8 != 0) return Q40_E_SHAPE;
  if (ss_in && ss_count < 1) return Q40_E_SHAPE;
  if (!q40_aligned(h, 16) || !q40_aligned(norm_w, 16) || !q40_aligned(w, 16) || (scratch && !q40_aligned(scratch, 8)))
    return Q40_E_ALIGN;
  Params p{};
  p.h = (const __half*)h; p.ldh = ldh; p.ss_in = ss_in; p.ss_count = ss_count;
  p.norm_w = (const __half*)norm_w; p.eps = eps; p.w = (const __half*)w;
  p.logits = (__half*)logits; p.ldl = ldl; p.M = M; p.V = V; p.K = K;
  p.tok_out = tok_out; p.pos = pos;
  p.best = (unsigned long long*)scratch;
  p.counter = scratch ? (unsigned int*)((char*)scratch + 16 * 8) : nullptr;
  const int MT = M <= 8 ? 1 : 2;
  const size_t smem = (size_t)M * (K + XS_PAD) * 2 + (size_t)2 * 4 * 16 * 8 * MT * 4 + 16 * 4 + 16 * 8;
  auto kern = MT == 1 ? lm_head_kernel<1> : lm_head_kernel<2>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return Q40_E_UNSUPPORTED;
  }
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return Q40_E_UNSUPPORTED;
  const int npairs = ((V + 15) / 16 + 1) / 2;
  const int per_sm = smem <= 100 * 1024 ? 2 : 1;
  int grid = sms * per_sm;
  if (grid > npairs) grid = npairs;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = use_pdl ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}

// Bytes of zero-filled scratch q40_lm_head needs when it writes tokens (the kernel leaves it zeroed).
extern "C" size_t q40_lm_head_scratch_bytes(void) { return 16 * 8 + 16; }
