// Q4_0 dequant-matmul for batches above 16 rows on the 5th-generation tensor cores
// (tcgen05.mma, accumulator in tensor memory).
//
// Roles are swapped with respect to the textbook GEMM ("swap-AB"): the 128 output features of
// one packed 64-byte block of the weight matrix are the MMA's M dimension and the batch rows
// its N dimension (padded to a multiple of 16, up to 256), so hardly any tensor work is spent on
// padding.  Per 64-row k block a CTA
//   * loads 64 x 64 packed bytes and their scale pairs into registers (prefetched one block
//     ahead), turns the nibbles into fp16(code * scale) — the reference's operand value,
//     triton_kernels.py:444-445 — and stores them as the A operand in MN-major, 128-byte-swizzled
//     shared memory: the 64 high-nibble features are one 128-byte row segment per k, the 64
//     low-nibble features the other (inside each group of four the features sit in the order
//     0,2,1,3, which is undone when the accumulator is read back);
//   * copies the 64-wide slice of the activations as the K-major B operand;
//   * one thread issues four tcgen05.mma (K = 16 each) that accumulate into tensor memory, and
//     a tcgen05.commit on the stage's mbarrier lets the stage be refilled three blocks later.
// The k range is split over a thread-block cluster; the partial accumulators are exchanged
// through distributed shared memory (no global scratch).  Every mbarrier wait is bounded: on
// expiry the kernel records an error code, skips the remaining work, frees its tensor memory
// and returns.
//
// Replaces matmul_q40_kernel (triton_kernels.py:357-469) for M > 16.
#include <cooperative_groups.h>

#include "q40_common.cuh"

namespace cg = cooperative_groups;

namespace q40 {

constexpr int TC_THREADS = 256;
constexpr int TC_BK = 64;                      // k rows per pipeline stage
constexpr int TC_STAGES = 3;
constexpr int TC_TILE_N = 128;                 // output features per CTA
constexpr int TC_A_BYTES = TC_TILE_N * TC_BK * 2;   // 16 KB
constexpr unsigned TC_SPIN_LIMIT = 1u << 22;   // polls of ~50 ns each before giving up

struct TcParams {
  const __half* a;      // [M, lda]
  int64_t lda;
  const uint8_t* bw;    // [K, N/2]
  const __half* bs;     // [K, N/64]
  __half* c;            // [M, ldc]
  int64_t ldc;
  int M, N, K, Mpad, rows_per_split;
  int* err;             // device word, set non-zero when a bounded wait expired
};

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;      // descriptor version of this architecture
  d |= (uint64_t)2 << 61;      // 128-byte swizzle
  return d;
}

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// bounded wait; returns false when the limit was reached
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned it = 0; it < TC_SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// feature index inside a 64-feature half for MMA row p: the dequantiser writes each group of four
// features in the order 0,2,1,3
__device__ __forceinline__ int tc_unpermute(int p) { return (p & ~3) | ((p & 1) << 1) | ((p >> 1) & 1); }

__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const TcParams p) {
  extern __shared__ unsigned char tc_smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int kb = split * p.rows_per_split;
  const int ke = min(p.K, kb + p.rows_per_split);
  const int nblk = (ke - kb) / TC_BK;                       // host guarantees >= 1 and exact
  const int b_bytes = p.Mpad * 128;                          // B stage: Mpad rows x 64 k x 2 B
  const int stage_bytes = TC_A_BYTES + b_bytes;

  // 1024-byte aligned carve-up: [stages][barriers][tmem slot]; the fp32 tile reuses the stages
  const uint32_t raw = tc_smem_u32(tc_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = tc_smem_raw + (base - raw);
  const uint32_t bars = base + TC_STAGES * stage_bytes;      // free[0..STAGES), done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + TC_STAGES * stage_bytes + 64);

  int ncols = 32;
  while (ncols < p.Mpad) ncols <<= 1;

  if (tid == 0) {
    for (int s = 0; s <= TC_STAGES; ++s) tc_mbar_init(bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"(ncols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  // instruction descriptor: D fp32, A/B fp16, A MN-major, B K-major, N = Mpad, M = 128
  const uint32_t idesc = (1u << 4) | (1u << 15) | ((uint32_t)(p.Mpad >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

  // this thread's share of a stage: 16 packed bytes of k row (tid / 4)
  const int kr = tid >> 2, qd = tid & 3;
  const int64_t w_ld = p.N / 2, s_ld = p.N / 64;
  const uint8_t* wp = p.bw + (int64_t)(kb + kr) * w_ld + tile * 64 + 16 * qd;
  const __half* sp = p.bs + (int64_t)(kb + kr) * s_ld + tile * 2;
  uint4 wreg = __ldg(reinterpret_cast<const uint4*>(wp));
  uint32_t sreg = __ldg(reinterpret_cast<const uint32_t*>(sp));

  bool failed = false;
  for (int i = 0; i < nblk; ++i) {
    const int s = i % TC_STAGES;
    uint4 wnext = wreg;
    uint32_t snext = sreg;
    if (i + 1 < nblk) {
      wnext = __ldg(reinterpret_cast<const uint4*>(wp + (int64_t)(i + 1) * TC_BK * w_ld));
      snext = __ldg(reinterpret_cast<const uint32_t*>(sp + (int64_t)(i + 1) * TC_BK * s_ld));
    }
    if (i >= TC_STAGES) failed |= !tc_mbar_wait(bars + 8 * s, (uint32_t)((i / TC_STAGES - 1) & 1));

    unsigned char* a_st = gbase + s * stage_bytes;
    unsigned char* b_st = a_st + TC_A_BYTES;
    // ---- A operand: row kr of k group kr/8; high nibbles -> feature chunk 0, low -> chunk 1 ----
    {
      const __half2 s_hi = __half2half2(__ushort_as_half((unsigned short)(sreg & 0xFFFF)));
      const __half2 s_lo = __half2half2(__ushort_as_half((unsigned short)(sreg >> 16)));
      const uint32_t wds[4] = {wreg.x, wreg.y, wreg.z, wreg.w};
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        const uint32_t w0 = wds[wi], w1 = w0 >> 8;
        hi[2 * wi] = h2_as_u32(__hmul2(codes_hi_to_h2(w0), s_hi));       // features (0, 2) of the group of 4
        hi[2 * wi + 1] = h2_as_u32(__hmul2(codes_hi_to_h2(w1), s_hi));   // features (1, 3)
        lo[2 * wi] = h2_as_u32(__hmul2(codes_lo_to_h2(w0), s_lo));
        lo[2 * wi + 1] = h2_as_u32(__hmul2(codes_lo_to_h2(w1), s_lo));
      }
      const int kg = kr >> 3, r8 = kr & 7;
      unsigned char* row_hi = a_st + (kg * 2 + 0) * 1024 + r8 * 128;
      unsigned char* row_lo = a_st + (kg * 2 + 1) * 1024 + r8 * 128;
      const int j0 = 2 * qd;            // 16 features = two 16-byte chunks of the 128-byte row
      *reinterpret_cast<uint4*>(row_hi + (((j0) ^ r8) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(row_hi + (((j0 + 1) ^ r8) << 4)) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
      *reinterpret_cast<uint4*>(row_lo + (((j0) ^ r8) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      *reinterpret_cast<uint4*>(row_lo + (((j0 + 1) ^ r8) << 4)) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
    }
    // ---- B operand: activations [Mpad, 64], K-major, rows beyond M are zero ----
    {
      const int k0 = kb + i * TC_BK;
      for (int idx = tid; idx < p.Mpad * 8; idx += TC_THREADS) {
        const int m = idx >> 3, j = idx & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < p.M) v = *reinterpret_cast<const uint4*>(p.a + (int64_t)m * p.lda + k0 + 8 * j);
        *reinterpret_cast<uint4*>(b_st + (m >> 3) * 1024 + (m & 7) * 128 + ((j ^ (m & 7)) << 4)) = v;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> tensor core reads
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    failed = __syncthreads_or(failed ? 1 : 0) != 0;
    if (failed) break;
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_u32 = base + s * stage_bytes, b_u32 = a_u32 + TC_A_BYTES;
#pragma unroll
      for (int ks = 0; ks < TC_BK / 16; ++ks) {
        const uint64_t ad = tc_desc(a_u32 + ks * 4096, 1024, 2048);   // two k groups per MMA
        const uint64_t bd = tc_desc(b_u32 + ks * 32, 16, 1024);       // 16 k = 32 bytes along the row
        tc_mma(tmem, ad, bd, idesc, (i > 0 || ks > 0) ? 1u : 0u);
      }
      tc_commit(bars + 8 * s);                      // stage s may be refilled when these MMAs are done
      if (i == nblk - 1) tc_commit(bars + 8 * TC_STAGES);
    }
    wreg = wnext;
    sreg = snext;
  }
  if (!failed) failed = !tc_mbar_wait(bars + 8 * TC_STAGES, 0);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  failed = __syncthreads_or(failed ? 1 : 0) != 0;
  if (failed && tid == 0) atomicExch(p.err, 1);

  // ---- accumulator -> fp32 tile in shared memory, [Mpad][128] with features in natural order ----
  float* tile_f = reinterpret_cast<float*>(gbase);
  if (!failed) {
    const int q = warp & 3;                         // TMEM lanes 32q .. 32q+31 belong to this warp
    const int row = 32 * q + lane;                  // MMA row = feature slot
    const int feat = (row < 64) ? tc_unpermute(row) : 64 + tc_unpermute(row - 64);
    const int nchunk = p.Mpad / 16;
    for (int ch = (warp >> 2); ch < nchunk; ch += 2) {   // warps 0-3 even chunks, warps 4-7 odd chunks
      uint32_t r[16];
      tc_ld16(tmem + ((uint32_t)(32 * q) << 16) + ch * 16, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 16; ++j) tile_f[(ch * 16 + j) * TC_TILE_N + feat] = __uint_as_float(r[j]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols));
  }
  cluster.sync();

  // ---- split-K over the cluster: every rank finishes a slice of the (m, feature) pairs ----
  const int nranks = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int total = p.M * TC_TILE_N;
  const int per = (total + nranks - 1) / nranks;
  const int e0 = rank * per, e1 = min(total, e0 + per);
  if (!failed) {
    for (int e = e0 + tid; e < e1; e += TC_THREADS) {
      float t[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) t[r] = (r < nranks) ? *cluster.map_shared_rank(tile_f + e, r) : 0.f;
      float v = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) v += t[r];
      const int m = e / TC_TILE_N, n = tile * TC_TILE_N + e % TC_TILE_N;
      if (n < p.N) p.c[(int64_t)m * p.ldc + n] = __float2half_rn(v);
    }
  }
  cluster.sync();
}

}  // namespace q40

// C[M,N] = A[M,K] @ deq(B)[K,N] for 16 < M, group 64, K % 64 == 0, N % 128 == 0, on tcgen05.
// `err` is a device int the kernel sets to 1 if one of its bounded waits expires (results are then
// undefined); the caller zeroes it beforehand and may read it after synchronising.
extern "C" int q40_gemm_kn_tc(const void* a, int64_t lda, const void* bw, const void* bs, void* c,
                              int64_t ldc, int M, int N, int K, int* err, void* stream) {
  using namespace q40;
  if (!a || !bw || !bs || !c || !err) return Q40_E_NULL;
  if (M < 1 || N <= 0 || K <= 0 || N % 128 != 0 || K % TC_BK != 0) return Q40_E_SHAPE;
  if (lda < K || ldc < N || lda % 8 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(a, 16) || !q40_aligned(bw, 16) || !q40_aligned(bs, 4)) return Q40_E_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const int tiles = N / TC_TILE_N;
  const int kblocks = K / TC_BK;
  // split K over a cluster (<= 8) so that about one CTA per SM is busy, each with >= 4 k blocks
  int nsplit = 1;
  while (nsplit < 8 && tiles * nsplit * 2 <= 160 && kblocks % (nsplit * 2) == 0 && kblocks / (nsplit * 2) >= 4)
    nsplit *= 2;
  const __half* ah = (const __half*)a;
  __half* ch = (__half*)c;
  for (int m0 = 0; m0 < M; m0 += 256) {
    const int mc = (M - m0) < 256 ? (M - m0) : 256;
    TcParams p{};
    p.a = ah + (int64_t)m0 * lda; p.lda = lda;
    p.bw = (const uint8_t*)bw; p.bs = (const __half*)bs;
    p.c = ch + (int64_t)m0 * ldc; p.ldc = ldc;
    p.M = mc; p.N = N; p.K = K; p.Mpad = (mc + 15) / 16 * 16;
    p.rows_per_split = K / nsplit;
    p.err = err;
    const size_t stage = (size_t)TC_A_BYTES + (size_t)p.Mpad * 128;
    size_t smem = TC_STAGES * stage;
    const size_t tile_f = (size_t)p.Mpad * TC_TILE_N * 4;
    if (tile_f > smem) smem = tile_f;
    smem += 1024 /* alignment slack */ + 128 /* barriers + tmem slot */;
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(tiles, nsplit, 1);
    cfg.blockDim = dim3(TC_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = nsplit;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel, p);
    if (e != cudaSuccess) return (int)e;
  }
  return Q40_OK;
}
