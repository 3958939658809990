// Q4_0 dequant-matmul for batches above 16 rows on the 5th-generation tensor cores
// (tcgen05.mma, accumulator in tensor memory).
//
// Roles are swapped with respect to the textbook GEMM ("swap-AB"): the 128 output features of
// one packed 64-byte block of the weight matrix are the MMA's M dimension and the batch rows
// its N dimension (padded to a multiple of 16, up to 256), so hardly any tensor work is spent on
// padding.  Per 64-row k block a CTA
//   * has its 64 x 64 packed bytes and scale pairs copied asynchronously into a lane-private ring
//     (the HBM stream), turns the nibbles into fp16(code * scale) — the reference's operand value,
//     triton_kernels.py:444-445 — and stores them as the A operand in MN-major, 128-byte-swizzled
//     shared memory: the 64 high-nibble features are one 128-byte row segment per k, the 64
//     low-nibble features the other (inside each group of four the features sit in the order
//     0,2,1,3, which is undone when the accumulator is read back);
//   * has the 64-wide slice of the activations copied asynchronously straight into the K-major,
//     swizzled B operand;
//   * one more warp issues four tcgen05.mma (K = 16 each) that accumulate into tensor memory as soon
//     as the block's producers have arrived on its "full" mbarrier, and a tcgen05.commit on the
//     stage's "free" mbarrier lets the stage be refilled.
// The eight producer warps work as G groups (4, or 2 above 112 batch rows where shared memory is the
// limit) that take the k blocks in turn, each with its own A stage: a group's chain of waits, copies,
// dequantisation, proxy fence and arrival spans G blocks of tensor-core time, and its copies for its
// next block (G blocks ahead) are in flight meanwhile.  There is no CTA-wide barrier in the loop.
// The k range is split over a thread-block cluster; the partial accumulators are exchanged
// through distributed shared memory (no global scratch).  Every mbarrier wait is bounded: on
// expiry the kernel records an error code, skips the remaining work, frees its tensor memory
// and returns.
//
// Replaces matmul_q40_kernel (triton_kernels.py:357-469) for M > 16.
#include <cooperative_groups.h>
#include <cstdio>

#include "q40_common.cuh"

namespace cg = cooperative_groups;

namespace q40 {

constexpr int TC_THREADS = 256;                // producer threads (8 warps; 16 measured no faster)
constexpr int TC_BLOCK = TC_THREADS + 32;      // + the warp that issues the MMAs
constexpr int TC_BK = 64;                      // k rows per pipeline stage
constexpr int TC_TILE_N = 128;                 // output features per CTA
constexpr int TC_A_BYTES = TC_TILE_N * TC_BK * 2;   // 16 KB per A stage
constexpr int TC_MAX_G = 4;                    // most producer groups (= A stages) of any variant
constexpr unsigned TC_SPIN_LIMIT = 1u << 22;   // polls of ~50 ns each before giving up

struct TcParams {
  const __half* a;      // [M, lda]
  int64_t lda;
  // up to three weight matrices that share the activations (wq, wk, wv): feature tiles of matrix 0
  // first, then matrix 1, ...
  const uint8_t* bw[3]; // [K, N/2]
  const __half* bs[3];  // [K, N/64]
  __half* c[3];         // [M, ldc]
  int64_t ldc[3];
  int N[3], tiles[3], nprob;
  int M, K, Mpad, rows_per_split;
  int* err;             // device word, set non-zero when a bounded wait expired
  void* trace;          // stage timestamps (trace builds only)
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

__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// NCOLS: tensor-memory columns of the accumulator, 32, 64, 128 or 256 (>= padded batch rows); G: producer
// groups = A stages.  One CTA per SM: the runtime never co-schedules two CTAs of a kernel that allocates
// tensor memory, so all latency hiding happens inside the CTA.
template <int NCOLS, int G>
__global__ void __launch_bounds__(TC_BLOCK, 1)
gemm_tc_kernel(const TcParams p) {
  extern __shared__ unsigned char tc_smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int pi = 0, tile = blockIdx.x;
  while (pi < p.nprob - 1 && tile >= p.tiles[pi]) { tile -= p.tiles[pi]; ++pi; }
  const int split = blockIdx.y;
  Q40_TRACE_DECL
  Q40_STAMP(0);
  const int kb = split * p.rows_per_split;
  const int ke = min(p.K, kb + p.rows_per_split);
  const int nblk = (ke - kb) / TC_BK;                       // host guarantees >= 1 and exact
  const int b_bytes = p.Mpad * 128;                          // B slot: Mpad rows x 64 k x 2 B
  constexpr int GT = TC_THREADS / G;                         // threads of a producer group
  constexpr int TPR = GT / 64;                               // threads per k row (64 packed bytes)
  constexpr int NQ = 4 / TPR;                                // 16-byte pieces per thread and block
  constexpr int BSLOTS = 2 * G;                              // block b+G is copied into the slot block b-G used
  constexpr int RAW_SLOT = 4096 + GT * 4;                    // a block's packed bytes + a scale pair per thread

  // 1024-byte aligned carve-up: [A stages][B slots][raw rings: 2 slots per group][barriers][tmem slot];
  // the fp32 tile of the epilogue reuses everything before the barriers
  const uint32_t raw = tc_smem_u32(tc_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = tc_smem_raw + (base - raw);
  const uint32_t b_base = base + G * TC_A_BYTES;
  unsigned char* ring = gbase + G * TC_A_BYTES + BSLOTS * b_bytes;
  const uint32_t ring_u32 = b_base + BSLOTS * b_bytes;
  const uint32_t bars = ring_u32 + G * 2 * RAW_SLOT;         // free[0..G), done, full[0..G)
  const uint32_t bar_done = bars + 8 * G, bar_full = bars + 8 * (G + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ring + G * 2 * RAW_SLOT + 8 * (2 * TC_MAX_G + 1));
  volatile int* s_failed = reinterpret_cast<volatile int*>(tmem_slot + 2);
  if (tid == 0) *s_failed = 0;

  constexpr int ncols = NCOLS;

  if (tid == 0) {
    for (int s = 0; s <= G; ++s) tc_mbar_init(bars + 8 * s, 1);
    for (int s = 0; s < G; ++s) tc_mbar_init(bar_full + 8 * s, GT);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "n"(ncols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  asm volatile("griddepcontrol.launch_dependents;");
  Q40_STAMP(1);

  // instruction descriptor: D fp32, A/B fp16, A MN-major, B K-major, N = Mpad, M = 128
  const uint32_t idesc = (1u << 4) | (1u << 15) | ((uint32_t)(p.Mpad >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

  bool failed = false;
  if (warp < TC_THREADS / 32) {
    // ================= producers: weights -> A operand, activations -> B operand =================
    // group `grp` takes the k blocks grp, grp + G, ...; inside it, thread gt owns NQ 16-byte pieces of
    // k row gt / TPR of every block
    const int grp = tid / GT, gt = tid % GT;
    const int kr = gt / TPR, q0 = (gt % TPR) * NQ;
    const int64_t w_ld = p.N[pi] / 2, s_ld = p.N[pi] / 64;
    const uint8_t* wp = p.bw[pi] + (int64_t)(kb + kr) * w_ld + tile * 64 + 16 * q0;
    const __half* sp = p.bs[pi] + (int64_t)(kb + kr) * s_ld + tile * 2;
    const uint32_t my_ring = ring_u32 + grp * 2 * RAW_SLOT;
    unsigned char* my_ring_g = ring + grp * 2 * RAW_SLOT;
    // raw weights of block blk into ring slot `rs`: piece q of row kr at [q][kr] (conflict-free reads)
    auto issue_raw = [&](int blk, int rs) {
      const uint32_t dst = my_ring + rs * RAW_SLOT;
#pragma unroll
      for (int q = 0; q < NQ; ++q)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + ((q0 + q) * 64 + kr) * 16),
                     "l"(wp + (int64_t)blk * TC_BK * w_ld + 16 * q));
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4096 + gt * 4),
                   "l"(sp + (int64_t)blk * TC_BK * s_ld));
    };
    // activations of block blk straight into B slot blk % BSLOTS: this thread copies chunk gt % 8
    // (16 bytes) of the 128-byte k slice of rows gt / 8, + GT / 8, ...; rows beyond M are zero-filled
    // (copy of size 0)
    const int bm0 = gt >> 3, bjj = gt & 7;
    const __half* bsrc = p.a + (int64_t)bm0 * p.lda + kb + 8 * bjj;
    const uint32_t bdst = b_base + (bm0 >> 3) * 1024 + (bm0 & 7) * 128 + ((bjj ^ (bm0 & 7)) << 4);
    auto issue_b = [&](int blk) {
      const uint32_t dst = bdst + (blk % BSLOTS) * b_bytes;
      const __half* src = bsrc + blk * TC_BK;
      for (int m = bm0, j = 0; m < p.Mpad; m += GT / 8, ++j) {
        const bool ok = m < p.M;
        const int sz = ok ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + j * (GT / 64) * 1024),
                     "l"(ok ? src + (int64_t)(GT / 8) * j * p.lda : p.a), "r"(sz));
      }
    };
    // the weights do not depend on the previous launch: their first block is requested before this
    // launch waits for it (programmatic dependent launch), the activations after
    if (grp < nblk) issue_raw(grp, 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (grp < nblk) issue_b(grp);
    asm volatile("cp.async.commit_group;");
    unsigned char* a_st = gbase + grp * TC_A_BYTES;
    for (int k = 0, blk = grp; blk < nblk; ++k, blk += G) {
      // the MMAs of this group's previous block are done: its A stage and the B slot of block blk + G
      // (the one block blk - G used) may be overwritten
      if (k >= 1 && !tc_mbar_wait(bars + 8 * grp, (uint32_t)((k - 1) & 1))) { failed = true; break; }
      if (blk + G < nblk) { issue_raw(blk + G, (k + 1) & 1); issue_b(blk + G); }
      asm volatile("cp.async.commit_group;");
      asm volatile("cp.async.wait_group 1;" ::: "memory");     // this thread's copies for block blk have landed
      // ---- A operand: row kr of k group kr/8; high nibbles -> feature chunk 0, low -> chunk 1 ----
      const unsigned char* slot = my_ring_g + (k & 1) * RAW_SLOT;
      const uint32_t sreg = *reinterpret_cast<const uint32_t*>(slot + 4096 + gt * 4);
      const __half2 s_hi = __half2half2(__ushort_as_half((unsigned short)(sreg & 0xFFFF)));
      const __half2 s_lo = __half2half2(__ushort_as_half((unsigned short)(sreg >> 16)));
      const int kg = kr >> 3, r8 = kr & 7;
      unsigned char* row_hi = a_st + (kg * 2 + 0) * 1024 + r8 * 128;
      unsigned char* row_lo = a_st + (kg * 2 + 1) * 1024 + r8 * 128;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const uint4 wreg = *reinterpret_cast<const uint4*>(slot + ((q0 + q) * 64 + kr) * 16);
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
        const int j0 = 2 * (q0 + q);      // 16 features = two 16-byte chunks of the 128-byte row
        *reinterpret_cast<uint4*>(row_hi + (((j0) ^ r8) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(row_hi + (((j0 + 1) ^ r8) << 4)) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
        *reinterpret_cast<uint4*>(row_lo + (((j0) ^ r8) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<uint4*>(row_lo + (((j0 + 1) ^ r8) << 4)) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> tensor core reads
      tc_mbar_arrive(bar_full + 8 * grp);
      if (blk == 0) Q40_STAMP(2);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else {
    // ================= the MMA warp: lane 0 issues, the warp stays converged =================
    // descriptors of A stage 0 / B slot 0; the others differ only in the 16-byte-granular start address
    // field (the low 14 bits; all of shared memory is below 256 KB, so the additions cannot carry out)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint64_t ad_base = tc_desc(base, 1024, 2048);          // A: two k groups per MMA
    const uint64_t bd_base = tc_desc(b_base, 16, 1024);          // B: 16 k = 32 bytes along the row
    for (int i = 0; i < nblk; ++i) {
      const int s = i % G;
      if (!tc_mbar_wait(bar_full + 8 * s, (uint32_t)((i / G) & 1))) { failed = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint64_t ad0 = ad_base + (uint64_t)((s * TC_A_BYTES) >> 4);
        const uint64_t bd0 = bd_base + (uint64_t)(((i % BSLOTS) * b_bytes) >> 4);
#pragma unroll
        for (int ks = 0; ks < TC_BK / 16; ++ks)
          tc_mma(tmem, ad0 + (uint64_t)((ks * 4096) >> 4), bd0 + (uint64_t)((ks * 32) >> 4), idesc,
                 (i > 0 || ks > 0) ? 1u : 0u);
        tc_commit(bars + 8 * s);                    // stage s may be refilled when these MMAs are done
        if (i == nblk - 1) tc_commit(bar_done);
      }
      __syncwarp();
    }
  }
  Q40_STAMP(3);
  if (failed) *s_failed = 1;
  if (!failed && !tc_mbar_wait(bar_done, 0)) *s_failed = 1;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncthreads();
  failed = *s_failed != 0;
  if (failed && tid == 0) atomicExch(p.err, 1);
  Q40_STAMP(4);

  // ---- accumulator -> fp32 tile in shared memory, [Mpad][128] with features in natural order ----
  float* tile_f = reinterpret_cast<float*>(gbase);
  if (!failed && warp < TC_THREADS / 32) {
    const int q = warp & 3;                         // TMEM lanes 32q .. 32q+31 belong to this warp
    const int row = 32 * q + lane;                  // MMA row = feature slot
    const int feat = (row < 64) ? tc_unpermute(row) : 64 + tc_unpermute(row - 64);
    const int nchunk = p.Mpad / 16;
    for (int ch = (warp >> 2); ch < nchunk; ch += TC_THREADS / 128) {   // four warps per chunk of 16 batch rows
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(ncols));
  }
  Q40_STAMP(5);
  cluster.sync();
  Q40_STAMP(6);

  // ---- split-K over the cluster: every rank finishes a slice of the (m, feature) pairs ----
  const int nranks = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int total = p.M * TC_TILE_N;                       // a multiple of 128
  const int per = ((total / 4 + nranks - 1) / nranks) * 4;
  const int e0 = rank * per, e1 = min(total, e0 + per);
  if (!failed) {
    for (int e = e0 + tid * 4; e < e1; e += TC_BLOCK * 4) {
      float4 t[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        t[r] = (r < nranks) ? *reinterpret_cast<const float4*>(cluster.map_shared_rank(tile_f + e, r))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) { v.x += t[r].x; v.y += t[r].y; v.z += t[r].z; v.w += t[r].w; }
      const int m = e / TC_TILE_N, n = tile * TC_TILE_N + e % TC_TILE_N;      // four features of one row
      if (n + 3 < p.N[pi]) {
        __half2* dst = reinterpret_cast<__half2*>(p.c[pi] + (int64_t)m * p.ldc[pi] + n);
        dst[0] = __floats2half2_rn(v.x, v.y);
        dst[1] = __floats2half2_rn(v.z, v.w);
      }
    }
  }
  Q40_STAMP(7);
  cluster.sync();
  Q40_TRACE_FLUSH(p.trace, 300);
}

}  // namespace q40

// How many clusters of (1, nsplit) CTAs with this much dynamic shared memory run at once (cached per
// shape of the question; 0 when the runtime cannot tell).
using TcKernel = void (*)(const q40::TcParams);
static int tc_groups_for(int mpad) { return mpad <= 112 ? 4 : 2; }      // what fits in shared memory
static TcKernel tc_kernel_for(int mpad) {
  if (mpad <= 32) return q40::gemm_tc_kernel<32, 4>;
  if (mpad <= 64) return q40::gemm_tc_kernel<64, 4>;
  if (mpad <= 112) return q40::gemm_tc_kernel<128, 4>;
  if (mpad <= 128) return q40::gemm_tc_kernel<128, 2>;
  return q40::gemm_tc_kernel<256, 2>;
}
static int tc_max_clusters(TcKernel kern, int mpad, int nsplit, size_t smem) {
  // [device][nsplit][padded rows / 16] -> fit + 1 (the shared memory size follows from the rows)
  static int cache_all[16][9][17] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) dev = 0;
  int (*cache)[17] = cache_all[dev];
  const int cls = mpad / 16;
  if (cache[nsplit][cls]) return cache[nsplit][cls] - 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1024, nsplit, 1);     // more clusters than any device holds: the answer is not capped
  cfg.blockDim = dim3(q40::TC_BLOCK, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = nsplit;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
#ifdef Q40_TRACE
  fprintf(stderr, "tc_max_clusters(nsplit %d, smem %zu) = %d\n", nsplit, smem, n);
#endif
  cache[nsplit][cls] = n + 1;
  return n;
}

// C[M,N] = A[M,K] @ deq(B)[K,N] for 16 < M, group 64, K % 64 == 0, N % 128 == 0, on tcgen05.
// `err` is a device int the kernel sets to 1 if one of its bounded waits expires (results are then
// undefined); the caller zeroes it beforehand and may read it after synchronising.
extern "C" int q40_gemm_kn_tc_multi(int nmat, const void* a, int64_t lda, const void* const* bw,
                                    const void* const* bs, void* const* c, const int64_t* ldc, const int* n_cols,
                                    int M, int K, int* err, int use_pdl, void* stream) {
  using namespace q40;
  if (!a || !bw || !bs || !c || !ldc || !n_cols || !err) return Q40_E_NULL;
  if (nmat < 1 || nmat > 3) return Q40_E_UNSUPPORTED;
  if (M < 1 || K <= 0 || K % TC_BK != 0 || lda < K || lda % 8 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(a, 16)) return Q40_E_ALIGN;
  int tiles = 0;
  for (int i = 0; i < nmat; ++i) {
    if (!bw[i] || !bs[i] || !c[i]) return Q40_E_NULL;
    if (n_cols[i] <= 0 || n_cols[i] % 128 != 0 || ldc[i] < n_cols[i] || ldc[i] % 2 != 0) return Q40_E_SHAPE;
    if (!q40_aligned(bw[i], 16) || !q40_aligned(bs[i], 4) || !q40_aligned(c[i], 4)) return Q40_E_ALIGN;
    tiles += n_cols[i] / TC_TILE_N;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int kblocks = K / TC_BK;
  const __half* ah = (const __half*)a;
  for (int m0 = 0; m0 < M; m0 += 256) {
    const int mc = (M - m0) < 256 ? (M - m0) : 256;
    TcParams p{};
    p.a = ah + (int64_t)m0 * lda; p.lda = lda;
    p.nprob = nmat;
    for (int i = 0; i < nmat; ++i) {
      p.bw[i] = (const uint8_t*)bw[i]; p.bs[i] = (const __half*)bs[i];
      p.c[i] = (__half*)c[i] + (int64_t)m0 * ldc[i]; p.ldc[i] = ldc[i];
      p.N[i] = n_cols[i]; p.tiles[i] = n_cols[i] / TC_TILE_N;
    }
    p.M = mc; p.K = K; p.Mpad = (mc + 15) / 16 * 16;
    p.err = err;
#ifdef Q40_TRACE
    p.trace = q40_trace_ptr;
#endif
    const int groups = tc_groups_for(p.Mpad);
    size_t smem = (size_t)groups * TC_A_BYTES + (size_t)(2 * groups) * p.Mpad * 128;
    const size_t tile_f = (size_t)p.Mpad * TC_TILE_N * 4;          // fp32 tile of the epilogue, same region
    smem += (size_t)groups * 2 * (4096 + TC_THREADS / groups * 4);
    if (tile_f > smem) smem = tile_f;
    smem += 1024 /* alignment slack */ + 128 /* barriers + tmem slot */;
    TcKernel kern = tc_kernel_for(p.Mpad);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    // split K over a cluster (<= 8): as many CTAs as the device holds at once (one per SM; the runtime
    // is asked, because clusters cannot straddle GPCs), each with at least 4 k blocks; the last split
    // may be shorter
    int nsplit = 8, bps = 0;
    for (; nsplit >= 1; nsplit >>= 1) {
      bps = (kblocks + nsplit - 1) / nsplit;
      if (nsplit > 1 && (bps < 4 || (nsplit - 1) * bps >= kblocks)) continue;
      if (nsplit == 1) break;
      const int fit = tc_max_clusters(kern, p.Mpad, nsplit, smem);
      if (fit >= tiles) break;
    }
    if (nsplit < 1) { nsplit = 1; bps = kblocks; }
    p.rows_per_split = bps * TC_BK;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(tiles, nsplit, 1);
    cfg.blockDim = dim3(TC_BLOCK, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = nsplit;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return (int)e;
  }
  return Q40_OK;
}

extern "C" int q40_gemm_kn_tc(const void* a, int64_t lda, const void* bw, const void* bs, void* c,
                              int64_t ldc, int M, int N, int K, int* err, void* stream) {
  return q40_gemm_kn_tc_multi(1, a, lda, &bw, &bs, &c, &ldc, &N, M, K, err, 0, stream);
}
