// Q4_0 dequant-matmul for batches above 16 rows on the 5th-generation tensor cores, reading the
// TILED copy of the weights (the format of q40_gemv_tiled.cu: [span of 256 columns][16 k rows] steps of
// 2176 contiguous bytes), so that the decode step's wide path and its narrow path share one weight copy.
//
// Swap-AB as in q40_gemm_tc.cu: the 256 output features of a span are the M dimension of two
// tcgen05.mma accumulators (128 features each, in tensor memory), the batch rows the N dimension
// (padded to a multiple of 16, up to 128 per launch; wider batches go in row chunks).  What differs is how
// the operands arrive:
//   * one elected thread streams the weights: a 64-row k block of a span is 4 steps = 8704 contiguous
//     bytes = ONE cp.async.bulk into a ring stage, and the matching 64-wide slice of the activations is
//     ONE tiled TMA copy (cp.async.bulk.tensor.2d, 128-byte swizzle, rows beyond M zero-filled) into the
//     same stage; both complete on the stage's mbarrier.  The ring is up to 8 stages deep, so up to 200 KB
//     are in flight per SM (the cp.async version held one block per producer group in flight and was
//     bound by that);
//   * sixteen dequantiser warps (two sets that take the k blocks in turn) turn a stage's nibbles into the
//     reference's operand value fp16(code * scale) (triton_kernels.py:444-445) and write it as the A
//     operand straight into TENSOR MEMORY: the tiled format hands every lane the four A-fragment words of
//     mma.m16n8k16 (rows g and g + 8 at four consecutive k per word), and that is the register layout of
//     tcgen05.st.16x256b, so a warp stores two 16-row tiles x 64 k with two instructions and the
//     dequantised weights never touch shared memory (through shared memory they cost 64 KB of traffic per
//     k block, more than the operands themselves);
//   * four warps issue the tcgen05.mma (A from tensor memory, B from the stage): a k block is 2 x 4 MMAs of
//     128 x Mpad x 16, small enough that the issuing thread's fixed latencies (mbarrier test, fences, commit:
//     ~800 cycles per k block measured) matter, so each accumulator has two issuing warps that alternate k
//     blocks and hand over in order through shared memory (every accumulator sees its MMAs in k order:
//     results do not depend on which warp was faster).  A commit per warp arrives on the block's "MMAs done"
//     mbarrier, which frees both the stage and the A buffer.
// The k range is split over a thread-block cluster; partial accumulators meet through distributed
// shared memory (no global scratch).  Every mbarrier wait is bounded: on expiry the kernel records an
// error code, skips the remaining work, frees its tensor memory and returns.
//
// Replaces matmul_q40_kernel (triton_kernels.py:357-469) for M > 16 when the caller holds tiled weights.
#include <cooperative_groups.h>
#include <cuda.h>

#include <atomic>
#include <cstdio>

#include "q40_common.cuh"

namespace cg = cooperative_groups;

namespace q40 {
namespace ttc {

constexpr int DQ_WARPS = 16;                    // dequantiser warps: two sets of 8 that take the k blocks in turn
constexpr int DQ_WARP0 = 4;                     // warp 0: copies, warps 1..3 and 20: MMA issue,
constexpr int MMA_WARPS = 4;                    // warps 4..19: dequantise (aligned to the tensor-memory quadrants)
constexpr int THREADS = (DQ_WARP0 + DQ_WARPS + MMA_WARPS - 3) * 32;
constexpr int BK = 64;                          // k rows per pipeline stage
constexpr int SPAN = 256;                       // output features per CTA
constexpr int STEP_BYTES = 2048 + 128;
constexpr int RAW_BYTES = 4 * STEP_BYTES;       // 8704: a k block of a span in the tiled stream
constexpr int RAW_PAD = 9216;                   // next multiple of 1024 (the B tile wants that alignment)
constexpr int NA = 4;                           // A buffers (in tensor memory)
constexpr int MAX_STAGES = 8;                   // a multiple of NA: block i owns barrier i % MAX_STAGES
constexpr unsigned SPIN_LIMIT = 1u << 22;       // polls of ~50 ns each before giving up

struct Params {
  const uint8_t* bw[3];   // tiled streams of up to three matrices that share the activations
  __half* c[3];           // [M, ldc]
  int64_t ldc[3];
  int N[3], spans[3], nprob;
  int M, K, Mpad, rows_per_split, stages;
  int split_acc;          // Mpad <= 64: even and odd k blocks have accumulators of their own
  int* err;               // device word, set non-zero when a bounded wait expired
  void* trace;            // stage timestamps (trace builds only)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major operand with 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)(16 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;      // descriptor version of this architecture
  d |= (uint64_t)2 << 61;      // 128-byte swizzle
  return d;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if (it > 64) __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 2-D tiled copy: box {64 k, Mpad rows} at (k element x, row y); x * 2 bytes is a multiple of 128
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// fp16 pair (72 + code) -> fp16(code * scale), the reference's operand rounding: 72 + code and code
// are exact in fp16, the product rounds once
__device__ __forceinline__ uint32_t deq_pair(uint32_t a72, __half2 scale) {
  return h2_as_u32(__hmul2(__hsub2(u32_as_h2(a72), u32_as_h2(0x54805480u)), scale));
}

// Tensor memory (all 512 columns of the SM): accumulators of the two 128-feature halves at columns
// 0 and 128, A buffer ab of half hh at column 256 + 64 ab + 32 hh (64 k as 32 columns of fp16 pairs).
constexpr int ACC_COLS = 128;
constexpr int A_COL0 = 2 * ACC_COLS;

// 16 rows x 16 columns of 32 bits to tensor memory: lane (g, t) gives, per group of 8 columns, rows g and
// g + 8 at columns 2t and 2t + 1 — the accumulator-fragment layout of mma.m16n8, which is also how the
// tiled weight format hands out its words
__device__ __forceinline__ void st_16x256b_x4(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
// Per-role cycle stamps of k blocks 9 and 10 (trace builds only)
#ifdef Q40_TRACE
#define TTC_ROLE_DECL long long rc_[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define TTC_ROLE(i, blk, idx) do { if (lane == 0 && (blk) == 10) rc_[idx] = clock64(); if (lane == 0 && (blk) == 12 && (idx) == 0) rc_[7] = clock64(); } while (0)
#define TTC_ROLE_FLUSH(kind)                                                                        \
  do {                                                                                              \
    unsigned long long* tb_ = (unsigned long long*)(p.trace);                                       \
    if (lane == 0 && tb_ && nblk > 12) {                                                            \
      const unsigned long long slot_ = atomicAdd(tb_, 1ull);                                        \
      if (slot_ < tb_[1]) {                                                                         \
        unsigned long long* r_ = tb_ + 16 + slot_ * 10;                                             \
        r_[0] = (kind);                                                                             \
        r_[1] = (unsigned long long)blockIdx.x + (unsigned long long)gridDim.x * blockIdx.y;        \
        for (int i_ = 0; i_ < 8; ++i_) r_[2 + i_] = (unsigned long long)rc_[i_];                    \
      }                                                                                             \
    }                                                                                               \
  } while (0)
#else
#define TTC_ROLE_DECL
#define TTC_ROLE(i, blk, idx) do { } while (0)
#define TTC_ROLE_FLUSH(kind) do { } while (0)
#endif

// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_tiled_tc_kernel(const Params p, const __grid_constant__ CUtensorMap amap) {
  extern __shared__ unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int pi = 0, span = blockIdx.x;
  while (pi < p.nprob - 1 && span >= p.spans[pi]) { span -= p.spans[pi]; ++pi; }
  const int split = blockIdx.y;
  Q40_TRACE_DECL
  Q40_STAMP(0);
  const int kb = split * p.rows_per_split;
  const int ke = min(p.K, kb + p.rows_per_split);
  const int nblk = (ke - kb) / BK;                           // host guarantees >= 1 and exact
  const int S = p.stages;
  const uint32_t b_bytes = (uint32_t)p.Mpad * 128u;          // B tile: Mpad rows x 64 k x 2 B
  const uint32_t stage_bytes = RAW_PAD + b_bytes;

  // 1024-byte aligned carve-up: [ring stages: raw | B][barriers][tmem slot][failed flag]; the fp32 tile of the
  // epilogue reuses the ring
  const uint32_t raw0 = smem_u32(smem_raw);
  const uint32_t ring = (raw0 + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (ring - raw0);
  const size_t ring_bytes = max((size_t)S * stage_bytes, ((size_t)p.Mpad * SPAN + 64) * 4);
  const uint32_t bars = ring + (uint32_t)ring_bytes;
  // full[s]: the stage's copies have landed; mdone[i % MAX_STAGES]: the MMAs of block i are complete (its
  // stage and its A buffer may be refilled); afull[ab]: the A buffer is written; done: all MMAs complete
  const uint32_t bar_full = bars, bar_mdone = bars + 8 * MAX_STAGES, bar_afull = bars + 16 * MAX_STAGES;
  const uint32_t bar_done = bar_afull + 8 * NA;
  unsigned char* tail = gbase + ring_bytes + 16 * MAX_STAGES + 8 * NA + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail);
  volatile int* s_failed = reinterpret_cast<volatile int*>(tail + 8);
  volatile int* s_issued = reinterpret_cast<volatile int*>(tail + 16);     // [2] k blocks issued per accumulator

  if (tid == 0) {
    *s_failed = 0;
    s_issued[0] = 0;
    s_issued[1] = 0;
    for (int s = 0; s < MAX_STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_mdone + 8 * s, 2); }
    for (int s = 0; s < NA; ++s) mbar_init(bar_afull + 8 * s, DQ_WARPS / 2);
    mbar_init(bar_done, MMA_WARPS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  asm volatile("griddepcontrol.launch_dependents;");
  Q40_STAMP(1);

  bool failed = false;
  if (warp == 0) {
    // ================= the copy thread: weights and activations of block i into stage i % S =================
    if (lane == 0) {
      const int ksteps = p.K / 16;
      const uint8_t* src = p.bw[pi] + ((int64_t)span * ksteps + kb / 16) * STEP_BYTES;
      // the weights do not depend on the previous launch: the first stages are requested before this
      // launch waits for it (programmatic dependent launch), the activations after
      const int first = min(S, nblk);
      for (int i = 0; i < first; ++i) {
        mbar_expect_tx(bar_full + 8 * i, RAW_BYTES + b_bytes);
        bulk_g2s(ring + i * stage_bytes, src + (int64_t)i * RAW_BYTES, RAW_BYTES, bar_full + 8 * i);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < first; ++i)
        tma_2d(ring + i * stage_bytes + RAW_PAD, &amap, kb + i * BK, 0, bar_full + 8 * i);
      Q40_STAMP(2);
      TTC_ROLE_DECL
      for (int i = first; i < nblk; ++i) {
        const int s = i % S;
        TTC_ROLE(0, i, 0);
        if (!mbar_wait(bar_mdone + 8 * s, (uint32_t)(((i / S) - 1) & 1))) { failed = true; break; }
        TTC_ROLE(0, i, 1);
        mbar_expect_tx(bar_full + 8 * s, RAW_BYTES + b_bytes);
        bulk_g2s(ring + s * stage_bytes, src + (int64_t)i * RAW_BYTES, RAW_BYTES, bar_full + 8 * s);
        tma_2d(ring + s * stage_bytes + RAW_PAD, &amap, kb + i * BK, 0, bar_full + 8 * s);
        TTC_ROLE(0, i, 2);
      }
      TTC_ROLE_FLUSH(313);
      Q40_STAMP(3);
    }
    __syncwarp();
  } else if (warp < DQ_WARP0 || warp >= DQ_WARP0 + DQ_WARPS) {
    // ================= the four MMA warps: lane 0 issues, the warp stays converged =================
    // Per k block an issuing warp spends ~800 cycles on fixed latencies (mbarrier test, fences, commit) and
    // 60-120 per tcgen05.mma, whatever the tile size, so one thread cannot feed eight small MMAs per k block.
    // Warp (hh, set) issues the four k steps of feature half hh for the k blocks of its set (even or odd).
    // fp32 accumulation is not associative, and the result must not depend on which warp was faster, so every
    // accumulator has to see its MMAs in a fixed order.  Up to 64 padded batch rows tensor memory has room for
    // an accumulator per (half, set): each warp owns one and the epilogue adds even + odd.  Above, the two
    // warps of a half share one accumulator: a warp issues block i only after the other has published block
    // i - 1 in shared memory (tcgen05 fences around the hand-over), so their waits and commits overlap but not
    // their MMAs (about 10 % slower than issuing in arbitrary order).
    // The dequantisers' arrival on afull also covers the stage's copies, which they waited for.
    // instruction descriptor: D fp32, A and B fp16 and K-major, N = Mpad, M = 128
    const int mi = (warp < DQ_WARP0) ? warp - 1 : 3;
    const int hh = mi & 1, mset = mi >> 1;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(p.Mpad >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    TTC_ROLE_DECL
    for (int i = mset; i < nblk && !failed; i += 2) {
      const int s = i % S, ab = i % NA;
      TTC_ROLE(1, i, 0);
      if (!mbar_wait(bar_afull + 8 * ab, (uint32_t)((i / NA) & 1))) { failed = true; break; }
      TTC_ROLE(1, i, 1);
      int ok = 1;
      if (lane == 0 && !p.split_acc) {
        unsigned spins = 0;
        while (s_issued[hh] != i && ++spins < (SPIN_LIMIT << 4)) { }
        ok = s_issued[hh] == i;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { failed = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint64_t bd0 = kmajor_desc(ring + s * stage_bytes + RAW_PAD);
        const uint32_t a0 = tmem + A_COL0 + ab * 64 + hh * 32;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks)
          mma_ts(tmem + (p.split_acc ? (2 * hh + mset) * 64 : hh * ACC_COLS), a0 + ks * 8,
                 bd0 + (uint64_t)((ks * 32) >> 4), idesc, (i > (p.split_acc ? mset : 0) || ks > 0) ? 1u : 0u);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        s_issued[hh] = i + 1;
        TTC_ROLE(1, i, 3);
        commit(bar_mdone + 8 * s);                  // the stage and the A buffer may be refilled when the MMAs
      }                                             // of both accumulators are done
      TTC_ROLE(1, i, 6);
      __syncwarp();
    }
    if (lane == 0 && !failed) commit(bar_done);     // all of this thread's MMAs
    __syncwarp();
    if (warp == 1) TTC_ROLE_FLUSH(312);
  } else {
    // ================= dequantisers: a stage's nibbles -> A operand in tensor memory =================
    // A warp may touch only the 32 tensor-memory lanes of its quadrant (warp index mod 4) = 32 feature rows
    // of a half = two 16-row tiles of one 64-column group; the other warp of the quadrant serves the other
    // half.  Lane (g, t) holds, per 16-row tile and 16-row k step, rows g and g + 8 at k = 4t .. 4t + 3.
    const int quad = warp & 3, hh = ((warp - DQ_WARP0) >> 2) & 1, dset = (warp - DQ_WARP0) >> 3;
    const int q = 2 * hh + (quad >> 1);                       // 64-column group of the span
    const int t = lane & 3;
    const unsigned char* lane_w = gbase + (q * 32 + lane) * 16 + (quad & 1) * 8;     // words of tiles 2 (quad & 1), + 1
    const unsigned char* lane_s = gbase + 2048 + q * 32 + t * 8;
    TTC_ROLE_DECL
    for (int i = dset; i < nblk; i += 2) {                    // the set's k blocks
      const int s = i % S, ab = i % NA;
      TTC_ROLE(2, i, 0);
      if (!mbar_wait(bar_full + 8 * s, (uint32_t)((i / S) & 1))) { failed = true; break; }
      TTC_ROLE(2, i, 1);
      // the A buffer was last read by the MMAs of block i - NA
      if (i >= NA && !mbar_wait(bar_mdone + 8 * ((i - NA) % S), (uint32_t)(((i - NA) / S) & 1))) { failed = true; break; }
      TTC_ROLE(2, i, 2);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const size_t so = (size_t)s * stage_bytes;
      uint32_t r[2][16];
#pragma unroll
      for (int st = 0; st < 4; ++st) {
        const uint2 w = *reinterpret_cast<const uint2*>(lane_w + so + st * STEP_BYTES);
        const uint2 sc = *reinterpret_cast<const uint2*>(lane_s + so + st * STEP_BYTES);
        const __half2 s01 = u32_as_h2(sc.x), s23 = u32_as_h2(sc.y);     // scales of k = 4t, 4t+1 and 4t+2, 4t+3
        const uint32_t wds[2] = {w.x, w.y};
#pragma unroll
        for (int j2 = 0; j2 < 2; ++j2) {
          const uint32_t v = wds[j2];
          const uint32_t a0 = lop3_and_xor(v, 0x00F000F0u, 0x54805480u);        // row g,     k + 0, 1
          const uint32_t a1 = lop3_and_xor(v << 4, 0x00F000F0u, 0x54805480u);   // row g + 8, k + 0, 1
          const uint32_t a2 = lop3_and_xor(v >> 8, 0x00F000F0u, 0x54805480u);   // row g,     k + 2, 3
          const uint32_t a3 = lop3_and_xor(v >> 4, 0x00F000F0u, 0x54805480u);   // row g + 8, k + 2, 3
          r[j2][4 * st + 0] = deq_pair(a0, s01);      // row g,     column 8 st + 2t
          r[j2][4 * st + 1] = deq_pair(a2, s23);      // row g,     column 8 st + 2t + 1
          r[j2][4 * st + 2] = deq_pair(a1, s01);      // row g + 8, column 8 st + 2t
          r[j2][4 * st + 3] = deq_pair(a3, s23);      // row g + 8, column 8 st + 2t + 1
        }
      }
      const uint32_t ta = tmem + ((uint32_t)(32 * quad) << 16) + A_COL0 + ab * 64 + hh * 32;
      TTC_ROLE(2, i, 3);
      st_16x256b_x4(ta, r[0]);
      st_16x256b_x4(ta + (16u << 16), r[1]);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      TTC_ROLE(2, i, 4);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_afull + 8 * ab);
      TTC_ROLE(2, i, 5);
    }
    if (warp == DQ_WARP0) TTC_ROLE_FLUSH(311);
  }
  if (failed) *s_failed = 1;
  if (!failed && !mbar_wait(bar_done, 0)) *s_failed = 1;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncthreads();
  failed = *s_failed != 0;
  if (failed && tid == 0) atomicExch(p.err, 1);
  Q40_STAMP(4);

  // ---- accumulators -> fp32 tile [Mpad][256] in shared memory (over the ring, idle by now) -> split-K sum
  // over the cluster through distributed shared memory: rank r finishes the r-th slice of the (m, feature)
  // pairs, adding the ranks' tiles in rank order -> fp16 store ----
  float* tile_f = reinterpret_cast<float*>(gbase);
  if (!failed && warp >= DQ_WARP0 && warp < DQ_WARP0 + DQ_WARPS) {
    // TMEM lanes 32 quad .. + 31 of accumulator hh; the two sets take the 16-row chunks in turn
    const int quad = warp & 3, hh = ((warp - DQ_WARP0) >> 2) & 1, dset = (warp - DQ_WARP0) >> 3;
    const int feat = hh * 128 + 32 * quad + lane;     // MMA row = feature of the span
    const int nchunk = p.Mpad / 16;
    for (int ch = dset; ch < nchunk; ch += 2) {
      uint32_t r[16];
      const uint32_t lane_base = tmem + ((uint32_t)(32 * quad) << 16);
      if (p.split_acc) {
        // even blocks + odd blocks (the odd accumulator was never written when the k range is one block)
        uint32_t r2[16];
        ld16(lane_base + (2 * hh) * 64 + ch * 16, r);
        ld16(lane_base + (2 * hh + 1) * 64 + ch * 16, r2);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (nblk > 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        }
      } else {
        ld16(lane_base + hh * ACC_COLS + ch * 16, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) tile_f[(ch * 16 + j) * SPAN + feat] = __uint_as_float(r[j]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();
  Q40_STAMP(5);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(512));
  }
  const int nranks = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int total = p.M * SPAN;
  const int per = ((total / 4 + nranks - 1) / nranks) * 4;
  const int e0 = rank * per, e1 = min(total, e0 + per);
  if (!failed) {
    for (int e = e0 + tid * 4; e < e1; e += THREADS * 4) {
      float4 tt[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        tt[r] = (r < nranks) ? *reinterpret_cast<const float4*>(cluster.map_shared_rank(tile_f + e, r))
                             : make_float4(0.f, 0.f, 0.f, 0.f);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) { v.x += tt[r].x; v.y += tt[r].y; v.z += tt[r].z; v.w += tt[r].w; }
      const int m = e / SPAN, n = span * SPAN + e % SPAN;       // four features of one row
      __half2* dst = reinterpret_cast<__half2*>(p.c[pi] + (int64_t)m * p.ldc[pi] + n);
      dst[0] = __floats2half2_rn(v.x, v.y);
      dst[1] = __floats2half2_rn(v.z, v.w);
    }
  }
  Q40_STAMP(6);
  cluster.sync();       // every rank has read the tiles: shared memory may go away
  Q40_STAMP(7);
  Q40_TRACE_FLUSH(p.trace, 310);
}

}  // namespace ttc
}  // namespace q40

using TtcKernel = void (*)(const q40::ttc::Params, const CUtensorMap);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against the driver library)
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn ttc_encode_fn() {
  static std::atomic<void*> cached{nullptr};
  void* fn = cached.load(std::memory_order_acquire);
  if (fn) return (EncodeTiledFn)fn;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !fn) {
    (void)cudaGetLastError();
    return nullptr;
  }
  cached.store(fn, std::memory_order_release);
  return (EncodeTiledFn)fn;
}

// How many clusters of (1, nsplit) CTAs with this much dynamic shared memory run at once (cached per
// device, split and padded row class; 0 when the runtime cannot tell).
static int ttc_max_clusters(TtcKernel kern, int mpad, int nsplit, size_t smem) {
  static int cache_all[16][9][17] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) dev = 0;
  int (*cache)[17] = cache_all[dev];
  const int cls = mpad / 16;
  if (cache[nsplit][cls]) return cache[nsplit][cls] - 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1024, nsplit, 1);
  cfg.blockDim = dim3(q40::ttc::THREADS, 1, 1);
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
  cache[nsplit][cls] = n + 1;
  return n;
}

// C[M, N_i] = A[M, K] @ deq(B_i)[K, N_i] for 1..3 matrices given as TILED copies (q40_relayout_tiled),
// 16 < M, K % 64 == 0, N_i % 256 == 0, on tcgen05.  `err` is a device int the kernel sets to 1 if one of its
// bounded waits expires (results are then undefined); the caller zeroes it beforehand and may read it after
// synchronising.
extern "C" int q40_gemm_tiled_tc_multi(int nmat, const void* a, int64_t lda, const void* const* bw_tiled,
                                       void* const* c, const int64_t* ldc, const int* n_cols, int M, int K, int* err,
                                       int use_pdl, void* stream) {
  using namespace q40;
  using namespace q40::ttc;
  if (!a || !bw_tiled || !c || !ldc || !n_cols || !err) return Q40_E_NULL;
  if (nmat < 1 || nmat > 3) return Q40_E_UNSUPPORTED;
  if (M < 1 || K <= 0 || K % BK != 0 || lda < K || lda % 8 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(a, 16)) return Q40_E_ALIGN;
  int spans = 0;
  for (int i = 0; i < nmat; ++i) {
    if (!bw_tiled[i] || !c[i]) return Q40_E_NULL;
    if (n_cols[i] <= 0 || n_cols[i] % SPAN != 0 || ldc[i] < n_cols[i] || ldc[i] % 2 != 0) return Q40_E_SHAPE;
    if (!q40_aligned(bw_tiled[i], 16) || !q40_aligned(c[i], 4)) return Q40_E_ALIGN;
    spans += n_cols[i] / SPAN;
  }
  EncodeTiledFn encode = ttc_encode_fn();
  if (!encode) return Q40_E_UNSUPPORTED;
  int sms = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    return Q40_E_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const int kblocks = K / BK;
  const __half* ah = (const __half*)a;
  // the two accumulators hold 128 batch rows: wider batches go in chunks (the weights of the later chunks
  // come from L2 when the matrix fits there)
  for (int m0 = 0; m0 < M; m0 += ACC_COLS) {
    const int mc = (M - m0) < ACC_COLS ? (M - m0) : ACC_COLS;
    Params p{};
    p.nprob = nmat;
    for (int i = 0; i < nmat; ++i) {
      p.bw[i] = (const uint8_t*)bw_tiled[i];
      p.c[i] = (__half*)c[i] + (int64_t)m0 * ldc[i]; p.ldc[i] = ldc[i];
      p.N[i] = n_cols[i]; p.spans[i] = n_cols[i] / SPAN;
    }
    p.M = mc; p.K = K; p.Mpad = (mc + 15) / 16 * 16;
    p.split_acc = p.Mpad <= 64 ? 1 : 0;
    p.err = err;
#ifdef Q40_TRACE
    p.trace = q40_trace_ptr;
#endif
    // activations [mc rows, K] as a 2-D tensor, box {64 k, Mpad rows}, 128-byte swizzle, zero fill beyond row mc
    CUtensorMap amap;
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)mc};
    const cuuint64_t gstride[1] = {(cuuint64_t)lda * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)p.Mpad};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(&amap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)(ah + (int64_t)m0 * lda), gdim, gstride, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return Q40_E_UNSUPPORTED;
    // ring depth: what fits, at most MAX_STAGES; the fp32 tile of the epilogue reuses the ring
    const size_t stage_bytes = (size_t)RAW_PAD + (size_t)p.Mpad * 128;
    const size_t fixed = 1024 /* alignment slack */ + 256 /* barriers, tmem slot, flag */;
    int stages = (int)((227 * 1024 - fixed) / stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) return Q40_E_UNSUPPORTED;
    p.stages = stages;
    size_t ring_bytes = (size_t)stages * stage_bytes;
    const size_t tile_f = ((size_t)p.Mpad * SPAN + 64) * 4;     // slices are rounded up to 4 elements per rank
    if (tile_f > ring_bytes) ring_bytes = tile_f;
    const size_t smem = fixed + ring_bytes;
    TtcKernel kern = gemm_tiled_tc_kernel;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return Q40_E_UNSUPPORTED; }
    // split K over a cluster (<= 8 ranks, each with at least 4 k blocks): the split that minimises
    // waves x (k blocks per rank + a fixed cost of about 10 k blocks for allocation and epilogue)
    int best = 1;
    double best_cost = 1e30;
    for (int ns = 1; ns <= 8; ++ns) {
      const int bps = (kblocks + ns - 1) / ns;
      if (ns > 1 && (bps < 4 || (ns - 1) * bps >= kblocks)) continue;
      int fit = sms / ns;
      if (ns > 1) {
        fit = ttc_max_clusters(kern, p.Mpad, ns, smem);
        if (fit < 1) continue;
      }
      const int waves = (spans + fit - 1) / fit;
      const double cost = (double)waves * (bps + 10.0 + 1.5 * ns);
      if (cost < best_cost) { best_cost = cost; best = ns; }
    }
    const int nsplit = best, bps = (kblocks + nsplit - 1) / nsplit;
    p.rows_per_split = bps * BK;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(spans, nsplit, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
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
    e = cudaLaunchKernelEx(&cfg, kern, p, amap);
    if (e != cudaSuccess) return (int)e;
  }
  return Q40_OK;
}
