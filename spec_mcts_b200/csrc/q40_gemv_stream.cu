// Decode-step Q4_0 matmul as one byte-balanced wave: every launch has one CTA per SM (at most), and
// each CTA owns an equal, contiguous share of the launch's weight bytes.
//
// The weights are read in the "tiled" format of q40_gemv_tiled.cu (q40_relayout_tiled): a matrix is a
// sequence of steps [span of 256 output columns][16 k rows], 2176 bytes each, contiguous in memory.
// All steps of all matrices of a launch form one sequence of T steps (stream-K); CTA c of G takes steps
// [c*T/G, (c+1)*T/G).  Inside a CTA
//   * one elected thread of a producer warp moves its share through a ring of shared-memory slots with
//     1-D bulk copies (cp.async.bulk, 4 steps = 8704 bytes per copy) that signal an mbarrier per slot;
//     it starts before griddepcontrol.wait, so under programmatic dependent launch a CTA that becomes
//     resident while the previous launch still runs has its ring full when its activations arrive;
//   * eight consumer warps wait for a slot, each takes one of its four steps and two of the four
//     64-column groups, and runs the same arithmetic as the tiled kernel: codes expanded to fp16
//     (72 + code) with mask operations, B operand fp16(scale * x), mma.m16n8k16 with fp32 accumulators,
//     the constant 72 removed by one extra MMA per group against an all-ones tile;
//   * where the CTA's share crosses from one span to the next (and at its end) the warps' partial sums
//     are added in shared memory and written to a scratch area in global memory; the CTA that arrives
//     last at a span's counter adds the partials of that span in CTA order (so the result does not
//     depend on timing), applies the epilogue and stores the outputs.  No CTA waits for another one.
// Prologue / epilogue modes as in q40_gemv_tiled: RMSNorm prologue (with the reference's rounding points:
// fp32 normalisation, rounded to fp16, times the fp16 norm weight), residual add + sum of squares for
// the next norm, SiLU-mul of a (w1, w3) pair.
#include "q40_common.cuh"

namespace q40 {
namespace stream {

constexpr int STEP_BYTES = 2048 + 128;
constexpr int SLOT_STEPS = 4;
constexpr int SLOT_BYTES = SLOT_STEPS * STEP_BYTES;
constexpr int CONS_WARPS = 8;
constexpr int CONS_THREADS = CONS_WARPS * 32;
constexpr int THREADS = CONS_THREADS + 32;
constexpr int SPAN_COLS = 256;
constexpr int HEADER_BYTES = 4096;          // workspace: [status][pad ..][unit counters from byte 64]
constexpr int MAX_UNITS = (HEADER_BYTES - 64) / 4;
constexpr long long WAIT_LIMIT = 1ll << 31;  // cycles a wait may take before the kernel gives up (about a second)

enum { PRO_NONE = 0, PRO_NORM = 1 };
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU = 2 };
enum { ERR_FULL_WAIT = 1, ERR_EMPTY_WAIT = 2 };

struct Mat {
  const uint8_t* bw;   // tiled stream [N/256][K/16][STEP_BYTES]
  __half* out;
  int nspans;
};

struct Params {
  Mat mat[3];
  int nmat;
  const __half* a;
  int64_t lda, ldc;
  int M, K, ksteps, total_steps, nseg_max;
  const __half* norm_w;
  const float* ss_in;
  int ss_in_count;
  float eps;
  const __half* h_in;
  int64_t ldh;
  float* ss_out;
  int ss_out_count;
  float* scratch;      // [G][nseg_max][M][256] partial sums
  int* counters;       // one per span (per span pair for the SiLU epilogue), zero between launches
  int* status;
  void* trace;         // stage timestamps (trace builds only)
  int ring_slots;
  int xs_ld;           // halfs per activation row in shared memory
  int off_bar, off_misc, off_xs, off_slab;
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on the slot's mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(CONS_THREADS) : "memory"); }

// Bounded wait: gives up after WAIT_LIMIT cycles, records why, and makes every later wait of the CTA
// return at once (all warps keep walking the same control flow, so no barrier is left short of threads;
// the outputs of that launch are then undefined and the status word says so).
__device__ __forceinline__ void wait_slot(uint32_t bar, uint32_t parity, volatile int* s_abort, int* status, int code) {
  if (*s_abort) return;
  if (mbar_try_wait(bar, parity)) return;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*s_abort) return;
    if (clock64() - t0 > WAIT_LIMIT) {
      *s_abort = 1;
      atomicExch(status, code);
      return;
    }
  }
}

// share of CTA c: steps [c*T/G, (c+1)*T/G); T * G < 2^31 is checked on the host
__device__ __forceinline__ uint32_t cta_begin(int c, int T, int G) { return (uint32_t)c * (uint32_t)T / (uint32_t)G; }
// the CTA whose share contains step s
__device__ __forceinline__ int cta_of(uint32_t s, int T, int G) { return (int)(((s + 1u) * (uint32_t)G - 1u) / (uint32_t)T); }

template <int EPI>
__device__ __forceinline__ void span_to_mat(const Params& p, int span, int& pi, int& lspan) {
  if (EPI == EPI_SILU) {
    pi = span & 1;
    lspan = span >> 1;
  } else {
    pi = 0;
    lspan = span;
    while (pi < p.nmat - 1 && lspan >= p.mat[pi].nspans) { lspan -= p.mat[pi].nspans; ++pi; }
  }
}

template <int MT, int PRO, int EPI>
__global__ void __launch_bounds__(THREADS, MT == 1 ? 2 : 1) gemv_stream_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x, c = blockIdx.x, T = p.total_steps, ksteps = p.ksteps, R = p.ring_slots;
  const int g0 = (int)cta_begin(c, T, G), g1 = (int)cta_begin(c + 1, T, G);
  const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t full_u32 = ring_u32 + p.off_bar, empty_u32 = full_u32 + 8 * R;
  float* s_inv = reinterpret_cast<float*>(smem + p.off_misc);            // [16] 1/rms per row
  float* s_red = s_inv + 16;                                             // [16][8] sum-of-squares partials
  volatile int* s_flag = reinterpret_cast<volatile int*>(s_red + 128);   // [0] abort
  volatile int* s_last = s_flag + 4;                                     // [nseg_max] this CTA arrived last
  __half* xs = reinterpret_cast<__half*>(smem + p.off_xs);
  float* slab = reinterpret_cast<float*>(smem + p.off_slab);             // [2][4 k slices][M][256]
  Q40_TRACE_DECL
  Q40_STAMP(0);

  if (tid == 0) {
    for (int i = 0; i < R; ++i) {
      mbar_init(full_u32 + 8 * i, 1);
      mbar_init(empty_u32 + 8 * i, CONS_WARPS);
    }
    s_flag[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;");

  if (warp == CONS_WARPS) {
    // ---- producer: weights only, nothing here depends on the previous launch ----
    if (lane == 0) {
#ifdef Q40_TRACE
      unsigned long long pw_ = 0, pt0_ = 0, pt1_ = 0;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(pt0_)::"memory");
#endif
      int cur = g0, it = 0, span = g0 / ksteps, kstep = g0 % ksteps;
      while (cur < g1) {
        const int n = min(SLOT_STEPS, min(ksteps - kstep, g1 - cur));
        const int slot = it % R;
#ifdef Q40_TRACE
        const long long pe0_ = clock64();
#endif
        if (it >= R) wait_slot(empty_u32 + 8 * slot, ((it / R) - 1) & 1, s_flag, p.status, ERR_EMPTY_WAIT);
#ifdef Q40_TRACE
        pw_ += (unsigned long long)(clock64() - pe0_);
#endif
        if (s_flag[0]) break;
        int pi, lspan;
        span_to_mat<EPI>(p, span, pi, lspan);
        const uint8_t* src = p.mat[pi].bw + ((int64_t)lspan * ksteps + kstep) * STEP_BYTES;
        const uint32_t bytes = (uint32_t)n * STEP_BYTES;
        mbar_arrive_expect_tx(full_u32 + 8 * slot, bytes);
        bulk_g2s(ring_u32 + slot * SLOT_BYTES, src, bytes, full_u32 + 8 * slot);
        cur += n;
        kstep += n;
        if (kstep == ksteps) { kstep = 0; ++span; }
        ++it;
      }
#ifdef Q40_TRACE
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(pt1_)::"memory");
      unsigned long long* tb_ = (unsigned long long*)p.trace;
      if (tb_) {
        const unsigned long long sl_ = atomicAdd(tb_, 1ull);
        if (sl_ < tb_[1]) {
          unsigned long long* r_ = tb_ + 16 + sl_ * 10;
          r_[0] = 450 + 10 * PRO + EPI; r_[1] = blockIdx.x; r_[2] = pt0_; r_[3] = pw_; r_[4] = (unsigned long long)it;
          r_[5] = (unsigned long long)R; r_[6] = pt1_; r_[7] = 0; r_[8] = 0; r_[9] = 0;
        }
      }
#endif
    }
    return;
  }

  // ---- consumers ----
  const int g = lane >> 2, t = lane & 3;
  const int ks = warp >> 1, half = warp & 1;       // step of the slot, pair of column groups
  asm volatile("griddepcontrol.wait;" ::: "memory");
  Q40_STAMP(2);

  const int nst = g1 - g0;
  // activations of the CTA's steps, in the order the steps are consumed: xs[m][local step][16].
  // RMSNorm prologue with the reference's rounding points: fp16(fp16(float(a) * 1/rms) * norm_w).
  const int nchunks = p.M * nst * 2;
  auto chunk_src = [&](int idx, int& m, int& k, int& dst) {
    m = idx / (nst * 2);
    const int r = idx % (nst * 2), i = r >> 1, hf = r & 1;
    k = ((g0 + i) % ksteps) * 16 + hf * 8;
    dst = m * p.xs_ld + i * 16 + hf * 8;
  };
  auto chunk_store = [&](uint4 v, int m, int k, int dst) {
    if (PRO == PRO_NORM) {
      const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + k);
      const float inv = s_inv[m];
      __half2* vh = reinterpret_cast<__half2*>(&v);
      const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(vh[j]);
        vh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);
      }
    }
    *reinterpret_cast<uint4*>(xs + dst) = v;
  };
  // the first chunk of every thread is requested before the row statistics are summed
  uint4 v_first = make_uint4(0u, 0u, 0u, 0u);
  int m_first = 0, k_first = 0, d_first = 0;
  if (tid < nchunks) {
    chunk_src(tid, m_first, k_first, d_first);
    v_first = *reinterpret_cast<const uint4*>(p.a + (int64_t)m_first * p.lda + k_first);
  }
  if (PRO == PRO_NORM) {
    for (int m = warp; m < p.M; m += CONS_WARPS) {
      float s = 0.f;
      for (int i = lane; i < p.ss_in_count; i += 32) s += __ldcg(p.ss_in + (int64_t)m * p.ss_in_count + i);
      s = warp_sum(s);
      if (lane == 0) s_inv[m] = rsqrtf(s / (float)p.K + p.eps);
    }
    bar_consumers();
  }
  if (tid < nchunks) chunk_store(v_first, m_first, k_first, d_first);
  for (int idx = tid + CONS_THREADS; idx < nchunks; idx += CONS_THREADS) {
    int m, k, dst;
    chunk_src(idx, m, k, dst);
    chunk_store(*reinterpret_cast<const uint4*>(p.a + (int64_t)m * p.lda + k), m, k, dst);
  }
  bar_consumers();
#ifdef Q40_TRACE
  if (threadIdx.x == 0) q40_ts_[3] = 0;     // words 1 and 3 of a trace record: cycles spent waiting for slots / in span flushes
#endif

  float acc[MT][8][4];
  // per 64-column group: this lane's part of sum_k scale * x for batch row g (its four k rows of every step);
  // 72 times the full sum is what the weight operands' constant adds to every column of the group
  float ysum[MT][2];
  auto zero_acc = [&]() {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[mt][i][j] = 0.f;
#pragma unroll
      for (int q = 0; q < 2; ++q) ysum[mt][q] = 0.f;
    }
  };
  zero_acc();

  int cur = g0, it = 0, seg = 0, span = g0 / ksteps, kstep = g0 % ksteps;
  while (cur < g1) {
    const int n = min(SLOT_STEPS, min(ksteps - kstep, g1 - cur));
    const int slot = it % R;
#ifdef Q40_TRACE
    const long long tw0_ = clock64();
#endif
    wait_slot(full_u32 + 8 * slot, (it / R) & 1, s_flag, p.status, ERR_FULL_WAIT);
#ifdef Q40_TRACE
    if (threadIdx.x == 0) q40_ts_[1] += (unsigned long long)(clock64() - tw0_);
#endif
#ifdef Q40_TRACE
    const long long tc0_ = clock64();
#endif
    if (ks < n) {
      const unsigned char* sb = smem + slot * SLOT_BYTES + ks * STEP_BYTES;
      const int li = cur - g0 + ks;
      uint2 xv[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int row = mt * 8 + g;
        xv[mt] = (row < p.M) ? *reinterpret_cast<const uint2*>(xs + (int64_t)row * p.xs_ld + li * 16 + 4 * t)
                             : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int grp = half * 2 + q;
        const uint4 w = *reinterpret_cast<const uint4*>(sb + (grp * 32 + lane) * 16);
        const uint2 sc = *reinterpret_cast<const uint2*>(sb + 2048 + grp * 32 + t * 8);
        uint32_t yb[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          yb[mt][0] = h2_as_u32(__hmul2(u32_as_h2(xv[mt].x), u32_as_h2(sc.x)));   // scale * x, k rows 4t, 4t+1
          yb[mt][1] = h2_as_u32(__hmul2(u32_as_h2(xv[mt].y), u32_as_h2(sc.y)));   // k rows 4t+2, 4t+3
          const float2 f0 = __half22float2(u32_as_h2(yb[mt][0])), f1 = __half22float2(u32_as_h2(yb[mt][1]));
          ysum[mt][q] += (f0.x + f0.y) + (f1.x + f1.y);
        }
        const uint32_t wds[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int jt = 0; jt < 4; ++jt) {
          const uint32_t v = wds[jt];
          // nibble -> fp16 value 72 + code (see q40_gemv_tiled.cu)
          const uint32_t a0 = lop3_and_xor(v, 0x00F000F0u, 0x54805480u);
          const uint32_t a1 = lop3_and_xor(v << 4, 0x00F000F0u, 0x54805480u);
          const uint32_t a2 = lop3_and_xor(v >> 8, 0x00F000F0u, 0x54805480u);
          const uint32_t a3 = lop3_and_xor(v >> 4, 0x00F000F0u, 0x54805480u);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma16816(acc[mt][q * 4 + jt], a0, a1, a2, a3, yb[mt][0], yb[mt][1]);
        }
      }
    }
#ifdef Q40_TRACE
    const long long tc1_ = clock64();
    if (threadIdx.x == 0) q40_ts_[4] += (unsigned long long)(tc1_ - tc0_);
#endif
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_u32 + 8 * slot);
    cur += n;
    kstep += n;
    ++it;
#ifdef Q40_TRACE
    if (threadIdx.x == 0) q40_ts_[6] += (unsigned long long)(clock64() - tc1_);
#endif
    if (kstep != ksteps && cur != g1) continue;

    // ---- the CTA's share of this span is complete: add the warps' sums in shared memory and store
    // the CTA's partial for the span; nothing waits here for global memory ----
    {
#ifdef Q40_TRACE
      const long long tf0_ = clock64();
#endif
      // double-buffered up to 8 rows (one barrier per span); above, one buffer and a second barrier
      float* sl = slab + ((MT == 1) ? (seg & 1) * (4 * p.M * SPAN_COLS) : 0);
      // the accumulator fragment of a lane holds batch rows 2t, 2t+1; their sums of scale * x sit, split over
      // the four lanes of a quad, in the lanes whose g is that batch row
      float corr[MT][2][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          float v = ysum[mt][q];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          corr[mt][q][0] = __shfl_sync(0xffffffffu, v, (2 * t) * 4);
          corr[mt][q][1] = __shfl_sync(0xffffffffu, v, (2 * t + 1) * 4);
        }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int col = (half * 2 + (i >> 2)) * 64 + (i & 3) * 16 + g;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int m = mt * 8 + 2 * t + (j & 1);
            if (m < p.M)
              sl[(ks * p.M + m) * SPAN_COLS + col + 8 * (j >> 1)] = fmaf(-72.0f, corr[mt][i >> 2][j & 1], acc[mt][i][j]);
          }
        }
      zero_acc();
      bar_consumers();
      float* part = p.scratch + ((int64_t)c * p.nseg_max + seg) * p.M * SPAN_COLS;
      for (int m = 0; m < p.M; ++m) {
        float v = 0.f;
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) v += sl[(s4 * p.M + m) * SPAN_COLS + tid];
        part[m * SPAN_COLS + tid] = v;
      }
      if (MT != 1) bar_consumers();
#ifdef Q40_TRACE
      if (threadIdx.x == 0) q40_ts_[3] += (unsigned long long)(clock64() - tf0_);
#endif
    }
    ++seg;
    ++span;
    kstep = 0;
  }
  Q40_STAMP(5);

  // ---- all partials of this CTA are on their way: publish them, arrive at the counter of every unit
  // (span, or (w1, w3) span pair) this CTA contributed to, and finish the units where it arrived last ----
  const int nseg = seg, span0 = g0 / ksteps;
  constexpr int nsp = (EPI == EPI_SILU) ? 2 : 1;
  __threadfence();
  bar_consumers();
  if (tid < nseg) {
    const int sp = span0 + tid;
    const int unit = (EPI == EPI_SILU) ? (sp >> 1) : sp;
    int expected = 0;
    for (int s2 = 0; s2 < nsp; ++s2) {
      const uint32_t b = (uint32_t)(unit * nsp + s2) * (uint32_t)ksteps;
      expected += cta_of(b + ksteps - 1, T, G) - cta_of(b, T, G) + 1;
    }
    const int old = atomicAdd(p.counters + unit, 1);
    s_last[tid] = (old == expected - 1) ? 1 : 0;
  }
  bar_consumers();
  for (int sg = 0; sg < nseg; ++sg) {
    if (!s_last[sg]) continue;
    __threadfence();
    const int unit = (EPI == EPI_SILU) ? ((span0 + sg) >> 1) : (span0 + sg);
    const int first_span = unit * nsp;
    int pi, lspan;
    span_to_mat<EPI>(p, first_span, pi, lspan);
    const int ncol = lspan * SPAN_COLS + tid;
    // partial (cc, segment) of span sp lives at scratch[(cc * nseg_max + sp - first span of cc)][m][col]
    int c_lo[nsp], c_n[nsp], seg_lo[nsp];
#pragma unroll
    for (int s2 = 0; s2 < nsp; ++s2) {
      const uint32_t b = (uint32_t)(first_span + s2) * (uint32_t)ksteps;
      c_lo[s2] = cta_of(b, T, G);
      c_n[s2] = cta_of(b + ksteps - 1, T, G) - c_lo[s2] + 1;
      seg_lo[s2] = (first_span + s2) - (int)(cta_begin(c_lo[s2], T, G) / (uint32_t)ksteps);
    }
    for (int m = 0; m < p.M; ++m) {
      float v[2] = {0.f, 0.f};
#pragma unroll
      for (int s2 = 0; s2 < nsp; ++s2) {
        // the first contributor holds the span as its segment seg_lo, every later one as its segment 0
        const float* base = p.scratch + ((int64_t)m * SPAN_COLS + tid);
        const int64_t seg_stride = (int64_t)p.M * SPAN_COLS;
        float sum = 0.f;
        for (int j0 = 0; j0 < c_n[s2]; j0 += 8) {
          float part8[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int jj = j0 + j;
            const int64_t segi = (int64_t)(c_lo[s2] + jj) * p.nseg_max + (jj == 0 ? seg_lo[s2] : 0);
            part8[j] = (jj < c_n[s2]) ? __ldcg(base + segi * seg_stride) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) sum += part8[j];
        }
        v[s2] = sum;
      }
      if (EPI == EPI_STORE) {
        p.mat[pi].out[(int64_t)m * p.ldc + ncol] = __float2half_rn(v[0]);
      } else if (EPI == EPI_RESIDUAL) {
        const __half hn = __hadd_rn(p.h_in[(int64_t)m * p.ldh + ncol], __float2half_rn(v[0]));
        p.mat[0].out[(int64_t)m * p.ldc + ncol] = hn;
        const float f = __half2float(hn);
        const float sq = warp_sum(f * f);
        if (lane == 0) s_red[m * 8 + warp] = sq;
      } else {
        const float a1 = __half2float(__float2half_rn(v[0]));
        const __half sil = __float2half_rn(a1 / (1.0f + expf(-a1)));
        p.mat[0].out[(int64_t)m * p.ldc + ncol] = __hmul_rn(sil, __float2half_rn(v[1]));
      }
    }
    if (EPI == EPI_RESIDUAL) {
      bar_consumers();
      if (tid < p.M) {
        float s8 = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s8 += s_red[tid * 8 + w];
        p.ss_out[(int64_t)tid * p.ss_out_count + first_span] = s8;
      }
      bar_consumers();     // s_red is reused by the next unit this CTA finishes
    }
    if (tid == 0) p.counters[unit] = 0;      // ready for the next launch that uses this workspace
  }
  Q40_STAMP(7);
  Q40_TRACE_FLUSH(p.trace, 400 + 10 * PRO + EPI);
}

static int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

struct Plan {
  int G, T, ksteps, nseg_max, units;
  size_t scratch_bytes;
};

static Plan make_plan(int M, int total_spans, int K, bool pairs, int sms) {
  Plan pl{};
  pl.ksteps = K / 16;
  pl.T = total_spans * pl.ksteps;
  pl.G = pl.T < sms ? pl.T : sms;
  if (pl.G < 1) pl.G = 1;
  const int per = (pl.T + pl.G - 1) / pl.G;
  pl.nseg_max = (per + pl.ksteps - 1) / pl.ksteps + 1;
  pl.units = pairs ? total_spans / 2 : total_spans;
  pl.scratch_bytes = (size_t)pl.G * pl.nseg_max * M * SPAN_COLS * sizeof(float);
  return pl;
}

template <int MT, int PRO, int EPI>
static int launch(Params& p, const Plan& pl, int smem_budget, cudaStream_t st, bool pdl) {
  auto kern = gemv_stream_kernel<MT, PRO, EPI>;
  const int per = (pl.T + pl.G - 1) / pl.G;
  // shared memory: ring | barriers | 1/rms, sum-of-squares partials, flags | activations | slab
  const int xs_rows = p.M;
  int xs_ld = per * 16;
  xs_ld = (xs_ld + 63) / 64 * 64 + 16;
  const size_t xs_bytes = (size_t)xs_rows * xs_ld * 2;
  const size_t slab_bytes = (size_t)(MT == 1 ? 2 : 1) * 4 * p.M * SPAN_COLS * 4;
  const size_t misc_bytes = 16 * 4 + 128 * 4 + 16 + (size_t)((pl.nseg_max + 3) / 4 * 4) * 4;
  if (pl.nseg_max > CONS_THREADS) return Q40_E_UNSUPPORTED;
  const int slots_needed = (per + SLOT_STEPS - 1) / SLOT_STEPS + pl.nseg_max;
  long long room = (long long)smem_budget - (long long)(xs_bytes + slab_bytes + misc_bytes + 1024);
  int R = (int)(room / (SLOT_BYTES + 16));
  if (R > slots_needed) R = slots_needed;
  if (R < 2) return Q40_E_UNSUPPORTED;
  size_t off = (size_t)R * SLOT_BYTES;
  p.off_bar = (int)off;
  off += (size_t)R * 16;
  off = (off + 15) / 16 * 16;
  p.off_misc = (int)off;
  off += misc_bytes;
  off = (off + 15) / 16 * 16;
  p.off_xs = (int)off;
  off += xs_bytes;
  off = (off + 15) / 16 * 16;
  p.off_slab = (int)off;
  off += slab_bytes;
  p.ring_slots = R;
  p.xs_ld = xs_ld;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)off);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return Q40_E_UNSUPPORTED;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.G, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = off;
  cfg.stream = st;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = pdl ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}

}  // namespace stream
}  // namespace q40

// Bytes of workspace q40_gemv_stream needs for M rows, total_cols output columns (summed over the
// matrices of the launch) and K input features.  Zero-fill it once; the kernels leave the counters zeroed.
extern "C" size_t q40_gemv_stream_workspace_bytes(int M, int total_cols, int K) {
  using namespace q40::stream;
  if (M < 1 || M > 16 || total_cols <= 0 || total_cols % SPAN_COLS != 0 || K < 16 || K % 16 != 0) return 0;
  const int sms = sm_count();
  if (sms <= 0) return 0;
  const Plan pl = make_plan(M, total_cols / SPAN_COLS, K, false, sms);
  return HEADER_BYTES + pl.scratch_bytes;
}

extern "C" int q40_gemv_stream(int mode, int nmat, const void* const* bw_tiled, void* const* out, const int* n_cols,
                               int64_t ldc, const void* a, int64_t lda, int M, int K, const void* norm_w,
                               const float* ss_in, int ss_in_count, float eps, const void* h_in, int64_t ldh,
                               float* ss_out, int ss_out_count, void* workspace, size_t workspace_bytes,
                               int smem_budget, int use_pdl, void* stream) {
  using namespace q40;
  using namespace q40::stream;
  if (!bw_tiled || !out || !n_cols || !a || !workspace) return Q40_E_NULL;
  if (mode < 0 || mode > 3 || nmat < 1 || nmat > 3) return Q40_E_UNSUPPORTED;
  if (mode == 3 && nmat != 2) return Q40_E_UNSUPPORTED;
  if (mode == 2 && nmat != 1) return Q40_E_UNSUPPORTED;
  if (M < 1 || M > 16 || K < 16 || K % 16 != 0 || lda < K || lda % 8 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(a, 16) || !q40_aligned(workspace, 16)) return Q40_E_ALIGN;
  if ((mode == 1 || mode == 3) && (!norm_w || !ss_in || ss_in_count < 1 || !q40_aligned(norm_w, 16)))
    return Q40_E_NULL;
  if (mode == 2 && (!h_in || !ss_out)) return Q40_E_NULL;
  Params p{};
  int total_spans = 0;
  for (int i = 0; i < nmat; ++i) {
    if (!bw_tiled[i] || !out[i]) return Q40_E_NULL;
    if (n_cols[i] <= 0 || n_cols[i] % SPAN_COLS != 0 || ldc < n_cols[i]) return Q40_E_SHAPE;
    if (!q40_aligned(bw_tiled[i], 16)) return Q40_E_ALIGN;
    p.mat[i].bw = (const uint8_t*)bw_tiled[i];
    p.mat[i].out = (__half*)out[i];
    p.mat[i].nspans = n_cols[i] / SPAN_COLS;
    total_spans += p.mat[i].nspans;
  }
  if (mode == 3 && n_cols[0] != n_cols[1]) return Q40_E_SHAPE;
  const int sms = sm_count();
  if (sms <= 0) return Q40_E_UNSUPPORTED;
  const Plan pl = make_plan(M, total_spans, K, mode == 3, sms);
  if (pl.units > MAX_UNITS || (int64_t)(pl.T + 1) * pl.G >= (1ll << 31)) return Q40_E_UNSUPPORTED;
  if (workspace_bytes < HEADER_BYTES + pl.scratch_bytes) return Q40_E_WORKSPACE;
  if (mode == 2 && ss_out_count != total_spans) return Q40_E_SHAPE;
  // default: up to 4 rows leave room for the CTA of the next launch on the same SM; wider batches need
  // the space for their activations and partial sums
  if (smem_budget <= 0) smem_budget = (M <= 4 ? 100 : 200) * 1024;
  if (smem_budget > 220 * 1024) smem_budget = 220 * 1024;
  p.nmat = nmat;
  p.a = (const __half*)a; p.lda = lda; p.ldc = ldc; p.M = M; p.K = K;
  p.ksteps = pl.ksteps; p.total_steps = pl.T; p.nseg_max = pl.nseg_max;
  p.norm_w = (const __half*)norm_w; p.ss_in = ss_in; p.ss_in_count = ss_in_count; p.eps = eps;
  p.h_in = (const __half*)h_in; p.ldh = ldh; p.ss_out = ss_out; p.ss_out_count = ss_out_count;
  p.status = (int*)workspace;
#ifdef Q40_TRACE
  p.trace = q40_trace_ptr;
#endif
  p.counters = (int*)((char*)workspace + 64);
  p.scratch = (float*)((char*)workspace + HEADER_BYTES);
  cudaStream_t st = (cudaStream_t)stream;
  const bool pdl = use_pdl != 0;
#define Q40_STREAM_MODES(MTV)                                                               \
  switch (mode) {                                                                           \
    case 0: return launch<MTV, PRO_NONE, EPI_STORE>(p, pl, smem_budget, st, pdl);           \
    case 1: return launch<MTV, PRO_NORM, EPI_STORE>(p, pl, smem_budget, st, pdl);           \
    case 2: return launch<MTV, PRO_NONE, EPI_RESIDUAL>(p, pl, smem_budget, st, pdl);        \
    default: return launch<MTV, PRO_NORM, EPI_SILU>(p, pl, smem_budget, st, pdl);           \
  }
  if (M <= 8) { Q40_STREAM_MODES(1) }
  Q40_STREAM_MODES(2)
#undef Q40_STREAM_MODES
}

// Sum-of-squares partials per row that a mode-2 launch writes for N output columns.
extern "C" int q40_gemv_stream_ss_count(int N) {
  if (N <= 0 || N % q40::stream::SPAN_COLS != 0) return 0;
  return N / q40::stream::SPAN_COLS;
}
