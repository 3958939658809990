// Decode-step Q4_0 matmul on a re-laid-out copy of the weights ("tiled" format): the same
// launch structure as q40_gemv_fused.cu (cp.async ring, programmatic dependent launch, cluster
// split-K through distributed shared memory, RMSNorm prologue, residual / SiLU-mul epilogues)
// with an inner loop of about one instruction per weight instead of almost three.
//
// The checkpoint layout ([K, N/2] bytes, two 64-column scale groups interleaved per byte) needs a
// byte shuffle to pair consecutive k, a sign fix-up and a scale multiply per pair of weights.  A
// one-time device pass (q40_relayout_tiled) rewrites each matrix, without changing a single code
// or scale, as a sequence of steps [span of 256 columns][16 k rows]:
//     4 groups of 64 columns x 32 lanes x 16 bytes   one 32-bit word per 16x16 MMA tile and lane,
//                                                    nibbles placed so that four mask operations
//                                                    (three after a shift) yield the four A-fragment
//                                                    registers of mma.m16n8k16 as fp16 values 72 + code
//     4 groups x 16 fp16 scales                      the scales of the 16 k rows
// The scale is applied to the activations instead of the weights (B operand = fp16(scale * x),
// one multiply per k and group instead of one per weight), and the constant 72 is removed exactly
// once per group by an extra MMA against an all-ones tile that accumulates sum_k scale*x.
// Products are exact in the tensor core and accumulated in fp32; compared with the reference's
// fp16(code*scale) operand the fp16 rounding moves from the weight to scale*x, which stays far
// inside the matmul tolerance (rel 2e-2) but is not the reference's rounding point — the
// checkpoint-layout kernels keep that one.  Steps are contiguous in memory, so a CTA's weight
// stream is one sequential run.
#include <cooperative_groups.h>

#include "q40_common.cuh"

namespace cg = cooperative_groups;

namespace q40 {
namespace tiled {

// Work split inside a CTA, chosen per batch width: a warp serves NG of the span's four 64-column
// groups and one of KS interleaved k slices, so a CTA has (4 / NG) * KS warps.  NG = 4, KS = 4 (four
// warps, 64 accumulator registers per 8 batch rows) measured fastest for up to 8 rows; NG = 2, KS = 2
// (four warps, two of them per k slice) for 9..16 rows; eight-warp splits (NG = 1 or 2 with KS = 2 or 4)
// were slower at every width.
constexpr int F_DEPTH = 4;                  // ring slots (16-row steps) per warp
constexpr int F_GROUP_W = 32 * 16;          // weights of one group-step: 32 lanes x 16 B (four 16x16 tiles)
constexpr int F_GROUP_BYTES = F_GROUP_W + 32 * 8;   // + 32 lanes x 8 B of scales (lane-private copies)
constexpr int T_STEP_BYTES = 2048 + 128;    // one step in the tiled stream: weights + 4 x 16 scales
constexpr int F_SPAN_BYTES = 128;
constexpr int F_SPAN_COLS = 256;
constexpr int F_XS_PAD = 16;

enum { PRO_NONE = 0, PRO_NORM = 1 };
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU = 2 };

struct TiledProblem {
  const uint8_t* bw;   // tiled stream: [N/256 spans][K/16 steps][T_STEP_BYTES]
  const __half* bs;    // unused (scales live in the stream)
  __half* out;         // [M, ldc]
  int N, nspans;
};

struct TiledParams {
  TiledProblem prob[3];
  int nprob;
  const __half* a;     // [M, lda] activations; with PRO_NORM the un-normalised residual stream
  int64_t lda, ldc;
  int M, K, rows_per_split;
  // PRO_NORM: the activations are fp16(fp16(float(a) * rsqrt(sum(ss_in[m][:]) / K + eps)) * norm_w), the
  // reference's RMSNorm (hf_model_q40_kv_shared.py:129-134)
  const __half* norm_w;
  const float* ss_in;
  int ss_in_count;
  float eps;
  // EPI_RESIDUAL: out = fp16(h_in + fp16(acc)); ss_out[m][span * nranks + rank] = sum of out^2
  const __half* h_in;
  int64_t ldh;
  float* ss_out;
  int ss_out_count;
  void* trace;             // stage timestamps (trace builds only)
  int recv_off;            // byte offset of the receive buffer in dynamic shared memory
};

__device__ __forceinline__ void f_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                      uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void f_cp16(uint32_t dst, const void* src, bool ok) {
  const int sz = ok ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void f_cp4(uint32_t dst, const void* src, bool ok) {
  const int sz = ok ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void f_cp8(uint32_t dst, const void* src, bool ok) {
  const int sz = ok ? 8 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void f_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void f_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ int f_span_col(int span, int lc) { return span * F_SPAN_COLS + lc; }

template <int MT, int NG, int KS, int PRO, int EPI>
__global__ void __launch_bounds__((4 / NG) * KS * 32, (NG == 4 ? (MT == 1 ? 3 : 2) : (MT == 1 ? 4 : 3)))
gemv_tiled_kernel(const TiledParams p) {
  constexpr int NGW = 4 / NG;                // warps that share a k slice
  constexpr int FW = NGW * KS;               // warps per CTA
  constexpr int FT = FW * 32;
  constexpr int F_SLOT_BYTES = NG * F_GROUP_BYTES;
  constexpr int NT = NG * 4;                 // 16x16 tiles per warp and step
  extern __shared__ __align__(16) unsigned char smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  Q40_TRACE_DECL
  Q40_STAMP(0);
  // phase 1 of the cluster barrier only says "this CTA is running" (waited for before the first
  // store into a neighbour's shared memory); phase 2 publishes those stores
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  const int nranks = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int slice = F_SPAN_COLS / nranks;            // 16, 32, 64, 128 or 256 columns finished by this rank

  // ---- which matrix and which 128-byte span of its rows ----
  int pi = 0, span = blockIdx.x;
  if (EPI == EPI_SILU) {
    pi = span & 1;
    span >>= 1;
  } else {
    while (pi < p.nprob - 1 && span >= p.prob[pi].nspans) { span -= p.prob[pi].nspans; ++pi; }
  }
  const TiledProblem& pr = p.prob[pi];
  const int split = blockIdx.y;
  const int kb = split * p.rows_per_split;
  const int ke = min(p.K, kb + p.rows_per_split);
  const int nsteps = (ke > kb) ? (ke - kb + 15) / 16 : 0;
  const int xs_ld = p.rows_per_split + F_XS_PAD;

  // shared memory: [ring: FW x DEPTH slots][xs: MT*8 rows] ... [s_inv: 16 floats][recv]; after the main
  // loop the front is reused for the warp slabs
  unsigned char* ring = smem;
  __half* xs = reinterpret_cast<__half*>(smem + FW * F_DEPTH * F_SLOT_BYTES);
  // 1/rms per row (RMSNorm prologue): 16 floats right below the receive buffer, clear of everything the
  // reduction reuses
  float* s_inv = reinterpret_cast<float*>(smem + p.recv_off - 64);
  const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring) + warp * (F_DEPTH * F_SLOT_BYTES);
  // [recv: nranks x M x slice floats] partial sums pushed by the cluster; a region of its own, because
  // neighbours may push while this CTA is still in its main loop
  float* recv = reinterpret_cast<float*>(smem + p.recv_off);

  // tiled stream of this span: K/16 steps of T_STEP_BYTES; this warp reads the part of column groups
  // gq0 .. gq0 + NG - 1 of the steps (kb/16 + ksl), + KS, ...
  const int gq0 = (warp % NGW) * NG, ksl = warp / NGW;
  const int ksteps_total = p.K / 16;
  const bool col_ok = span < pr.nspans;
  const uint8_t* sbase = pr.bw + ((int64_t)span * ksteps_total + kb / 16 + ksl) * T_STEP_BYTES;
  auto issue = [&](int j, int slot) {      // j-th step of this warp
    const uint32_t base = ring_u32 + slot * F_SLOT_BYTES;
    const uint8_t* sp = sbase + (int64_t)j * KS * T_STEP_BYTES;
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      f_cp16(base + q * F_GROUP_BYTES + lane * 16, sp + ((gq0 + q) * 32 + lane) * 16, col_ok);   // four tiles of the group
      f_cp8(base + q * F_GROUP_BYTES + F_GROUP_W + lane * 8, sp + 2048 + (gq0 + q) * 32 + t * 8,
            col_ok);                                                                            // scales of k rows 4t..4t+3
    }
  };

  // ---- prologue: weights only; nothing here depends on the previous kernel ----
  // its j-th step lives in ring slot j % DEPTH
  const int my_steps = (nsteps > ksl) ? (nsteps - ksl + KS - 1) / KS : 0;
#pragma unroll
  for (int j = 0; j < F_DEPTH; ++j) {
    if (j < my_steps) issue(j, j);
    f_commit();
  }
  Q40_STAMP(1);
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  Q40_STAMP(2);
  // the residual value of the first output this thread finishes, fetched now instead of at the very end
  __half h_first = __float2half(0.f);
  if (EPI == EPI_RESIDUAL && warp < p.M && lane < slice && col_ok)
    h_first = p.h_in[(int64_t)warp * p.ldh + f_span_col(span, rank * slice + lane)];

  // ---- activations of this k range.  RMSNorm prologue with the reference's rounding points:
  // fp16(fp16(float(a) * 1/rms) * norm_w).  The raw values are requested first, then the row statistics
  // are summed while they are in flight ----
  {
    const int chunks = p.rows_per_split / 8;
    const int total = MT * 8 * chunks;
    auto load_chunk = [&](int idx) {
      const int m = idx / chunks, k = kb + (idx % chunks) * 8;
      return (m < p.M && k < ke) ? *reinterpret_cast<const uint4*>(p.a + (int64_t)m * p.lda + k)
                                 : make_uint4(0, 0, 0, 0);
    };
    auto store_chunk = [&](int idx, uint4 v) {
      const int m = idx / chunks, kk = (idx % chunks) * 8;
      const int k = kb + kk;
      if (PRO == PRO_NORM && m < p.M && k < ke) {
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
      *reinterpret_cast<uint4*>(xs + m * xs_ld + kk) = v;
    };
    uint4 v_first = make_uint4(0, 0, 0, 0);
    if (tid < total) v_first = load_chunk(tid);
    if (PRO == PRO_NORM) {
      for (int m = warp; m < p.M; m += FW) {
        // all loads in flight before the first add (the partials sit in L2)
        float s = 0.f;
        const float* sp = p.ss_in + (int64_t)m * p.ss_in_count;
        for (int i0 = 0; i0 < p.ss_in_count; i0 += 256) {
          float part[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * 32 + lane;
            part[u] = (i < p.ss_in_count) ? __ldcg(sp + i) : 0.f;
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) s += part[u];
        }
        s = warp_sum(s);
        if (lane == 0) s_inv[m] = rsqrtf(s / (float)p.K + p.eps);
      }
      __syncthreads();
    }
    if (tid < total) store_chunk(tid, v_first);
    for (int idx = tid + FT; idx < total; idx += FT) store_chunk(idx, load_chunk(idx));
  }
  __syncthreads();

  Q40_STAMP(3);
  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[mt][i][j] = 0.f;
  float corr[MT][NG][4];     // per 64-column group: sum over k of scale * x (every row of a tile the same)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int q = 0; q < NG; ++q)
#pragma unroll
      for (int j = 0; j < 4; ++j) corr[mt][q][j] = 0.f;

  // ---- main loop: consume the oldest slot, refill it with the step DEPTH ahead ----
  const __half* xlane = xs + g * xs_ld + 4 * t;
  for (int j = 0; j < my_steps; ++j) {
    f_wait<F_DEPTH - 1>();            // the oldest outstanding group (step j) has landed
    const int slot = j % F_DEPTH;
    const unsigned char* sb = ring + (warp * F_DEPTH + slot) * F_SLOT_BYTES;
    const int step = ksl + j * KS;
    // activations of k rows 4t .. 4t+3 of this step for batch row g
    uint2 xv[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xv[mt] = *reinterpret_cast<const uint2*>(xlane + step * 16 + mt * 8 * xs_ld);
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const uint4 w = *reinterpret_cast<const uint4*>(sb + q * F_GROUP_BYTES + lane * 16);
      const uint2 sc = *reinterpret_cast<const uint2*>(sb + q * F_GROUP_BYTES + F_GROUP_W + lane * 8);
      uint32_t yb[MT][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        yb[mt][0] = h2_as_u32(__hmul2(u32_as_h2(xv[mt].x), u32_as_h2(sc.x)));   // scale * x, k rows 4t, 4t+1
        yb[mt][1] = h2_as_u32(__hmul2(u32_as_h2(xv[mt].y), u32_as_h2(sc.y)));   // k rows 4t+2, 4t+3
        f_mma(corr[mt][q], 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, yb[mt][0], yb[mt][1]);
      }
      const uint32_t wds[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int jt = 0; jt < 4; ++jt) {
        const uint32_t v = wds[jt];
        // nibble -> fp16 value 72 + code: bits 4..7 of each 16-bit half under exponent 0x5400, sign bit flipped
        const uint32_t a0 = lop3_and_xor(v, 0x00F000F0u, 0x54805480u);          // column g,   k 4t, 4t+1
        const uint32_t a1 = lop3_and_xor(v << 4, 0x00F000F0u, 0x54805480u);     // column g+8, k 4t, 4t+1
        const uint32_t a2 = lop3_and_xor(v >> 8, 0x00F000F0u, 0x54805480u);     // column g,   k 4t+2, 4t+3
        const uint32_t a3 = lop3_and_xor(v >> 4, 0x00F000F0u, 0x54805480u);     // column g+8, k 4t+2, 4t+3
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) f_mma(acc[mt][q * 4 + jt], a0, a1, a2, a3, yb[mt][0], yb[mt][1]);
      }
    }
    // each lane reads back only what it copied itself and has consumed it by now, so the slot can
    // be refilled without a barrier
    if (j + F_DEPTH < my_steps) issue(j + F_DEPTH, slot);
    f_commit();
  }
  f_wait<0>();
  __syncthreads();   // every warp is done with its ring slots and with xs
  Q40_STAMP(4);

  // remove the constant 72 carried by every weight operand: acc -= 72 * sum_k(scale * x)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[mt][i][j] = fmaf(-72.0f, corr[mt][i >> 2][j], acc[mt][i][j]);

  // ---- sum the warps: each stores its fragment slab; then every (m, column) sum of the CTA is pushed
  // into the shared memory of the cluster rank that finishes that column ----
  float4* slab = reinterpret_cast<float4*>(smem);                 // [FW][MT][NT][32] float4
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < NT; ++i)
      slab[((warp * MT + mt) * NT + i) * 32 + lane] =
          make_float4(acc[mt][i][0], acc[mt][i][1], acc[mt][i][2], acc[mt][i][3]);
  __syncthreads();
  Q40_STAMP(5);
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");     // every CTA of the cluster is running
  {
    const float* sl = reinterpret_cast<const float*>(slab);
    const int total = p.M * F_SPAN_COLS;
    for (int idx = tid; idx < total; idx += FT) {
      const int m = idx / F_SPAN_COLS, lc = idx % F_SPAN_COLS;
      // column lc = 64*group + 16*tile + row; row r -> lane group r & 7, upper half of the tile if r >= 8
      const int grp = lc >> 6, jt = (lc >> 4) & 3, r = lc & 15;
      const int mt = m >> 3, mm = m & 7;
      const int fl = (r & 7) * 4 + (mm >> 1);
      const int off = (((mt * NT + (grp % NG) * 4 + jt) * 32 + fl) << 2) + (mm & 1) + 2 * (r >> 3);
      float v = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)        // the k slices of the group
        v += sl[off + (grp / NG + NGW * ks) * (MT * NT * 32 * 4)];
      float* dst = cluster.map_shared_rank(recv, lc / slice);
      dst[(rank * p.M + m) * slice + (lc % slice)] = v;
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  Q40_STAMP(6);

  // ---- split-K over the cluster: rank r finishes columns [r*slice, (r+1)*slice) of the span from the
  // partials it received (added in rank order) ----
  const int npart = (EPI == EPI_SILU) ? nranks / 2 : nranks;
  for (int m = warp; m < p.M; m += FW) {
    float ssq = 0.f;
    for (int cidx = lane; cidx < slice; cidx += 32) {
      const int lc = rank * slice + cidx;
      const float* rp = recv + m * slice + cidx;
      const int rstride = p.M * slice;
      float v0 = 0.f, v1 = 0.f;
      if (EPI == EPI_SILU) {
        for (int r = 0; r < npart; ++r) {
          v0 += rp[(2 * r) * rstride];         // w1 partials
          v1 += rp[(2 * r + 1) * rstride];     // w3 partials
        }
      } else {
        for (int r = 0; r < npart; ++r) v0 += rp[r * rstride];
      }
      const int n = f_span_col(span, lc);
      if (n < pr.N) {
        if (EPI == EPI_STORE) {
          pr.out[(int64_t)m * p.ldc + n] = __float2half_rn(v0);
        } else if (EPI == EPI_RESIDUAL) {
          const __half hres = (m == warp && cidx == lane) ? h_first : p.h_in[(int64_t)m * p.ldh + n];
          const __half hn = __hadd_rn(hres, __float2half_rn(v0));
          pr.out[(int64_t)m * p.ldc + n] = hn;
          const float f = __half2float(hn);
          ssq = fmaf(f, f, ssq);
        } else {
          const float a1 = __half2float(__float2half_rn(v0));
          const __half s = __float2half_rn(a1 / (1.0f + expf(-a1)));
          p.prob[0].out[(int64_t)m * p.ldc + n] = __hmul_rn(s, __float2half_rn(v1));
        }
      }
    }
    if (EPI == EPI_RESIDUAL) {
      ssq = warp_sum(ssq);
      if (lane == 0) p.ss_out[(int64_t)m * p.ss_out_count + span * nranks + rank] = ssq;
    }
  }
  Q40_STAMP(7);
  Q40_TRACE_FLUSH(p.trace, 100 + 10 * PRO + EPI);
}

template <int MT, int NG, int KS, int PRO, int EPI>
static int launch_tiled(const TiledParams& p, int grid_x, int nsplit, int cluster_x, cudaStream_t st, bool pdl) {
  auto kern = gemv_tiled_kernel<MT, NG, KS, PRO, EPI>;
  constexpr int FW = (4 / NG) * KS, FT = FW * 32, NT = NG * 4;
  const size_t ring = (size_t)FW * F_DEPTH * NG * F_GROUP_BYTES;
  const size_t xs = (size_t)MT * 8 * (p.rows_per_split + F_XS_PAD) * 2;
  const size_t red = (size_t)FW * MT * NT * 32 * 16;
  size_t smem = (ring + xs) > red ? (ring + xs) : red;
  smem = (smem + 15) / 16 * 16 + 64;            // + the table of 1/rms per row
  TiledParams pp = p;
  pp.recv_off = (int)smem;
  smem += (size_t)p.M * F_SPAN_COLS * 4;        // receive buffer of the cluster reduction
  // a shape whose shared-memory need exceeds what a CTA of this device may have is refused with a
  // negative status (callers fall back to the workspace kernel), not reported as a CUDA error
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return Q40_E_UNSUPPORTED;
  }
  // set on every variant, not only those that need it (see the note at q40_gemv_tiled)
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid_x, nsplit, 1);
  cfg.blockDim = dim3(FT, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = cluster_x;
  attrs[0].val.clusterDim.y = nsplit;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  if (cluster_x * nsplit > 8) {
    // a 16-CTA cluster is outside the portable limit: ask whether this device can schedule one
    int nclusters = 0;
    e = cudaOccupancyMaxActiveClusters(&nclusters, kern, &cfg);
    if (e != cudaSuccess || nclusters < 1) {
      (void)cudaGetLastError();
      return Q40_E_UNSUPPORTED;
    }
  }
  cfg.numAttrs = pdl ? 2 : 1;
  e = cudaLaunchKernelEx(&cfg, kern, pp);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}

}  // namespace tiled
}  // namespace q40

// One fused decode matmul launch.  mode: 0 = plain store (1-3 matrices sharing the activations),
// 1 = RMSNorm prologue + store, 2 = residual-add epilogue, 3 = RMSNorm prologue + SiLU-mul of a
// (w1, w3) pair.  See include/q40b200.h for the argument contract.
extern "C" int q40_gemv_tiled(int mode, int nmat, const void* const* bw, const void* const* bs,
                              void* const* out, const int* n_cols, int64_t ldc, const void* a, int64_t lda,
                              int M, int K, const void* norm_w, const float* ss_in, int ss_in_count,
                              float eps, const void* h_in, int64_t ldh, float* ss_out, int ss_out_count,
                              int max_cluster, int use_pdl, void* stream) {
  using namespace q40;
  using namespace q40::tiled;
  if (!bw || !out || !n_cols || !a) return Q40_E_NULL;
  if (mode < 0 || mode > 3 || nmat < 1 || nmat > 3) return Q40_E_UNSUPPORTED;
  if (mode == 3 && nmat != 2) return Q40_E_UNSUPPORTED;
  if (mode == 2 && nmat != 1) return Q40_E_UNSUPPORTED;
  if (M < 1 || M > 16 || K < 16 || K % 16 != 0 || lda < K || lda % 8 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(a, 16)) return Q40_E_ALIGN;
  if ((mode == 1 || mode == 3) && (!norm_w || !ss_in || ss_in_count < 1 || !q40_aligned(norm_w, 16)))
    return Q40_E_NULL;
  if (mode == 2 && (!h_in || !ss_out)) return Q40_E_NULL;
  if (max_cluster != 8 && max_cluster != 16) return Q40_E_UNSUPPORTED;
  TiledParams p{};
  int total_spans = 0;
  for (int i = 0; i < nmat; ++i) {
    if (!bw[i] || !out[i]) return Q40_E_NULL;
    if (n_cols[i] <= 0 || n_cols[i] % 256 != 0) return Q40_E_SHAPE;
    if (!q40_aligned(bw[i], 16)) return Q40_E_ALIGN;
    p.prob[i].bw = (const uint8_t*)bw[i];
    p.prob[i].bs = nullptr;
    p.prob[i].out = (__half*)out[i];
    p.prob[i].N = n_cols[i];
    p.prob[i].nspans = (n_cols[i] / 2 + F_SPAN_BYTES - 1) / F_SPAN_BYTES;
    total_spans += p.prob[i].nspans;
    if (ldc < n_cols[i]) return Q40_E_SHAPE;
  }
  if (mode == 3 && n_cols[0] != n_cols[1]) return Q40_E_SHAPE;
  p.nprob = nmat;
  p.a = (const __half*)a; p.lda = lda; p.ldc = ldc; p.M = M; p.K = K;
  p.norm_w = (const __half*)norm_w; p.ss_in = ss_in; p.ss_in_count = ss_in_count; p.eps = eps;
  p.h_in = (const __half*)h_in; p.ldh = ldh; p.ss_out = ss_out; p.ss_out_count = ss_out_count;
#ifdef Q40_TRACE
  p.trace = q40_trace_ptr;
#endif

  // split K over the cluster: as many splits as the cluster allows while a split keeps >= 64 rows,
  // and few enough CTAs to be resident at once (3 per SM)
  const int cluster_x = (mode == 3) ? 2 : 1;
  const int grid_x = (mode == 3) ? 2 * p.prob[0].nspans : total_spans;
  int nsplit = max_cluster / cluster_x;
  while (nsplit > 1 && ((K / nsplit) < 64 || (int64_t)grid_x * nsplit > 148 * 3)) nsplit >>= 1;
  int rps = (K + nsplit - 1) / nsplit;
  rps = ((rps + 15) / 16) * 16;
  p.rows_per_split = rps;
  if (mode == 2 && ss_out_count != p.prob[0].nspans * nsplit * cluster_x) return Q40_E_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const bool pdl = use_pdl != 0;
  const int mt = (M <= 8) ? 1 : 2;
#define Q40_TILED_MODES(MTV, NGV, KSV)                                                              \
  switch (mode) {                                                                                    \
    case 0: return launch_tiled<MTV, NGV, KSV, PRO_NONE, EPI_STORE>(p, grid_x, nsplit, cluster_x, st, pdl);    \
    case 1: return launch_tiled<MTV, NGV, KSV, PRO_NORM, EPI_STORE>(p, grid_x, nsplit, cluster_x, st, pdl);    \
    case 2: return launch_tiled<MTV, NGV, KSV, PRO_NONE, EPI_RESIDUAL>(p, grid_x, nsplit, cluster_x, st, pdl); \
    default: return launch_tiled<MTV, NGV, KSV, PRO_NORM, EPI_SILU>(p, grid_x, nsplit, cluster_x, st, pdl);    \
  }
  if (mt == 1) { Q40_TILED_MODES(1, 4, 4) }
  Q40_TILED_MODES(2, 2, 2)
#undef Q40_TILED_MODES
}

// Number of per-row sum-of-squares partials a mode-2 launch writes for this shape (so the caller can
// size ss_out and pass the count to the consumer's prologue).
extern "C" int q40_gemv_tiled_ss_count(int N, int K, int max_cluster) {
  if (N <= 0 || N % 256 != 0 || K < 16 || (max_cluster != 8 && max_cluster != 16)) return 0;
  const int nspans = (N / 2 + q40::tiled::F_SPAN_BYTES - 1) / q40::tiled::F_SPAN_BYTES;
  int nsplit = max_cluster;
  while (nsplit > 1 && ((K / nsplit) < 64 || (int64_t)nspans * nsplit > 148 * 3)) nsplit >>= 1;
  return nspans * nsplit;
}

namespace q40 {
namespace tiled {

// One thread per output word (or per scale): gathers eight nibbles of the checkpoint layout into the
// word of (span, k step, group, lane, tile) described at the top of this file.
__global__ void __launch_bounds__(256)
relayout_kernel(const uint8_t* __restrict__ bw, const __half* __restrict__ bs, uint8_t* __restrict__ out, int N,
                int K) {
  const int ksteps = K / 16;
  const int64_t nsteps = (int64_t)(N / 256) * ksteps;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stepi = gid / 576;            // 512 weight words + 64 scale slots per step
  const int w = (int)(gid % 576);
  if (stepi >= nsteps) return;
  const int span = (int)(stepi / ksteps), ks = (int)(stepi % ksteps);
  uint8_t* dst = out + stepi * T_STEP_BYTES;
  const int64_t w_ld = N / 2, s_ld = N / 64;
  if (w < 512) {
    const int q = w >> 7, lane = (w >> 2) & 31, jt = w & 3;
    const int g = lane >> 2, t = lane & 3;
    // native layout: group q of the span = block q/2 of the span's two 64-byte blocks, high nibble if q even
    const int byte_col = span * 128 + (q >> 1) * 64 + jt * 16 + g;     // column g of the tile; column g+8 is 8 bytes on
    const bool high = (q & 1) == 0;
    uint32_t nib[2][4];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint8_t b = bw[(int64_t)(ks * 16 + 4 * t + kk) * w_ld + byte_col + 8 * c];
        nib[c][kk] = high ? (b >> 4) : (b & 0xF);
      }
    // byte0 = A | B<<4, byte1 = C | D<<4, byte2 = E | F<<4, byte3 = G | H<<4 with
    // B,F,D,H = column g at k+0,+1,+2,+3 and A,E,C,G = column g+8 at k+0,+1,+2,+3
    const uint32_t word = (nib[1][0] | (nib[0][0] << 4)) | ((nib[1][2] | (nib[0][2] << 4)) << 8) |
                          ((nib[1][1] | (nib[0][1] << 4)) << 16) | ((nib[1][3] | (nib[0][3] << 4)) << 24);
    reinterpret_cast<uint32_t*>(dst)[w] = word;
  } else {
    const int i = w - 512, q = i >> 4, kk = i & 15;
    reinterpret_cast<__half*>(dst + 2048)[i] = bs[(int64_t)(ks * 16 + kk) * s_ld + span * 4 + q];
  }
}

}  // namespace tiled
}  // namespace q40

// Bytes of the tiled copy of a [K, N] matrix (N % 256 == 0, K % 16 == 0): same size as packed + scales.
extern "C" size_t q40_tiled_bytes(int N, int K) {
  if (N <= 0 || K <= 0 || N % 256 != 0 || K % 16 != 0) return 0;
  return (size_t)(N / 256) * (K / 16) * q40::tiled::T_STEP_BYTES;
}

extern "C" int q40_relayout_tiled(const void* bw, const void* bs, void* out, int N, int K, void* stream) {
  if (!bw || !bs || !out) return Q40_E_NULL;
  if (N <= 0 || K <= 0 || N % 256 != 0 || K % 16 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(out, 16)) return Q40_E_ALIGN;
  const int64_t threads = (int64_t)(N / 256) * (K / 16) * 576;
  const int64_t grid = (threads + 255) / 256;
  if (grid > 0x7fffffffLL) return Q40_E_SHAPE;
  q40::tiled::relayout_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)bw, (const __half*)bs,
                                                                              (uint8_t*)out, N, K);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}
