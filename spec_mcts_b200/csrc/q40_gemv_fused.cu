// Decode-step form of the Q4_0 dequant-matmul ("kn" orientation, G = 64, M <= 16): the same
// register-level scheme as gemv_kn_kernel (q40_gemm.cu) — nibbles -> exact fp16 via the
// 0x6400 exponent trick, x fp16 scale, fed as the 16x16 A tile of mma.m16n8k16 with fp32
// accumulation — reorganised so that a chain of dependent matmuls streams weights without
// gaps:
//
//   * weight prefetch does not depend on the previous kernel, so every lane first queues
//     cp.async copies of its own next DEPTH 16-row steps (weights + scales) into a
//     lane-private shared-memory ring, then signals `griddepcontrol.launch_dependents` and
//     only then waits (`griddepcontrol.wait`) for the producer of its activations
//     (programmatic dependent launch): the HBM stream of kernel n+1 runs under the
//     reduction tail of kernel n;
//   * split-K partials never touch global memory: the CTAs that share an output span form a
//     thread-block cluster (up to 16 along K) and are summed through distributed shared
//     memory, each rank finishing a slice of the span's columns;
//   * the element-wise neighbours of the matmul are folded in: RMSNorm of the residual
//     stream as a prologue (row sums of squares arrive as per-slice partials from the
//     kernel that produced the stream), and as epilogues either the residual add (also
//     emitting those partials) or SiLU(w1 x) * (w3 x) for a w1/w3 pair whose CTAs share a
//     cluster.  Rounding points are the reference's (hf_model_q40_kv_shared.py:129-134,
//     434, 463-466): fp16 matmul outputs, fp16 adds and multiplies, fp32 inside the norm.
//   * up to three weight matrices that consume the same activations (wq, wk, wv) run as one
//     launch.
#include <cooperative_groups.h>

#include "q40_common.cuh"

namespace cg = cooperative_groups;

namespace q40 {

constexpr int FW = 4;                       // warps per CTA
constexpr int FT = FW * 32;
constexpr int F_DEPTH = 4;                  // ring slots (16-row steps) per warp
constexpr int F_SLOT_W = 4 * 32 * 16;       // weights of one step: 4 rows x 32 lanes x 16 B
constexpr int F_SLOT_BYTES = F_SLOT_W + 4 * 32 * 4;   // + 4 rows x 32 lanes x 4 B of scales
constexpr int F_SPAN_BYTES = 128;
constexpr int F_SPAN_COLS = 256;
constexpr int F_XS_PAD = 16;

enum { PRO_NONE = 0, PRO_NORM = 1 };
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU = 2 };

struct FusedProblem {
  const uint8_t* bw;   // [K, N/2]
  const __half* bs;    // [K, N/64]
  __half* out;         // [M, ldc]
  int N, nspans;
};

struct FusedParams {
  FusedProblem prob[3];
  int nprob;
  const __half* a;     // [M, lda] activations; with PRO_NORM the un-normalised residual stream
  int64_t lda, ldc;
  int M, K, rows_per_split;
  // PRO_NORM: x = fp16(fp16(a * rsqrt(sum(ss_in[m][:]) / K + eps)) * norm_w)
  const __half* norm_w;
  const float* ss_in;
  int ss_in_count;
  float eps;
  // EPI_RESIDUAL: out = fp16(h_in + fp16(acc)); ss_out[m][span * nranks + rank] = sum of out^2
  const __half* h_in;
  int64_t ldh;
  float* ss_out;
  int ss_out_count;
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
__device__ __forceinline__ void f_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void f_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ int f_span_col(int span, int lc) {
  const int cb = span * F_SPAN_BYTES + (lc & (F_SPAN_BYTES - 1));
  return 128 * (cb >> 6) + (cb & 63) + ((lc >> 7) ? 64 : 0);
}

template <int MT, int PRO, int EPI>
__global__ void __launch_bounds__(FT, (MT == 1 ? 3 : 2))
gemv_fused_kernel(const FusedParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  // ---- which matrix and which 128-byte span of its rows ----
  int pi = 0, span = blockIdx.x;
  if (EPI == EPI_SILU) {
    pi = span & 1;
    span >>= 1;
  } else {
    while (pi < p.nprob - 1 && span >= p.prob[pi].nspans) { span -= p.prob[pi].nspans; ++pi; }
  }
  const FusedProblem& pr = p.prob[pi];
  const int split = blockIdx.y;
  const int kb = split * p.rows_per_split;
  const int ke = min(p.K, kb + p.rows_per_split);
  const int nsteps = (ke > kb) ? (ke - kb + 15) / 16 : 0;
  const int xs_ld = p.rows_per_split + F_XS_PAD;

  // shared memory: [ring: FW x DEPTH slots][xs: MT*8 rows][s_inv: 16 floats]; after the main loop the
  // ring is reused for the warp slabs and the CTA partial
  unsigned char* ring = smem;
  __half* xs = reinterpret_cast<__half*>(smem + FW * F_DEPTH * F_SLOT_BYTES);
  float* s_inv = reinterpret_cast<float*>(smem + FW * F_DEPTH * F_SLOT_BYTES + MT * 8 * xs_ld * 2);
  const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring) + warp * (F_DEPTH * F_SLOT_BYTES);

  const int64_t w_ld = pr.N / 2, s_ld = pr.N / 64;
  const int colbyte = span * F_SPAN_BYTES + 16 * g;
  const bool col_ok = colbyte < w_ld;
  const uint8_t* wcol = pr.bw + (col_ok ? colbyte : 0);
  const __half* scol = pr.bs + (col_ok ? 2 * (colbyte >> 6) : 0);

  // queue one 16-row step: this lane's 16 bytes of rows k0 .. k0+3 and their scale pairs.
  // K and the split size are multiples of 16, so a step inside the range is never partial.
  const uint8_t* wstep = wcol + (int64_t)(kb + warp * 16 + 4 * t) * w_ld;   // this warp's step 0
  const __half* sstep = scol + (int64_t)(kb + warp * 16 + 4 * t) * s_ld;
  const int64_t w_adv = (int64_t)FW * 16 * w_ld, s_adv = (int64_t)FW * 16 * s_ld;
  auto issue = [&](int j, int slot) {      // j-th step of this warp
    const uint32_t base = ring_u32 + slot * F_SLOT_BYTES + lane * 16;
    const uint8_t* wp = wstep + j * w_adv;
    const __half* sp = sstep + j * s_adv;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      f_cp16(base + r * 512, wp + r * w_ld, col_ok);
      f_cp4(base + F_SLOT_W - lane * 12 + r * 128, sp + r * s_ld, col_ok);
    }
  };

  // ---- prologue: weights only; nothing here depends on the previous kernel ----
  // warp w owns steps w, w+FW, ...; its j-th step lives in ring slot j % DEPTH
  const int my_steps = (nsteps > warp) ? (nsteps - warp + FW - 1) / FW : 0;
#pragma unroll
  for (int j = 0; j < F_DEPTH; ++j) {
    if (j < my_steps) issue(j, j);
    f_commit();
  }
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activations of this k range: raw copy first (and the norm weights), so that the loads do
  // not wait for the row statistics; then, for the RMSNorm prologue, normalise in place ----
  __half* wn = reinterpret_cast<__half*>(s_inv + 16);     // [rows_per_split] norm weights of this range
  {
    const int chunks = p.rows_per_split / 8;
    for (int idx = tid; idx < MT * 8 * chunks; idx += FT) {
      const int m = idx / chunks, kk = (idx % chunks) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      const int k = kb + kk;
      if (m < p.M && k < ke) v = *reinterpret_cast<const uint4*>(p.a + (int64_t)m * p.lda + k);
      *reinterpret_cast<uint4*>(xs + m * xs_ld + kk) = v;
    }
    if (PRO == PRO_NORM) {
      for (int idx = tid; idx < chunks; idx += FT) {
        const int k = kb + idx * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (k < ke) v = *reinterpret_cast<const uint4*>(p.norm_w + k);
        *reinterpret_cast<uint4*>(wn + idx * 8) = v;
      }
      for (int m = warp; m < p.M; m += FW) {
        float s = 0.f;
        for (int i = lane; i < p.ss_in_count; i += 32) s += p.ss_in[(int64_t)m * p.ss_in_count + i];
        s = warp_sum(s);
        if (lane == 0) s_inv[m] = rsqrtf(s / (float)p.K + p.eps);
      }
    }
  }
  __syncthreads();
  if (PRO == PRO_NORM) {
    const int chunks = p.rows_per_split / 8;
    for (int idx = tid; idx < p.M * chunks; idx += FT) {
      const int m = idx / chunks, kk = (idx % chunks) * 8;
      uint4 v = *reinterpret_cast<const uint4*>(xs + m * xs_ld + kk);
      const uint4 wv = *reinterpret_cast<const uint4*>(wn + kk);
      __half2* vh = reinterpret_cast<__half2*>(&v);
      const __half2* wh = reinterpret_cast<const __half2*>(&wv);
      const float inv = s_inv[m];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(vh[j]);
        vh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);
      }
      *reinterpret_cast<uint4*>(xs + m * xs_ld + kk) = v;
    }
    __syncthreads();
  }

  float acc[MT][16][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[mt][i][j] = 0.f;

  // ---- main loop: consume the oldest slot, refill it with the step DEPTH ahead ----
  const __half* xlane = xs + g * xs_ld + 4 * t;
  for (int j = 0; j < my_steps; ++j) {
    f_wait<F_DEPTH - 1>();            // the oldest outstanding group (step j) has landed
    const int slot = j % F_DEPTH;
    const unsigned char* sb = ring + (warp * F_DEPTH + slot) * F_SLOT_BYTES;
    uint4 w[4];
    uint32_t sc[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      w[r] = *reinterpret_cast<const uint4*>(sb + (r * 32 + lane) * 16);
      sc[r] = *reinterpret_cast<const uint32_t*>(sb + F_SLOT_W + (r * 32 + lane) * 4);
    }
    const int step = warp + j * FW;
    uint32_t xb[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const uint2 v = *reinterpret_cast<const uint2*>(xlane + step * 16 + mt * 8 * xs_ld);
      xb[mt][0] = v.x;
      xb[mt][1] = v.y;
    }
    const __half2 sh01 = u32_as_h2(prmt(sc[0], sc[1], 0x5410)), sl01 = u32_as_h2(prmt(sc[0], sc[1], 0x7632));
    const __half2 sh23 = u32_as_h2(prmt(sc[2], sc[3], 0x5410)), sl23 = u32_as_h2(prmt(sc[2], sc[3], 0x7632));
    const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&w[0]);
    const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&w[1]);
    const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&w[2]);
    const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&w[3]);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t sel = (uint32_t)b | ((uint32_t)(4 + b) << 8);
        const uint32_t p01 = prmt(w0[wi], w1[wi], sel);
        const uint32_t p23 = prmt(w2[wi], w3[wi], sel);
        const uint32_t a0 = h2_as_u32(__hmul2(codes_hi_to_h2(p01), sh01));
        const uint32_t a1 = h2_as_u32(__hmul2(codes_lo_to_h2(p01), sl01));
        const uint32_t a2 = h2_as_u32(__hmul2(codes_hi_to_h2(p23), sh23));
        const uint32_t a3 = h2_as_u32(__hmul2(codes_lo_to_h2(p23), sl23));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) f_mma(acc[mt][wi * 4 + b], a0, a1, a2, a3, xb[mt][0], xb[mt][1]);
      }
    }
    // each lane reads back only what it copied itself and has consumed it by now, so the slot can
    // be refilled without a barrier
    if (j + F_DEPTH < my_steps) issue(j + F_DEPTH, slot);
    f_commit();
  }
  f_wait<0>();
  __syncthreads();   // every warp is done with its ring slots and with xs

  // ---- sum the warps: each stores its fragment slab, then the CTA partial is built per (m, column) ----
  float4* slab = reinterpret_cast<float4*>(smem);                 // [FW][MT][16][32] float4
  float* cta_part = reinterpret_cast<float*>(smem + FW * MT * 16 * 32 * 16);   // [M][256]
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 16; ++i)
      slab[((warp * MT + mt) * 16 + i) * 32 + lane] =
          make_float4(acc[mt][i][0], acc[mt][i][1], acc[mt][i][2], acc[mt][i][3]);
  __syncthreads();
  {
    const float* sl = reinterpret_cast<const float*>(slab);
    const int total = p.M * F_SPAN_COLS;
    for (int idx = tid; idx < total; idx += FT) {
      const int m = idx / F_SPAN_COLS, lc = idx % F_SPAN_COLS;
      const int c = lc & 127, is_lo = lc >> 7;
      const int fg = c >> 4, tb = c & 15;
      const int mt = m >> 3, mm = m & 7;
      const int fl = fg * 4 + (mm >> 1);
      const int off = (((mt * 16 + tb) * 32 + fl) << 2) + (mm & 1) + 2 * is_lo;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < FW; ++w) v += sl[off + w * (MT * 16 * 32 * 4)];
      cta_part[idx] = v;
    }
  }
  cluster.sync();

  // ---- split-K over the cluster: rank r finishes columns [r*slice, (r+1)*slice) of the span ----
  const int nranks = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int slice = F_SPAN_COLS / nranks;            // 16, 32, 64, 128 or 256
  const int npart = (EPI == EPI_SILU) ? nranks / 2 : nranks;
  for (int m = warp; m < p.M; m += FW) {
    float ssq = 0.f;
    for (int cidx = lane; cidx < slice; cidx += 32) {
      const int lc = rank * slice + cidx;
      const int idx = m * F_SPAN_COLS + lc;
      // all remote loads are issued before the first add; the adds keep rank order
      float v0 = 0.f, v1 = 0.f;
      if (EPI == EPI_SILU) {
        float t0[8], t1[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          t0[r] = (r < npart) ? *cluster.map_shared_rank(cta_part + idx, 2 * r) : 0.f;       // w1 partials
          t1[r] = (r < npart) ? *cluster.map_shared_rank(cta_part + idx, 2 * r + 1) : 0.f;   // w3 partials
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) { v0 += t0[r]; v1 += t1[r]; }
      } else {
        float t0[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) t0[r] = (r < npart) ? *cluster.map_shared_rank(cta_part + idx, r) : 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) v0 += t0[r];
      }
      const int n = f_span_col(span, lc);
      if (n < pr.N) {
        if (EPI == EPI_STORE) {
          pr.out[(int64_t)m * p.ldc + n] = __float2half_rn(v0);
        } else if (EPI == EPI_RESIDUAL) {
          const __half hn = __hadd_rn(p.h_in[(int64_t)m * p.ldh + n], __float2half_rn(v0));
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
  cluster.sync();   // nobody leaves while a neighbour may still read its partial
}

template <int MT, int PRO, int EPI>
static int launch_fused(const FusedParams& p, int grid_x, int nsplit, int cluster_x, cudaStream_t st, bool pdl) {
  auto kern = gemv_fused_kernel<MT, PRO, EPI>;
  const size_t ring = (size_t)FW * F_DEPTH * F_SLOT_BYTES;
  const size_t xs = (size_t)MT * 8 * (p.rows_per_split + F_XS_PAD) * 2 + 64 + (size_t)p.rows_per_split * 2;
  const size_t red = (size_t)FW * MT * 16 * 32 * 16 + (size_t)p.M * F_SPAN_COLS * 4;
  const size_t smem = (ring + xs) > red ? (ring + xs) : red;
  // a shape whose shared-memory need exceeds what a CTA of this device may have is refused with a
  // negative status (callers fall back to the workspace kernel), not reported as a CUDA error
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return Q40_E_UNSUPPORTED;
  }
  if (cluster_x * nsplit > 8) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
  }
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
  e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}

}  // namespace q40

// One fused decode matmul launch.  mode: 0 = plain store (1-3 matrices sharing the activations),
// 1 = RMSNorm prologue + store, 2 = residual-add epilogue, 3 = RMSNorm prologue + SiLU-mul of a
// (w1, w3) pair.  See include/q40b200.h for the argument contract.
extern "C" int q40_gemv_fused(int mode, int nmat, const void* const* bw, const void* const* bs,
                              void* const* out, const int* n_cols, int64_t ldc, const void* a, int64_t lda,
                              int M, int K, const void* norm_w, const float* ss_in, int ss_in_count,
                              float eps, const void* h_in, int64_t ldh, float* ss_out, int ss_out_count,
                              int max_cluster, int use_pdl, void* stream) {
  using namespace q40;
  if (!bw || !bs || !out || !n_cols || !a) return Q40_E_NULL;
  if (mode < 0 || mode > 3 || nmat < 1 || nmat > 3) return Q40_E_UNSUPPORTED;
  if (mode == 3 && nmat != 2) return Q40_E_UNSUPPORTED;
  if (mode == 2 && nmat != 1) return Q40_E_UNSUPPORTED;
  if (M < 1 || M > 16 || K < 16 || K % 16 != 0 || lda < K || lda % 8 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(a, 16)) return Q40_E_ALIGN;
  if ((mode == 1 || mode == 3) && (!norm_w || !ss_in || ss_in_count < 1 || !q40_aligned(norm_w, 16)))
    return Q40_E_NULL;
  if (mode == 2 && (!h_in || !ss_out)) return Q40_E_NULL;
  if (max_cluster != 8 && max_cluster != 16) return Q40_E_UNSUPPORTED;
  FusedParams p{};
  int total_spans = 0;
  for (int i = 0; i < nmat; ++i) {
    if (!bw[i] || !bs[i] || !out[i]) return Q40_E_NULL;
    if (n_cols[i] <= 0 || n_cols[i] % 128 != 0) return Q40_E_SHAPE;
    if (!q40_aligned(bw[i], 16) || !q40_aligned(bs[i], 4)) return Q40_E_ALIGN;
    p.prob[i].bw = (const uint8_t*)bw[i];
    p.prob[i].bs = (const __half*)bs[i];
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
#define Q40_FUSED(MTV, PROV, EPIV) launch_fused<MTV, PROV, EPIV>(p, grid_x, nsplit, cluster_x, st, pdl)
  if (mt == 1) {
    switch (mode) {
      case 0: return Q40_FUSED(1, PRO_NONE, EPI_STORE);
      case 1: return Q40_FUSED(1, PRO_NORM, EPI_STORE);
      case 2: return Q40_FUSED(1, PRO_NONE, EPI_RESIDUAL);
      default: return Q40_FUSED(1, PRO_NORM, EPI_SILU);
    }
  }
  switch (mode) {
    case 0: return Q40_FUSED(2, PRO_NONE, EPI_STORE);
    case 1: return Q40_FUSED(2, PRO_NORM, EPI_STORE);
    case 2: return Q40_FUSED(2, PRO_NONE, EPI_RESIDUAL);
    default: return Q40_FUSED(2, PRO_NORM, EPI_SILU);
  }
#undef Q40_FUSED
}

// Number of per-row sum-of-squares partials a mode-2 launch writes for this shape (so the caller can
// size ss_out and pass the count to the consumer's prologue).
extern "C" int q40_gemv_fused_ss_count(int N, int K, int max_cluster) {
  if (N <= 0 || N % 128 != 0 || K < 16 || (max_cluster != 8 && max_cluster != 16)) return 0;
  const int nspans = (N / 2 + q40::F_SPAN_BYTES - 1) / q40::F_SPAN_BYTES;
  int nsplit = max_cluster;
  while (nsplit > 1 && ((K / nsplit) < 64 || (int64_t)nspans * nsplit > 148 * 3)) nsplit >>= 1;
  return nspans * nsplit;
}
