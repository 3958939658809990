// Fused Q4_0 dequant-matmul for decode batches (M <= 16 rows per pass): a split-K,
// weight-streaming kernel that is bound by HBM.
//
// Orientation "kn" (the on-disk one): the quantised matrix is deq(B)[K, N] with groups of
// G along N.  Row k of the packed matrix is N/2 bytes; byte c of that row holds output
// column 2G*(c/G) + c%G in its high nibble and that column + G in its low nibble; the two
// fp16 scales of the byte's block are bs[k][2*(c/G)] and bs[k][2*(c/G)+1].
// (Reference: matmul_q40_kernel, triton_kernels.py:357-469; packing triton_kernels.py:33-39.)
//
// Mapping.  A CTA owns SPAN = 128 packed bytes of every weight row (256 output columns)
// and a contiguous range of k rows; its 4 warps take 16-row steps of that range in turn.
// In a step, lane (g = lane/4, t = lane%4) loads 16 bytes of rows 4t..4t+3 straight into
// registers (one 128-byte line per row per warp), converts the nibbles to exact fp16
// integers with the 0x6400 exponent trick, multiplies by the fp16 scale (so the operand is
// fp16(code*scale), the reference's rounding point) and feeds them as the 16x16 "A" tile of
// mma.m16n8k16 (rows = output columns, fp32 accumulate); the activations are the 16x8 "B"
// tile (8 batch rows per tile, MT tiles).  Which physical k row sits in which k slot of
// the MMA is free as long as both operands agree, which is what lets a lane take four
// consecutive rows.  Nothing is reduced with shuffles inside the loop: the MMA does the
// k reduction in fp32, warps are summed through shared memory and CTAs (split-K) through
// an fp32 workspace where the last CTA to arrive adds the partials in a fixed order, so
// results do not depend on scheduling.
#include <atomic>

#include "q40_common.cuh"

namespace q40 {

constexpr int GEMV_WARPS = 4;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int SPAN_BYTES = 128;            // packed bytes of a weight row per CTA
constexpr int SPAN_COLS = 2 * SPAN_BYTES;  // output columns per CTA
constexpr int STEP_K = 16;
constexpr int XS_PAD = 16;                 // row stride = 32 B mod 128 B: conflict-free 8-byte reads
constexpr int COUNTER_BYTES = 4096;        // workspace header: one arrival counter per span

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Sum of one element over the split-K partials, in split order (so the result does not depend
// on which CTA arrives last) but with eight L2 loads in flight at a time.
__device__ __forceinline__ float sum_partials(const float* __restrict__ p, int stride, int nsplit) {
  float v = 0.f;
  int sp = 0;
  for (; sp + 8 <= nsplit; sp += 8) {
    float t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = __ldcg(p + (int64_t)(sp + i) * stride);
#pragma unroll
    for (int i = 0; i < 8; ++i) v += t[i];
  }
  for (; sp < nsplit; ++sp) v += __ldcg(p + (int64_t)sp * stride);
  return v;
}

struct StepRegs {
  uint4 w[4];      // 16 packed bytes of rows 4t .. 4t+3
  uint32_t s[4];   // (scale of the high-nibble block, scale of the low-nibble block) per row
};

template <int G>
__device__ __forceinline__ void load_step(StepRegs& r, const uint8_t* __restrict__ wcol,
                                          const __half* __restrict__ scol, int64_t w_ld,
                                          int64_t s_ld, int k0, int k_end, bool col_ok) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int k = k0 + i;
    if (col_ok && k < k_end) {
      r.w[i] = __ldg(reinterpret_cast<const uint4*>(wcol + (int64_t)k * w_ld));
      r.s[i] = __ldg(reinterpret_cast<const uint32_t*>(scol + (int64_t)k * s_ld));
    } else {
      r.w[i] = make_uint4(0, 0, 0, 0);
      r.s[i] = 0u;
    }
  }
}

template <int MT>
__device__ __forceinline__ void compute_step(float (&acc)[MT][16][4], const StepRegs& r,
                                             const __half* __restrict__ xrow, int xs_ld) {
  // activations: rows g (and g+8) of the batch, k slots 4t..4t+3 of this step
  uint32_t xb[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const uint2 v = *reinterpret_cast<const uint2*>(xrow + mt * 8 * xs_ld);
    xb[mt][0] = v.x;
    xb[mt][1] = v.y;
  }
  // scales as (row 4t, row 4t+1) and (row 4t+2, row 4t+3) pairs
  const __half2 sh01 = u32_as_h2(prmt(r.s[0], r.s[1], 0x5410));
  const __half2 sl01 = u32_as_h2(prmt(r.s[0], r.s[1], 0x7632));
  const __half2 sh23 = u32_as_h2(prmt(r.s[2], r.s[3], 0x5410));
  const __half2 sl23 = u32_as_h2(prmt(r.s[2], r.s[3], 0x7632));
  const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&r.w[0]);
  const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&r.w[1]);
  const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&r.w[2]);
  const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&r.w[3]);
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      // byte b of the two rows -> bytes 0 and 2 of one register
      const uint32_t sel = (uint32_t)b | ((uint32_t)(4 + b) << 8);
      const uint32_t p01 = prmt(w0[wi], w1[wi], sel);
      const uint32_t p23 = prmt(w2[wi], w3[wi], sel);
      const uint32_t a0 = h2_as_u32(__hmul2(codes_hi_to_h2(p01), sh01));
      const uint32_t a1 = h2_as_u32(__hmul2(codes_lo_to_h2(p01), sl01));
      const uint32_t a2 = h2_as_u32(__hmul2(codes_hi_to_h2(p23), sh23));
      const uint32_t a3 = h2_as_u32(__hmul2(codes_lo_to_h2(p23), sl23));
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) mma16816(acc[mt][wi * 4 + b], a0, a1, a2, a3, xb[mt][0], xb[mt][1]);
    }
  }
}

// Output column of local column id lc (0..255) of span `span`: ids 0..127 are the high
// nibbles of the span's bytes, 128..255 the low nibbles.
template <int G>
__device__ __forceinline__ int span_col(int span, int lc) {
  const int cb = span * SPAN_BYTES + (lc & (SPAN_BYTES - 1));
  return 2 * G * (cb / G) + (cb % G) + ((lc >> 7) ? G : 0);
}

template <int G, int MT>
__global__ void __launch_bounds__(GEMV_THREADS, (MT == 1 ? 3 : 2))
gemv_kn_kernel(const __half* __restrict__ A, int64_t lda, const uint8_t* __restrict__ bw,
               const __half* __restrict__ bs, __half* __restrict__ C, int64_t ldc, int M, int N,
               int K, int kchunk, float* __restrict__ part, unsigned int* __restrict__ counters) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int span = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
  const int kb = split * kchunk;
  const int ke = min(K, kb + kchunk);
  const int xs_ld = kchunk + XS_PAD;

  __half* xs = reinterpret_cast<__half*>(smem_raw);                       // [MT*8][xs_ld]
  float4* slab = reinterpret_cast<float4*>(smem_raw);  // [2][MT][16][32] float4, reuses xs after the loop
  __shared__ unsigned int ticket_s;

  const int64_t w_ld = N / 2, s_ld = N / G;
  const int colbyte = span * SPAN_BYTES + 16 * g;
  const bool col_ok = colbyte < w_ld;
  const uint8_t* wcol = bw + (col_ok ? colbyte : 0);
  const __half* scol = bs + (col_ok ? 2 * (colbyte / G) : 0);

  const int nsteps = (ke - kb + STEP_K - 1) / STEP_K;
  // issue the first weight loads before touching the activations
  StepRegs ra, rb;
  int s = warp;
  if (s < nsteps) load_step<G>(ra, wcol, scol, w_ld, s_ld, kb + s * STEP_K + 4 * t, ke, col_ok);

  // stage the activations of this k range (zero-filled outside [0,M) x [kb,ke))
  for (int idx = tid; idx < MT * 8 * (kchunk / 8); idx += GEMV_THREADS) {
    const int m = idx / (kchunk / 8), kk = (idx % (kchunk / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m < M) {
      const int k = kb + kk;
      if (k + 8 <= ke) {
        v = *reinterpret_cast<const uint4*>(A + (int64_t)m * lda + k);
      } else {
        __half tmp[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) tmp[i] = (k + i < ke) ? A[(int64_t)m * lda + k + i] : __float2half(0.f);
        v = *reinterpret_cast<uint4*>(tmp);
      }
    }
    *reinterpret_cast<uint4*>(xs + m * xs_ld + kk) = v;
  }
  __syncthreads();

  float acc[MT][16][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[mt][i][j] = 0.f;

  const __half* xlane = xs + g * xs_ld + 4 * t;
  // two steps in flight per warp: while one is being converted the next is loading
  for (; s < nsteps; s += 2 * GEMV_WARPS) {
    const int s1 = s + GEMV_WARPS;
    if (s1 < nsteps) load_step<G>(rb, wcol, scol, w_ld, s_ld, kb + s1 * STEP_K + 4 * t, ke, col_ok);
    compute_step<MT>(acc, ra, xlane + s * STEP_K, xs_ld);
    const int s2 = s1 + GEMV_WARPS;
    if (s2 < nsteps) load_step<G>(ra, wcol, scol, w_ld, s_ld, kb + s2 * STEP_K + 4 * t, ke, col_ok);
    if (s1 < nsteps) compute_step<MT>(acc, rb, xlane + s1 * STEP_K, xs_ld);
  }

  // ---- sum the 4 warps: warps 0,1 store, warps 2,3 add ----
  __syncthreads();  // every warp is done reading the activations: the buffer becomes the slabs
  float4* my = slab + (warp & 1) * (MT * 16 * 32);
  if (warp < 2) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 16; ++i)
        my[(mt * 16 + i) * 32 + lane] = make_float4(acc[mt][i][0], acc[mt][i][1], acc[mt][i][2], acc[mt][i][3]);
  }
  __syncthreads();
  if (warp >= 2) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float4 v = my[(mt * 16 + i) * 32 + lane];
        v.x += acc[mt][i][0]; v.y += acc[mt][i][1]; v.z += acc[mt][i][2]; v.w += acc[mt][i][3];
        my[(mt * 16 + i) * 32 + lane] = v;
      }
  }
  __syncthreads();

  // ---- CTA result, indexed (m, local column) ----
  const float* sl0 = reinterpret_cast<const float*>(slab);
  const float* sl1 = reinterpret_cast<const float*>(slab + MT * 16 * 32);
  const int total = M * SPAN_COLS;
  float* mypart = part + ((int64_t)(span * nsplit + split) * M) * SPAN_COLS;
  for (int idx = tid; idx < total; idx += GEMV_THREADS) {
    const int m = idx / SPAN_COLS, lc = idx % SPAN_COLS;
    const int c = lc & 127, is_lo = lc >> 7;
    const int fg = c >> 4, tb = c & 15;
    const int mt = m >> 3, mm = m & 7;
    const int fl = fg * 4 + (mm >> 1);
    const int off = (((mt * 16 + tb) * 32 + fl) << 2) + (mm & 1) + 2 * is_lo;
    const float v = sl0[off] + sl1[off];
    if (nsplit == 1) {
      const int n = span_col<G>(span, lc);
      if (n < N) C[(int64_t)m * ldc + n] = __float2half_rn(v);
    } else {
      mypart[idx] = v;
    }
  }
  if (nsplit == 1) return;

  // ---- split-K: the last CTA of this span adds the partials in split order ----
  __threadfence();
  __syncthreads();
  if (tid == 0) ticket_s = atomicAdd(&counters[span], 1u);
  __syncthreads();
  if (ticket_s != (unsigned)(nsplit - 1)) return;
  __threadfence();
  const float* base = part + ((int64_t)span * nsplit * M) * SPAN_COLS;
  for (int idx = tid; idx < total; idx += GEMV_THREADS) {
    const float v = sum_partials(base + idx, total, nsplit);
    const int m = idx / SPAN_COLS, lc = idx % SPAN_COLS;
    const int n = span_col<G>(span, lc);
    if (n < N) C[(int64_t)m * ldc + n] = __float2half_rn(v);
  }
  if (tid == 0) counters[span] = 0u;  // leave the workspace ready for the next call
}

struct GemvPlan {
  int nspans, nsplit, kchunk;
  size_t smem_bytes(int MT) const {
    const size_t xs = ((size_t)MT * 8 * (kchunk + XS_PAD) * 2 + 15) & ~(size_t)15;
    const size_t slabs = (size_t)2 * MT * 16 * 32 * 16;
    return xs > slabs ? xs : slabs;
  }
};

static GemvPlan plan_kn(int N, int K) {
  GemvPlan p;
  p.nspans = (N / 2 + SPAN_BYTES - 1) / SPAN_BYTES;
  const int target_ctas = 148 * 3;
  int want = (target_ctas + p.nspans - 1) / p.nspans;
  if (want < 1) want = 1;
  int kchunk = (K + want - 1) / want;
  kchunk = ((kchunk + 63) / 64) * 64;          // multiple of 64 keeps the activation rows aligned
  if (kchunk < 64) kchunk = 64;
  if (kchunk > 1024) kchunk = 1024;            // bounds the activation staging buffer
  p.kchunk = kchunk;
  p.nsplit = (K + kchunk - 1) / kchunk;
  return p;
}


// ---------------------------------------------------------------------------------------
// Orientation "nk": W[N, K] quantised along K (quantize.py:217-223).  Row n of the packed
// matrix is K/2 bytes; byte c holds k = 2G*(c/G) + c%G (high nibble) and that k + G (low).
// A warp owns 16 consecutive output rows (the MMA "A" rows) and walks the CTA's k range in
// steps of 64 packed bytes per row (128 k values): lane (g,t) loads 16 bytes of rows g and
// g+8.  The four high nibbles of a 32-bit word are k0, k0+1, k0+2, k0+3; the exponent trick
// yields (k0,k0+2) and (k0+1,k0+3) as half2 without byte shuffles, so the activations are
// staged in shared memory in the matching order [x0,x2,x1,x3] and no permute is needed
// at all.  Warps do not share outputs; only split-K CTAs are summed (as in the kn kernel).
// ---------------------------------------------------------------------------------------
constexpr int NK_ROWS = 64;       // output rows per CTA (16 per warp)
constexpr int NK_STEP_BYTES = 64; // packed bytes per row per step
constexpr int NK_STEP_K = 128;
constexpr int NK_XS_PAD = 4;      // row stride = 8 B mod 128 B

struct NkRegs {
  uint4 w[2];      // rows g and g+8
  uint32_t s[2];   // their (high block, low block) scales
};

template <int G>
__device__ __forceinline__ void nk_load(NkRegs& r, const uint8_t* __restrict__ w0, const uint8_t* __restrict__ w1,
                                        const __half* __restrict__ s0, const __half* __restrict__ s1,
                                        int cb, bool ok0, bool ok1) {
  // cb: byte offset of this lane's 16 bytes inside the packed row
  const int sidx = 2 * (cb / G);
  if (ok0) {
    r.w[0] = __ldg(reinterpret_cast<const uint4*>(w0 + cb));
    r.s[0] = __ldg(reinterpret_cast<const uint32_t*>(s0 + sidx));
  } else { r.w[0] = make_uint4(0, 0, 0, 0); r.s[0] = 0u; }
  if (ok1) {
    r.w[1] = __ldg(reinterpret_cast<const uint4*>(w1 + cb));
    r.s[1] = __ldg(reinterpret_cast<const uint32_t*>(s1 + sidx));
  } else { r.w[1] = make_uint4(0, 0, 0, 0); r.s[1] = 0u; }
}

template <int G, int MT>
__device__ __forceinline__ void nk_compute(float (&acc)[MT][4], const NkRegs& r,
                                           const __half* __restrict__ xhi, int xs_ld) {
  // xhi points at this lane's activations for the high nibbles of word 0; low nibbles are G further
  const __half2 sh0 = u32_as_h2(prmt(r.s[0], r.s[0], 0x1010)), sl0 = u32_as_h2(prmt(r.s[0], r.s[0], 0x3232));
  const __half2 sh1 = u32_as_h2(prmt(r.s[1], r.s[1], 0x1010)), sl1 = u32_as_h2(prmt(r.s[1], r.s[1], 0x3232));
  const uint32_t* wa = reinterpret_cast<const uint32_t*>(&r.w[0]);
  const uint32_t* wb = reinterpret_cast<const uint32_t*>(&r.w[1]);
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    const uint32_t a = wa[wi], b = wb[wi];
    const uint32_t a8 = a >> 8, b8 = b >> 8;
    // high nibbles: k0 + {0,2 | 1,3}
    {
      const uint32_t f0 = h2_as_u32(__hmul2(codes_hi_to_h2(a), sh0));
      const uint32_t f1 = h2_as_u32(__hmul2(codes_hi_to_h2(b), sh1));
      const uint32_t f2 = h2_as_u32(__hmul2(codes_hi_to_h2(a8), sh0));
      const uint32_t f3 = h2_as_u32(__hmul2(codes_hi_to_h2(b8), sh1));
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint2 xv = *reinterpret_cast<const uint2*>(xhi + mt * 8 * xs_ld + 4 * wi);
        mma16816(acc[mt], f0, f1, f2, f3, xv.x, xv.y);
      }
    }
    // low nibbles: the same positions G further along k
    {
      const uint32_t f0 = h2_as_u32(__hmul2(codes_lo_to_h2(a), sl0));
      const uint32_t f1 = h2_as_u32(__hmul2(codes_lo_to_h2(b), sl1));
      const uint32_t f2 = h2_as_u32(__hmul2(codes_lo_to_h2(a8), sl0));
      const uint32_t f3 = h2_as_u32(__hmul2(codes_lo_to_h2(b8), sl1));
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint2 xv = *reinterpret_cast<const uint2*>(xhi + mt * 8 * xs_ld + G + 4 * wi);
        mma16816(acc[mt], f0, f1, f2, f3, xv.x, xv.y);
      }
    }
  }
}

template <int G, int MT>
__global__ void __launch_bounds__(GEMV_THREADS, 4)
gemv_nk_kernel(const __half* __restrict__ X, int64_t ldx, const uint8_t* __restrict__ wq,
               const __half* __restrict__ ws, __half* __restrict__ Y, int64_t ldy, int M, int N, int K,
               int kchunk, float* __restrict__ part, unsigned int* __restrict__ counters) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);   // [MT*8][kchunk + pad], order x0,x2,x1,x3
  __shared__ unsigned int ticket_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int nblk = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
  const int kb = split * kchunk, ke = min(K, kb + kchunk);
  const int xs_ld = kchunk + NK_XS_PAD;
  const int n0 = nblk * NK_ROWS + warp * 16 + g, n1 = n0 + 8;
  const bool ok0 = n0 < N, ok1 = n1 < N;
  const int64_t w_ld = K / 2, s_ld = K / G;
  const uint8_t* w0 = wq + (int64_t)(ok0 ? n0 : 0) * w_ld;
  const uint8_t* w1 = wq + (int64_t)(ok1 ? n1 : 0) * w_ld;
  const __half* s0 = ws + (int64_t)(ok0 ? n0 : 0) * s_ld;
  const __half* s1 = ws + (int64_t)(ok1 ? n1 : 0) * s_ld;
  const int nsteps = (ke - kb) / NK_STEP_K;            // K and kchunk are multiples of 128
  const int cb0 = kb / 2 + 16 * t;

  constexpr int DEPTH = 4;
  NkRegs regs[DEPTH];
#pragma unroll
  for (int d = 0; d < DEPTH; ++d)
    if (d < nsteps) nk_load<G>(regs[d], w0, w1, s0, s1, cb0 + d * NK_STEP_BYTES, ok0, ok1);

  for (int idx = tid; idx < MT * 8 * (kchunk / 4); idx += GEMV_THREADS) {
    const int m = idx / (kchunk / 4), kk = (idx % (kchunk / 4)) * 4;
    uint2 v = make_uint2(0, 0);
    if (m < M && kb + kk < ke) {
      const uint2 raw = *reinterpret_cast<const uint2*>(X + (int64_t)m * ldx + kb + kk);  // x0 x1 | x2 x3
      v.x = prmt(raw.x, raw.y, 0x5410);   // x0 x2
      v.y = prmt(raw.x, raw.y, 0x7632);   // x1 x3
    }
    *reinterpret_cast<uint2*>(xs + m * xs_ld + kk) = v;
  }
  __syncthreads();

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[mt][j] = 0.f;

  // position of this lane's first high-nibble k inside a step: byte 16t of the step -> k offset
  const int koff = 2 * G * ((16 * t) / G) + (16 * t) % G;
  const __half* xlane = xs + g * xs_ld + koff;
  for (int s = 0; s < nsteps; s += DEPTH) {
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (s + d < nsteps) {
        nk_compute<G, MT>(acc, regs[d], xlane + (s + d) * NK_STEP_K, xs_ld);
        if (s + d + DEPTH < nsteps)
          nk_load<G>(regs[d], w0, w1, s0, s1, cb0 + (s + d + DEPTH) * NK_STEP_BYTES, ok0, ok1);
      }
    }
  }

  // acc[mt][0..1]: row n0, batch 8mt+2t, +1 ; acc[mt][2..3]: row n1
  const int nloc0 = warp * 16 + g;
  if (nsplit == 1) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = mt * 8 + 2 * t + (j & 1);
        const int n = (j < 2) ? n0 : n1;
        if (m < M && n < N) Y[(int64_t)m * ldy + n] = __float2half_rn(acc[mt][j]);
      }
    return;
  }
  float* mypart = part + ((int64_t)(nblk * nsplit + split) * M) * NK_ROWS;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = mt * 8 + 2 * t + (j & 1);
      if (m < M) mypart[m * NK_ROWS + nloc0 + ((j < 2) ? 0 : 8)] = acc[mt][j];
    }
  __threadfence();
  __syncthreads();
  if (tid == 0) ticket_s = atomicAdd(&counters[nblk], 1u);
  __syncthreads();
  if (ticket_s != (unsigned)(nsplit - 1)) return;
  __threadfence();
  const int total = M * NK_ROWS;
  const float* base = part + ((int64_t)nblk * nsplit * M) * NK_ROWS;
  for (int idx = tid; idx < total; idx += GEMV_THREADS) {
    const float v = sum_partials(base + idx, total, nsplit);
    const int m = idx / NK_ROWS, n = nblk * NK_ROWS + idx % NK_ROWS;
    if (n < N) Y[(int64_t)m * ldy + n] = __float2half_rn(v);
  }
  if (tid == 0) counters[nblk] = 0u;
}

struct NkPlan {
  int nblocks, nsplit, kchunk;
  size_t smem_bytes(int MT) const { return ((size_t)MT * 8 * (kchunk + NK_XS_PAD) * 2 + 15) & ~(size_t)15; }
};

static NkPlan plan_nk(int N, int K) {
  NkPlan p;
  p.nblocks = (N + NK_ROWS - 1) / NK_ROWS;
  int want = (148 * 4 + p.nblocks - 1) / p.nblocks;
  if (want < 1) want = 1;
  int kchunk = (K + want - 1) / want;
  kchunk = ((kchunk + NK_STEP_K - 1) / NK_STEP_K) * NK_STEP_K;
  if (kchunk < 256) kchunk = 256;
  if (kchunk > 2048) kchunk = 2048;
  if (kchunk > K) kchunk = K;
  p.kchunk = kchunk;
  p.nsplit = (K + kchunk - 1) / kchunk;
  return p;
}

}  // namespace q40

extern "C" int q40_gemm_kn_tc(const void* a, int64_t lda, const void* bw, const void* bs, void* c, int64_t ldc,
                              int M, int N, int K, int* err, void* stream);

extern "C" size_t q40_gemm_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const q40::GemvPlan p = q40::plan_kn(N, K);
  const int mrows = M < 16 ? M : 16;
  const size_t kn = (size_t)p.nspans * p.nsplit * mrows * q40::SPAN_COLS * sizeof(float);
  size_t nk = 0;
  if (K % 128 == 0) {
    const q40::NkPlan pn = q40::plan_nk(N, K);
    nk = (size_t)pn.nblocks * pn.nsplit * mrows * q40::NK_ROWS * sizeof(float);
  }
  return q40::COUNTER_BYTES + (kn > nk ? kn : nk);
}

template <int G, int MT>
static int launch_gemv_kn(const __half* a, int64_t lda, const uint8_t* bw, const __half* bs, __half* c,
                          int64_t ldc, int M, int N, int K, const q40::GemvPlan& p, void* workspace,
                          cudaStream_t st) {
  const size_t smem = p.smem_bytes(MT);
  auto kern = q40::gemv_kn_kernel<G, MT>;
  dim3 grid(p.nspans, p.nsplit);
  kern<<<grid, q40::GEMV_THREADS, smem, st>>>(
      a, lda, bw, bs, c, ldc, M, N, K, p.kchunk,
      reinterpret_cast<float*>((char*)workspace + q40::COUNTER_BYTES),
      reinterpret_cast<unsigned int*>(workspace));
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}

extern "C" int q40_gemm_kn(const void* a, int64_t lda, const void* bw, const void* bs, void* c,
                           int64_t ldc, int M, int N, int K, int group, void* workspace,
                           size_t workspace_bytes, void* stream) {
  if (!a || !bw || !bs || !c) return Q40_E_NULL;
  if (group != 64 && group != 32) return Q40_E_UNSUPPORTED;
  if (M < 0 || N <= 0 || K <= 0 || N % (2 * group) != 0) return Q40_E_SHAPE;
  if (M == 0) return Q40_OK;
  if (lda < K || ldc < N || lda % 8 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(a, 16) || !q40_aligned(bw, 16) || !q40_aligned(bs, 4) || !q40_aligned(c, 2))
    return Q40_E_ALIGN;
  if ((N / 2) % 16 != 0) return Q40_E_SHAPE;
  const q40::GemvPlan p = q40::plan_kn(N, K);
  if (p.nspans * 4 > q40::COUNTER_BYTES) return Q40_E_SHAPE;
  if (p.nsplit > 1) {
    if (!workspace) return Q40_E_WORKSPACE;
    if (workspace_bytes < q40_gemm_workspace_bytes(M, N, K)) return Q40_E_WORKSPACE;
    if (!q40_aligned(workspace, 16)) return Q40_E_ALIGN;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const __half* ah = (const __half*)a;
  __half* ch = (__half*)c;
  // batches above 16 rows go to the tcgen05 kernel when the shape allows it; its error word is the
  // last int of the (zeroed) counter header of the workspace
  if (M > 16 && group == 64 && K % 64 == 0 && N % 128 == 0 && ldc % 2 == 0 && lda % 8 == 0 && workspace && workspace_bytes >= (size_t)q40::COUNTER_BYTES &&
      p.nspans * 4 <= q40::COUNTER_BYTES - 4)
    return q40_gemm_kn_tc(a, lda, bw, bs, c, ldc, M, N, K,
                          reinterpret_cast<int*>((char*)workspace + q40::COUNTER_BYTES - 4), stream);
  // otherwise batches above 16 rows are processed 16 rows at a time
  for (int m0 = 0; m0 < M; m0 += 16) {
    const int mc = (M - m0) < 16 ? (M - m0) : 16;
    int rc;
    if (group == 64) {
      rc = (mc <= 8) ? launch_gemv_kn<64, 1>(ah + m0 * lda, lda, (const uint8_t*)bw, (const __half*)bs,
                                            ch + m0 * ldc, ldc, mc, N, K, p, workspace, st)
                     : launch_gemv_kn<64, 2>(ah + m0 * lda, lda, (const uint8_t*)bw, (const __half*)bs,
                                            ch + m0 * ldc, ldc, mc, N, K, p, workspace, st);
    } else {
      rc = (mc <= 8) ? launch_gemv_kn<32, 1>(ah + m0 * lda, lda, (const uint8_t*)bw, (const __half*)bs,
                                            ch + m0 * ldc, ldc, mc, N, K, p, workspace, st)
                     : launch_gemv_kn<32, 2>(ah + m0 * lda, lda, (const uint8_t*)bw, (const __half*)bs,
                                            ch + m0 * ldc, ldc, mc, N, K, p, workspace, st);
    }
    if (rc != Q40_OK) return rc;
  }
  return Q40_OK;
}

template <int G, int MT>
static int launch_gemv_nk(const __half* x, int64_t ldx, const uint8_t* wq, const __half* ws, __half* y,
                          int64_t ldy, int M, int N, int K, const q40::NkPlan& p, void* workspace,
                          cudaStream_t st) {
  const size_t smem = p.smem_bytes(MT);
  auto kern = q40::gemv_nk_kernel<G, MT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(p.nblocks, p.nsplit);
  kern<<<grid, q40::GEMV_THREADS, smem, st>>>(
      x, ldx, wq, ws, y, ldy, M, N, K, p.kchunk,
      reinterpret_cast<float*>((char*)workspace + q40::COUNTER_BYTES),
      reinterpret_cast<unsigned int*>(workspace));
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}

extern "C" int q40_gemm_nk(const void* x, int64_t ldx, const void* wq, const void* ws, void* y,
                           int64_t ldy, int M, int N, int K, int group, void* workspace,
                           size_t workspace_bytes, void* stream) {
  if (!x || !wq || !ws || !y) return Q40_E_NULL;
  if (group != 64 && group != 32) return Q40_E_UNSUPPORTED;
  // the packer pairs groups over the flattened [N*K] tensor; K % (2*group) == 0 keeps pairs inside a
  // row, and the kernel walks rows in 128-wide k steps
  if (M < 0 || N <= 0 || K <= 0 || K % 128 != 0) return Q40_E_SHAPE;
  if (M == 0) return Q40_OK;
  if (ldx < K || ldy < N || ldx % 4 != 0) return Q40_E_SHAPE;
  if (!q40_aligned(x, 8) || !q40_aligned(wq, 16) || !q40_aligned(ws, 4) || !q40_aligned(y, 2))
    return Q40_E_ALIGN;
  const q40::NkPlan p = q40::plan_nk(N, K);
  if (p.nblocks * 4 > q40::COUNTER_BYTES) return Q40_E_SHAPE;
  if (p.nsplit > 1) {
    if (!workspace) return Q40_E_WORKSPACE;
    if (workspace_bytes < q40_gemm_workspace_bytes(M, N, K)) return Q40_E_WORKSPACE;
    if (!q40_aligned(workspace, 16)) return Q40_E_ALIGN;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const __half* xh = (const __half*)x;
  __half* yh = (__half*)y;
  for (int m0 = 0; m0 < M; m0 += 16) {
    const int mc = (M - m0) < 16 ? (M - m0) : 16;
    int rc;
    if (group == 64) {
      rc = (mc <= 8) ? launch_gemv_nk<64, 1>(xh + m0 * ldx, ldx, (const uint8_t*)wq, (const __half*)ws,
                                            yh + m0 * ldy, ldy, mc, N, K, p, workspace, st)
                     : launch_gemv_nk<64, 2>(xh + m0 * ldx, ldx, (const uint8_t*)wq, (const __half*)ws,
                                            yh + m0 * ldy, ldy, mc, N, K, p, workspace, st);
    } else {
      rc = (mc <= 8) ? launch_gemv_nk<32, 1>(xh + m0 * ldx, ldx, (const uint8_t*)wq, (const __half*)ws,
                                            yh + m0 * ldy, ldy, mc, N, K, p, workspace, st)
                     : launch_gemv_nk<32, 2>(xh + m0 * ldx, ldx, (const uint8_t*)wq, (const __half*)ws,
                                            yh + m0 * ldy, ldy, mc, N, K, p, workspace, st);
    }
    if (rc != Q40_OK) return rc;
  }
  return Q40_OK;
}

// ---------------------------------------------------------------------------------------
// q40_gemm_kn_static: q40_gemm_kn for callers that cannot hand over a workspace.
//
// Some hosts of this library own no allocator of their own on the device: a serving process
// that handed every byte of HBM to its memory planner at start-up, or a plug-in that is only
// given input and output buffers by the runtime that loads it.  For them the split-K scratch
// lives inside the library, in the fixed-size device array below.  Every GPU that loads the
// library carries these Q40_STATIC_WS_BYTES until the process exits; problems whose scratch
// need is larger are refused with Q40_E_WORKSPACE (use q40_gemm_kn with your own buffer).
//
// The array's name is only a handle on the host side; the kernels need its device address,
// which is looked up once per device (cudaGetSymbolAddress, with that device current) by the
// first call made on that device.  That first call also does nothing else unusual, but
// because it performs this look-up it should be made before any stream capture is begun.
// All calls share the one array: the arrival counters at its start are cleared on the
// stream before every launch, the partial sums behind them are fully overwritten before
// they are read, and two calls that overlap on the GPU (different streams) would race.
// The array is picked by the CURRENT device (cudaGetDevice), which must be the device `stream`
// belongs to.  Above 16 rows the tcgen05 kernel reports an expired bounded wait in the last word of
// the array's 4096-byte header; q40_gemm_kn_static_error copies that word to the host.
// Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
// ---------------------------------------------------------------------------------------
#define Q40_STATIC_WS_BYTES (8u * 1024u * 1024u)

static __device__ __align__(256) unsigned char q40_static_ws[Q40_STATIC_WS_BYTES];

// device address of the array per device ordinal; null = not looked up yet.  Two host threads that make
// the first call on a device at the same time both resolve the same address; the store/load pair only
// makes that formally race-free.
static std::atomic<void*> q40_static_ws_ptr[64];

extern "C" size_t q40_gemm_kn_static_max_workspace(void) { return (size_t)Q40_STATIC_WS_BYTES; }

static int q40_static_ws_lookup(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return Q40_E_UNSUPPORTED;
  void* ptr = q40_static_ws_ptr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    e = cudaGetSymbolAddress(&ptr, q40_static_ws);
    if (e != cudaSuccess) return (int)e;
    q40_static_ws_ptr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return Q40_OK;
}

extern "C" int q40_gemm_kn_static(const void* a, int64_t lda, const void* bw, const void* bs, void* c,
                                  int64_t ldc, int M, int N, int K, int group, void* stream) {
  if (M > 0 && N > 0 && K > 0 && q40_gemm_workspace_bytes(M, N, K) > (size_t)Q40_STATIC_WS_BYTES)
    return Q40_E_WORKSPACE;
  void* ws = nullptr;
  const int rc = q40_static_ws_lookup(&ws);
  if (rc != Q40_OK) return rc;
  // the arrival counters must read zero when a launch starts, whatever an earlier call left behind; the
  // last word of the header is the tensor-core kernel's error word (above 16 rows), which is sticky: it
  // is read and cleared only through q40_gemm_kn_static_error
  const cudaError_t e = cudaMemsetAsync(ws, 0, q40::COUNTER_BYTES - 4, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return q40_gemm_kn(a, lda, bw, bs, c, ldc, M, N, K, group, ws, (size_t)Q40_STATIC_WS_BYTES, stream);
}

extern "C" int q40_gemm_kn_static_error(int* host_out, int clear, void* stream) {
  if (!host_out) return Q40_E_NULL;
  void* ws = nullptr;
  const int rc = q40_static_ws_lookup(&ws);
  if (rc != Q40_OK) return rc;
  char* word = (char*)ws + q40::COUNTER_BYTES - 4;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(host_out, word, 4, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess && clear) e = cudaMemsetAsync(word, 0, 4, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  return e == cudaSuccess ? Q40_OK : (int)e;
}
