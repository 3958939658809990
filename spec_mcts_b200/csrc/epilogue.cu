// Element-wise pieces of a decode step, with the reference model's rounding points
// (hf_model_q40_kv_shared.py:123-134 RMSNorm, :166-203 rotary embedding, :434 SiLU-mul,
// :463-466 residual adds).  All HBM/L2-bound and tiny at decode batch sizes.
#include "q40_common.cuh"

namespace q40 {

// One CTA per row.  h = fp16(x + residual) (optional), y = fp16(fp16(h32 * rsqrt(mean(h32^2)+eps)) * w)
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ residual,
               const __half* __restrict__ w, __half* __restrict__ y, __half* __restrict__ h_out,
               int dim, float eps) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* row = reinterpret_cast<__half*>(smem_raw);  // [dim]
  __shared__ float red[8];
  asm volatile("griddepcontrol.launch_dependents;");   // a dependent may start prefetching its weights
  asm volatile("griddepcontrol.wait;" ::: "memory");               // ... but nothing of the previous launch is read before it is done
  const int r = blockIdx.x, tid = threadIdx.x;
  const __half* xr = x + (int64_t)r * dim;
  const __half* rr = residual ? residual + (int64_t)r * dim : nullptr;
  float ss = 0.f;
  for (int i = tid * 8; i < dim; i += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    __half2* vh = reinterpret_cast<__half2*>(&v);
    if (rr) {
      uint4 u = *reinterpret_cast<const uint4*>(rr + i);
      const __half2* uh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) vh[j] = __hadd2(vh[j], uh[j]);  // fp16 add, one rounding
      if (h_out) *reinterpret_cast<uint4*>(h_out + (int64_t)r * dim + i) = v;
    }
    *reinterpret_cast<uint4*>(row + i) = v;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(vh[j]);
      ss = fmaf(f.x, f.x, ss);
      ss = fmaf(f.y, f.y, ss);
    }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)dim + eps);
  for (int i = tid * 8; i < dim; i += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(row + i);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + i);
    __half2* vh = reinterpret_cast<__half2*>(&v);
    const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(vh[j]);
      const __half2 n = __floats2half2_rn(f.x * inv, f.y * inv);  // round to fp16 first
      vh[j] = __hmul2(n, wh[j]);                                   // then * weight in fp16
    }
    *reinterpret_cast<uint4*>(y + (int64_t)r * dim + i) = v;
  }
}

// One thread per (row, head, d < D/2): handles the pair (d, d + D/2).
__global__ void __launch_bounds__(256)
rope_kernel(__half* __restrict__ x, const int32_t* __restrict__ pos, const __half* __restrict__ cos_tbl,
            const __half* __restrict__ sin_tbl, int rows, int n_heads, int D, int64_t row_stride) {
  const int half_d = D / 2;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)rows * n_heads * half_d;
  if (idx >= total) return;
  const int d = (int)(idx % half_d);
  const int h = (int)((idx / half_d) % n_heads);
  const int r = (int)(idx / ((int64_t)half_d * n_heads));
  const int p = pos[r];
  const __half c = cos_tbl[(int64_t)p * half_d + d];
  const __half s = sin_tbl[(int64_t)p * half_d + d];
  __half* px = x + (int64_t)r * row_stride + (int64_t)h * D + d;
  const __half x1 = px[0], x2 = px[half_d];
  // q*cos + rotate_half(q)*sin, every operation rounded to fp16 (the _rn forms are never
  // contracted into a fused multiply-add)
  px[0] = __hadd_rn(__hmul_rn(x1, c), __hmul_rn(__hneg(x2), s));
  px[half_d] = __hadd_rn(__hmul_rn(x2, c), __hmul_rn(x1, s));
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half* __restrict__ a, const __half* __restrict__ b, __half* __restrict__ y,
                int64_t n) {
  asm volatile("griddepcontrol.launch_dependents;");   // a dependent may start prefetching its weights
  asm volatile("griddepcontrol.wait;" ::: "memory");               // ... but nothing of the previous launch is read before it is done
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  if (i + 8 <= n) {
    uint4 av = *reinterpret_cast<const uint4*>(a + i);
    const uint4 bv = *reinterpret_cast<const uint4*>(b + i);
    __half2* ah = reinterpret_cast<__half2*>(&av);
    const __half2* bh = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(ah[j]);
      const __half2 s = __floats2half2_rn(f.x / (1.0f + expf(-f.x)), f.y / (1.0f + expf(-f.y)));
      ah[j] = __hmul2(s, bh[j]);
    }
    *reinterpret_cast<uint4*>(y + i) = av;
  } else {
    for (int64_t j = i; j < n; ++j) {
      const float f = __half2float(a[j]);
      y[j] = __hmul(__float2half_rn(f / (1.0f + expf(-f))), b[j]);
    }
  }
}

// One CTA per row: h[r] = emb[token[r]] and the row's sum of squares in ss[r][0] (ss[r][1..] = 0),
// the form in which the fused decode matmuls expect it.
__global__ void __launch_bounds__(256)
embed_rows_kernel(const __half* __restrict__ emb, const int64_t* __restrict__ tokens, __half* __restrict__ h,
                  float* __restrict__ ss, int ss_count, int dim, int vocab) {
  __shared__ float red[8];
  asm volatile("griddepcontrol.launch_dependents;");
  const int r = blockIdx.x, tid = threadIdx.x;
  int64_t tok = tokens[r];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const __half* src = emb + tok * dim;
  float s = 0.f;
  for (int i = tid * 8; i < dim; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + i);
    *reinterpret_cast<uint4*>(h + (int64_t)r * dim + i) = v;
    const __half2* vh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(vh[j]);
      s = fmaf(f.x, f.x, s);
      s = fmaf(f.y, f.y, s);
    }
  }
  s = warp_sum(s);
  if ((tid & 31) == 0) red[tid >> 5] = s;
  __syncthreads();
  for (int i = tid; i < ss_count; i += blockDim.x) {
    float tot = 0.f;
    if (i == 0)
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
    ss[(int64_t)r * ss_count + i] = tot;
  }
}

}  // namespace q40

extern "C" int q40_embed_rows(const void* emb, const int64_t* tokens, void* h, float* ss, int ss_count,
                              int rows, int dim, int vocab, void* stream) {
  if (!emb || !tokens || !h || !ss) return Q40_E_NULL;
  if (rows < 0 || dim <= 0 || dim % 8 != 0 || vocab <= 0 || ss_count < 1) return Q40_E_SHAPE;
  if (rows == 0) return Q40_OK;
  if (!q40_aligned(emb, 16) || !q40_aligned(h, 16)) return Q40_E_ALIGN;
  q40::embed_rows_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>((const __half*)emb, tokens, (__half*)h, ss,
                                                              ss_count, dim, vocab);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}

extern "C" int q40_rmsnorm(const void* x, const void* residual, const void* w, void* y, void* h_out,
                           int rows, int dim, float eps, void* stream) {
  if (!x || !w || !y) return Q40_E_NULL;
  if (rows < 0 || dim <= 0 || dim % 8 != 0 || dim > 65536) return Q40_E_SHAPE;
  if (rows == 0) return Q40_OK;
  if (!q40_aligned(x, 16) || !q40_aligned(w, 16) || !q40_aligned(y, 16) ||
      (residual && !q40_aligned(residual, 16)) || (h_out && !q40_aligned(h_out, 16)))
    return Q40_E_ALIGN;
  const size_t smem = (size_t)dim * 2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(q40::rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const cudaError_t e2 = q40_launch_pdl(q40::rmsnorm_kernel, dim3(rows), dim3(256), smem, (cudaStream_t)stream,
                                        (const __half*)x, (const __half*)residual, (const __half*)w, (__half*)y,
                                        (__half*)h_out, dim, eps);
  if (e2 != cudaSuccess) return (int)e2;
  return Q40_OK;
}

extern "C" int q40_rope(void* x, const int32_t* pos, const void* cos_tbl, const void* sin_tbl, int rows,
                        int n_heads, int D, int64_t row_stride, void* stream) {
  if (!x || !pos || !cos_tbl || !sin_tbl) return Q40_E_NULL;
  if (rows < 0 || n_heads <= 0 || D <= 0 || D % 2 != 0 || row_stride < (int64_t)n_heads * D)
    return Q40_E_SHAPE;
  if (rows == 0) return Q40_OK;
  const int64_t total = (int64_t)rows * n_heads * (D / 2);
  const int64_t grid = (total + 255) / 256;
  if (grid > 0x7fffffffLL) return Q40_E_SHAPE;
  q40::rope_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(
      (__half*)x, pos, (const __half*)cos_tbl, (const __half*)sin_tbl, rows, n_heads, D, row_stride);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}

extern "C" int q40_silu_mul(const void* a, const void* b, void* y, int64_t n, void* stream) {
  if (!a || !b || !y) return Q40_E_NULL;
  if (n < 0) return Q40_E_SHAPE;
  if (n == 0) return Q40_OK;
  if (!q40_aligned(a, 16) || !q40_aligned(b, 16) || !q40_aligned(y, 16)) return Q40_E_ALIGN;
  const int64_t threads = (n + 7) / 8;
  const int64_t grid = (threads + 255) / 256;
  if (grid > 0x7fffffffLL) return Q40_E_SHAPE;
  const cudaError_t e = q40_launch_pdl(q40::silu_mul_kernel, dim3((unsigned)grid), dim3(256), 0, (cudaStream_t)stream,
                                       (const __half*)a, (const __half*)b, (__half*)y, n);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}
