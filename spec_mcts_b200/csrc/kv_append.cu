// Rotary embedding of the new token's q and k, and append of its K/V to the Q4_0 suffix
// cache, as one launch that reads the position from device memory (so a captured CUDA
// graph can be replayed for every decode step).
//
// Reference behaviour being reproduced (hf_model_q40_kv_shared.py:313-317, 331-371): q and k
// get the rotary embedding in fp16; the step that produces a token attends to its K/V
// un-quantised, and what is stored for later steps is the Q4_0 (group 64 along head_dim)
// quantisation of those fp16 rows: one 64-byte packed row and two fp16 scales per
// (branch, position, kv head): high nibble = dims 0..63, low nibble = dims 64..127.
#include "q40_common.cuh"

namespace q40 {

struct AppendArgs {
  __half* q;               // [B, H*D], rotated in place
  __half* k;               // [B, Hkv*D], rotated in place (stays un-quantised for this step)
  const __half* v;         // [B, Hkv*D]
  int64_t q_stride, k_stride, v_stride;   // row strides in elements
  const int32_t* pos;      // [B] absolute position of the new token
  const int32_t* prefix_len;  // device scalar: tokens held in the shared prompt cache
  const __half* cos_tbl;   // [n_pos, D/2]
  const __half* sin_tbl;
  int8_t* cache_kq;        // [maxB, maxT, Hkv, 64]
  __half* cache_ks;        // [maxB, maxT, Hkv, 2]
  int8_t* cache_vq;
  __half* cache_vs;
  int H, Hkv, max_t, n_pos;
};

__device__ __forceinline__ float block64_max(float v, float* red, int tid) {
  v = warp_max(v);
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  const float r = fmaxf(red[0], red[1]);
  __syncthreads();
  return r;
}

// scale and code exactly as the packer: scale = fp16(absmax/7); code = int8(rint(fp16(x/scale)))
__device__ __forceinline__ int q40_code(__half x, float scale_f) {
  float qv = __half2float(__float2half_rn(__fdiv_rn(__half2float(x), scale_f)));
  qv = rintf(qv);
  const int c = (fabsf(qv) <= 65504.0f) ? (int)qv : 0;
  return (int)(int8_t)c;
}

// grid (B, H + Hkv), 64 threads: thread d owns dims d and d + 64 of one head.
__global__ void __launch_bounds__(64)
rope_kv_append_kernel(const AppendArgs a) {
  constexpr int D = 128, HD = 64;
  __shared__ float red[2];
  asm volatile("griddepcontrol.launch_dependents;");   // a dependent may start prefetching its weights
  asm volatile("griddepcontrol.wait;" ::: "memory");               // ... but nothing of the previous launch is read before it is done
  const int b = blockIdx.x, hh = blockIdx.y, d = threadIdx.x;
  int p = a.pos[b];
  p = min(max(p, 0), a.n_pos - 1);
  const __half c = a.cos_tbl[(int64_t)p * HD + d];
  const __half s = a.sin_tbl[(int64_t)p * HD + d];
  if (hh < a.H) {   // a query head: rotate only
    __half* px = a.q + (int64_t)b * a.q_stride + hh * D + d;
    const __half x1 = px[0], x2 = px[HD];
    px[0] = __hadd_rn(__hmul_rn(x1, c), __hmul_rn(__hneg(x2), s));
    px[HD] = __hadd_rn(__hmul_rn(x2, c), __hmul_rn(x1, s));
    return;
  }
  const int hk = hh - a.H;
  __half* pk = a.k + (int64_t)b * a.k_stride + hk * D + d;
  const __half k1 = pk[0], k2 = pk[HD];
  const __half r1 = __hadd_rn(__hmul_rn(k1, c), __hmul_rn(__hneg(k2), s));
  const __half r2 = __hadd_rn(__hmul_rn(k2, c), __hmul_rn(k1, s));
  pk[0] = r1;
  pk[HD] = r2;
  const __half* pv = a.v + (int64_t)b * a.v_stride + hk * D + d;
  const __half v1 = pv[0], v2 = pv[HD];

  const int t = p - a.prefix_len[0];
  if (t < 0 || t >= a.max_t) return;    // uniform per block: no barrier is skipped by part of it
  const int64_t row = ((int64_t)b * a.max_t + t) * a.Hkv + hk;

  const float mk1 = block64_max(fabsf(__half2float(r1)), red, d);
  const float mk2 = block64_max(fabsf(__half2float(r2)), red, d);
  const float mv1 = block64_max(fabsf(__half2float(v1)), red, d);
  const float mv2 = block64_max(fabsf(__half2float(v2)), red, d);
  const __half sk1 = __float2half_rn(__fdiv_rn(mk1, 7.0f)), sk2 = __float2half_rn(__fdiv_rn(mk2, 7.0f));
  const __half sv1 = __float2half_rn(__fdiv_rn(mv1, 7.0f)), sv2 = __float2half_rn(__fdiv_rn(mv2, 7.0f));
  const int ck1 = q40_code(r1, __half2float(sk1)), ck2 = q40_code(r2, __half2float(sk2));
  const int cv1 = q40_code(v1, __half2float(sv1)), cv2 = q40_code(v2, __half2float(sv2));
  a.cache_kq[row * 64 + d] = (int8_t)(((ck1 << 4) | (ck2 & 0xF)) & 0xFF);
  a.cache_vq[row * 64 + d] = (int8_t)(((cv1 << 4) | (cv2 & 0xF)) & 0xFF);
  if (d == 0) {
    *reinterpret_cast<__half2*>(a.cache_ks + row * 2) = __halves2half2(sk1, sk2);
    *reinterpret_cast<__half2*>(a.cache_vs + row * 2) = __halves2half2(sv1, sv2);
  }
}

}  // namespace q40

extern "C" int q40_rope_kv_append(void* q, int64_t q_stride, void* k, int64_t k_stride, const void* v,
                                  int64_t v_stride, const int32_t* pos, const int32_t* prefix_len,
                                  const void* cos_tbl, const void* sin_tbl, int n_pos, void* cache_kq,
                                  void* cache_ks, void* cache_vq, void* cache_vs, int B, int H, int Hkv,
                                  int D, int max_t, void* stream) {
  if (!q || !k || !v || !pos || !prefix_len || !cos_tbl || !sin_tbl || !cache_kq || !cache_ks || !cache_vq ||
      !cache_vs)
    return Q40_E_NULL;
  if (D != 128) return Q40_E_UNSUPPORTED;
  if (B < 0 || H <= 0 || Hkv <= 0 || max_t <= 0 || n_pos <= 0) return Q40_E_SHAPE;
  if (q_stride < (int64_t)H * D || k_stride < (int64_t)Hkv * D || v_stride < (int64_t)Hkv * D) return Q40_E_SHAPE;
  if (B == 0) return Q40_OK;
  if (!q40_aligned(cache_ks, 4) || !q40_aligned(cache_vs, 4)) return Q40_E_ALIGN;
  q40::AppendArgs a{};
  a.q = (__half*)q; a.k = (__half*)k; a.v = (const __half*)v;
  a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
  a.pos = pos; a.prefix_len = prefix_len;
  a.cos_tbl = (const __half*)cos_tbl; a.sin_tbl = (const __half*)sin_tbl;
  a.cache_kq = (int8_t*)cache_kq; a.cache_ks = (__half*)cache_ks;
  a.cache_vq = (int8_t*)cache_vq; a.cache_vs = (__half*)cache_vs;
  a.H = H; a.Hkv = Hkv; a.max_t = max_t; a.n_pos = n_pos;
  const cudaError_t e = q40_launch_pdl(q40::rope_kv_append_kernel, dim3(B, H + Hkv), dim3(64), 0, (cudaStream_t)stream, a);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}
