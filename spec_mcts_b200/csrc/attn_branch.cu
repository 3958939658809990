// Decode attention for one query token per branch over that branch's own keys: a
// contiguous [B,Hkv,L,D] cache or a paged pool.  One CTA per (branch, query head).
//
// Eight lanes share a key: each lane owns 16 of the 128 head dims (two 16-byte loads of K,
// two of V), the partial dot products are summed with three shuffles, and every group of
// eight lanes keeps its own online-softmax state (running max, sum, 16 output dims) in
// fp32.  The 16 groups of a CTA are merged through shared memory at the end; the same
// merge can fold in partial results of a shared-prefix pass (see attn_prefix.cu), which is
// how the shared-prefix entry point finishes.
//
// Stands in for flash_attn_kernel2 / page_flash_attn_kernel2 of the reference
// (triton_kernels.py:559-647, 700-789), with fp32 softmax state and exact masking of the
// tail instead of the reference's fp16 state and multiple-of-32 length requirement.
#include <math_constants.h>

#include "attn_common.cuh"

namespace q40 {

constexpr int BR_THREADS = 128;
constexpr int BR_GROUPS = BR_THREADS / 8;   // key groups per CTA
constexpr int BR_UNROLL = 4;                // keys per group per iteration


template <int MODE>  // 0 contiguous, 1 paged with int16 ids, 2 paged with int32 ids
__device__ __forceinline__ int64_t key_slot(const BranchArgs& a, int b, int hk, int t) {
  if (MODE == 0 || MODE == 3) {
    return ((int64_t)(b * a.Hkv + hk) * a.L + t);
  } else {
    const int pg = t / a.page_size, in = t - pg * a.page_size;
    int64_t id;
    if (MODE == 1)
      id = (int64_t)(uint16_t) reinterpret_cast<const int16_t*>(a.tbl)[(int64_t)b * a.tbl_stride + pg];
    else
      id = (int64_t) reinterpret_cast<const int32_t*>(a.tbl)[(int64_t)b * a.tbl_stride + pg];
    int64_t slot = id * a.page_size + in;
    // a bad page id must not turn into a wild read: clamp into the pool
    if (slot < 0) slot = 0;
    if (slot >= a.P) slot = a.P - 1;
    return (int64_t)hk * a.P + slot;
  }
}

template <int MODE>
__global__ void __launch_bounds__(BR_THREADS)
attn_branch_kernel(const BranchArgs a) {
  constexpr int D = ATTN_D;
  asm volatile("griddepcontrol.launch_dependents;");   // a dependent may start prefetching its weights
  asm volatile("griddepcontrol.wait;" ::: "memory");               // ... but nothing of the previous launch is read before it is done
  const int bh = blockIdx.x;
  const int b = bh / a.H, h = bh % a.H;
  const int hk = h / (a.H / a.Hkv);
  const int tid = threadIdx.x, lane = tid & 31;
  const int grp = tid >> 3, sub = tid & 7;
  // the 8 lanes that share a key; groups of one warp may run different numbers of iterations,
  // so every shuffle names only its own group
  const unsigned gmask = 0xffu << (lane & 24);
  int len;
  if (MODE == 3) len = min(max(a.pos[b] - a.prefix_len[0], 0), a.max_t);
  else len = a.seq_lens ? min(max(a.seq_lens[b], 0), a.L) : a.L;

  __shared__ float sm_m[BR_GROUPS], sm_l[BR_GROUPS];
  __shared__ __align__(16) float sm_o[BR_GROUPS][D];

  // this lane's 16 query dims, pre-multiplied by scale*log2(e)
  float qf[16];
  {
    const __half* qp = a.q + (int64_t)b * a.q_stride + h * D + sub * 16;
    const uint4 q0 = *reinterpret_cast<const uint4*>(qp);
    const uint4 q1 = *reinterpret_cast<const uint4*>(qp + 8);
    const __half2* h0 = reinterpret_cast<const __half2*>(&q0);
    const __half2* h1 = reinterpret_cast<const __half2*>(&q1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f0 = __half22float2(h0[i]), f1 = __half22float2(h1[i]);
      qf[2 * i] = f0.x * a.scale_log2;
      qf[2 * i + 1] = f0.y * a.scale_log2;
      qf[8 + 2 * i] = f1.x * a.scale_log2;
      qf[8 + 2 * i + 1] = f1.y * a.scale_log2;
    }
  }
  float m = -CUDART_INF_F, l = 0.f, o[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i] = 0.f;

  if (MODE != 3)
  for (int t0 = grp; t0 < len; t0 += BR_GROUPS * BR_UNROLL) {
    uint4 kv[BR_UNROLL][4];
    float s[BR_UNROLL];
#pragma unroll
    for (int u = 0; u < BR_UNROLL; ++u) {
      const int t = t0 + u * BR_GROUPS;
      if (t < len) {
        const int64_t off = key_slot<MODE>(a, b, hk, t) * D + sub * 16;
        kv[u][0] = __ldg(reinterpret_cast<const uint4*>(a.k + off));
        kv[u][1] = __ldg(reinterpret_cast<const uint4*>(a.k + off + 8));
        kv[u][2] = __ldg(reinterpret_cast<const uint4*>(a.v + off));
        kv[u][3] = __ldg(reinterpret_cast<const uint4*>(a.v + off + 8));
      } else {
        kv[u][0] = kv[u][1] = kv[u][2] = kv[u][3] = make_uint4(0, 0, 0, 0);
      }
    }
    float mnew = m;
#pragma unroll
    for (int u = 0; u < BR_UNROLL; ++u) {
      const __half2* kh = reinterpret_cast<const __half2*>(&kv[u][0]);  // 8 half2 = 16 dims
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = __half22float2(kh[i]);
        acc = fmaf(qf[2 * i], f.x, acc);
        acc = fmaf(qf[2 * i + 1], f.y, acc);
      }
      acc += __shfl_xor_sync(gmask, acc, 1);
      acc += __shfl_xor_sync(gmask, acc, 2);
      acc += __shfl_xor_sync(gmask, acc, 4);
      s[u] = (t0 + u * BR_GROUPS < len) ? acc : -CUDART_INF_F;
      mnew = fmaxf(mnew, s[u]);
    }
    // t0 < len, so mnew is finite here
    const float corr = exp2f(m - mnew);
    l *= corr;
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] *= corr;
#pragma unroll
    for (int u = 0; u < BR_UNROLL; ++u) {
      const float p = exp2f(s[u] - mnew);
      l += p;
      const __half2* vh = reinterpret_cast<const __half2*>(&kv[u][2]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = __half22float2(vh[i]);
        o[2 * i] = fmaf(p, f.x, o[2 * i]);
        o[2 * i + 1] = fmaf(p, f.y, o[2 * i + 1]);
      }
    }
    m = mnew;
  }

  if (MODE == 3) {
    // Q4_0 cache: lane `sub` owns dims 16*sub..16*sub+15 = nibble half (sub>>2) of bytes 16*(sub&3)..+15
    const int nib_lo = sub >> 2;                 // 0: high nibbles (dims 0..63), 1: low nibbles
    const int boff = 16 * (sub & 3);
    for (int t0 = grp; t0 < len; t0 += BR_GROUPS * BR_UNROLL) {
      uint4 kb[BR_UNROLL], vb[BR_UNROLL];
      __half ksv[BR_UNROLL], vsv[BR_UNROLL];
      float s[BR_UNROLL];
#pragma unroll
      for (int u = 0; u < BR_UNROLL; ++u) {
        const int t = t0 + u * BR_GROUPS;
        if (t < len) {
          const int64_t row = ((int64_t)b * a.max_t + t) * a.Hkv + hk;
          kb[u] = __ldg(reinterpret_cast<const uint4*>(a.kq + row * 64 + boff));
          vb[u] = __ldg(reinterpret_cast<const uint4*>(a.vq + row * 64 + boff));
          ksv[u] = a.ksc[row * 2 + nib_lo];
          vsv[u] = a.vsc[row * 2 + nib_lo];
        } else {
          kb[u] = vb[u] = make_uint4(0, 0, 0, 0);
          ksv[u] = vsv[u] = __float2half(0.f);
        }
      }
      float mnew = m;
#pragma unroll
      for (int u = 0; u < BR_UNROLL; ++u) {
        const uint32_t* wd = reinterpret_cast<const uint32_t*>(&kb[u]);
        const __half2 sc = __half2half2(ksv[u]);
        float acc = 0.f;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint32_t w = nib_lo ? wd[wi] : (wd[wi] >> 4);
          const float2 f02 = __half22float2(__hmul2(codes_lo_to_h2(w), sc));        // bytes 0, 2
          const float2 f13 = __half22float2(__hmul2(codes_lo_to_h2(w >> 8), sc));   // bytes 1, 3
          acc = fmaf(qf[4 * wi + 0], f02.x, acc);
          acc = fmaf(qf[4 * wi + 2], f02.y, acc);
          acc = fmaf(qf[4 * wi + 1], f13.x, acc);
          acc = fmaf(qf[4 * wi + 3], f13.y, acc);
        }
        acc += __shfl_xor_sync(gmask, acc, 1);
        acc += __shfl_xor_sync(gmask, acc, 2);
        acc += __shfl_xor_sync(gmask, acc, 4);
        s[u] = (t0 + u * BR_GROUPS < len) ? acc : -CUDART_INF_F;
        mnew = fmaxf(mnew, s[u]);
      }
      const float corr = exp2f(m - mnew);
      l *= corr;
#pragma unroll
      for (int i = 0; i < 16; ++i) o[i] *= corr;
#pragma unroll
      for (int u = 0; u < BR_UNROLL; ++u) {
        const float p = exp2f(s[u] - mnew);
        l += p;
        const uint32_t* wd = reinterpret_cast<const uint32_t*>(&vb[u]);
        const __half2 sc = __half2half2(vsv[u]);
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint32_t w = nib_lo ? wd[wi] : (wd[wi] >> 4);
          const float2 f02 = __half22float2(__hmul2(codes_lo_to_h2(w), sc));
          const float2 f13 = __half22float2(__hmul2(codes_lo_to_h2(w >> 8), sc));
          o[4 * wi + 0] = fmaf(p, f02.x, o[4 * wi + 0]);
          o[4 * wi + 2] = fmaf(p, f02.y, o[4 * wi + 2]);
          o[4 * wi + 1] = fmaf(p, f13.x, o[4 * wi + 1]);
          o[4 * wi + 3] = fmaf(p, f13.y, o[4 * wi + 3]);
        }
      }
      m = mnew;
    }
  }
  // the token being decoded attends to its own, un-quantised K/V: one extra key for group 0
  if (a.cur_k != nullptr && grp == 0) {
    const __half* kp = a.cur_k + (int64_t)b * a.cur_stride + hk * D + sub * 16;
    const __half* vp = a.cur_v + (int64_t)b * a.cur_stride + hk * D + sub * 16;
    const uint4 k0 = *reinterpret_cast<const uint4*>(kp), k1 = *reinterpret_cast<const uint4*>(kp + 8);
    const uint4 v0 = *reinterpret_cast<const uint4*>(vp), v1 = *reinterpret_cast<const uint4*>(vp + 8);
    const __half2* kh0 = reinterpret_cast<const __half2*>(&k0);
    const __half2* kh1 = reinterpret_cast<const __half2*>(&k1);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f0 = __half22float2(kh0[i]), f1 = __half22float2(kh1[i]);
      acc = fmaf(qf[2 * i], f0.x, acc);
      acc = fmaf(qf[2 * i + 1], f0.y, acc);
      acc = fmaf(qf[8 + 2 * i], f1.x, acc);
      acc = fmaf(qf[8 + 2 * i + 1], f1.y, acc);
    }
    acc += __shfl_xor_sync(0x000000ffu, acc, 1);
    acc += __shfl_xor_sync(0x000000ffu, acc, 2);
    acc += __shfl_xor_sync(0x000000ffu, acc, 4);
    const float mnew = fmaxf(m, acc);
    const float corr = exp2f(m - mnew), p = exp2f(acc - mnew);
    l = l * corr + p;
    const __half2* vh0 = reinterpret_cast<const __half2*>(&v0);
    const __half2* vh1 = reinterpret_cast<const __half2*>(&v1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f0 = __half22float2(vh0[i]), f1 = __half22float2(vh1[i]);
      o[2 * i] = fmaf(p, f0.x, o[2 * i] * corr);
      o[2 * i + 1] = fmaf(p, f0.y, o[2 * i + 1] * corr);
      o[8 + 2 * i] = fmaf(p, f1.x, o[8 + 2 * i] * corr);
      o[8 + 2 * i + 1] = fmaf(p, f1.y, o[8 + 2 * i + 1] * corr);
    }
    m = mnew;
  }

  if (sub == 0) { sm_m[grp] = m; sm_l[grp] = l; }
#pragma unroll
  for (int i = 0; i < 16; i += 4)
    *reinterpret_cast<float4*>(&sm_o[grp][sub * 16 + i]) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
  __syncthreads();

  // merge: thread d owns output dim d
  const int d = tid;
  float M = -CUDART_INF_F;
#pragma unroll
  for (int gI = 0; gI < BR_GROUPS; ++gI) M = fmaxf(M, sm_m[gI]);
  const int64_t rows = (int64_t)gridDim.x;
  for (int sp = 0; sp < a.nsp; ++sp) M = fmaxf(M, a.pm[(int64_t)sp * rows + bh]);
  float Lsum = 0.f, acc = 0.f;
  if (M > -CUDART_INF_F) {
#pragma unroll
    for (int gI = 0; gI < BR_GROUPS; ++gI) {
      const float w = exp2f(sm_m[gI] - M);   // exp2(-inf) = 0 for empty groups
      Lsum = fmaf(sm_l[gI], w, Lsum);
      acc = fmaf(sm_o[gI][d], w, acc);
    }
    for (int sp = 0; sp < a.nsp; ++sp) {
      const int64_t r = (int64_t)sp * rows + bh;
      const float w = exp2f(a.pm[r] - M);
      Lsum = fmaf(a.pl[r], w, Lsum);
      acc = fmaf(a.po[r * D + d], w, acc);
    }
  }
  const float outv = (Lsum > 0.f) ? acc / Lsum : 0.f;
  a.o[((int64_t)b * a.H + h) * D + d] = __float2half_rn(outv);
}

int launch_branch(const BranchArgs& a, int mode, int B, cudaStream_t st) {
  const unsigned grid = (unsigned)(B * a.H);
  cudaError_t e;
  if (mode == 0) e = q40_launch_pdl(attn_branch_kernel<0>, dim3(grid), dim3(BR_THREADS), 0, st, a);
  else if (mode == 1) e = q40_launch_pdl(attn_branch_kernel<1>, dim3(grid), dim3(BR_THREADS), 0, st, a);
  else if (mode == 2) e = q40_launch_pdl(attn_branch_kernel<2>, dim3(grid), dim3(BR_THREADS), 0, st, a);
  else e = q40_launch_pdl(attn_branch_kernel<3>, dim3(grid), dim3(BR_THREADS), 0, st, a);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}

}  // namespace q40

static int check_common(int B, int H, int Hkv, int D) {
  if (D != q40::ATTN_D) return Q40_E_UNSUPPORTED;
  if (B < 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return Q40_E_SHAPE;
  if ((int64_t)B * H > 0x7fffffffLL) return Q40_E_SHAPE;
  return Q40_OK;
}

extern "C" int q40_attn_decode(const void* q, const void* k, const void* v, void* o, int B, int L, int H,
                               int Hkv, int D, void* stream) {
  if (!q || !o) return Q40_E_NULL;
  int rc = check_common(B, H, Hkv, D);
  if (rc) return rc;
  if (L < 0) return Q40_E_SHAPE;
  if (L > 0 && (!k || !v)) return Q40_E_NULL;
  if (B == 0) return Q40_OK;
  if (!q40_aligned(q, 16) || !q40_aligned(k, 16) || !q40_aligned(v, 16) || !q40_aligned(o, 2))
    return Q40_E_ALIGN;
  q40::BranchArgs a{};
  a.q = (const __half*)q; a.q_stride = (int64_t)H * D; a.k = (const __half*)k; a.v = (const __half*)v; a.o = (__half*)o;
  a.L = L; a.H = H; a.Hkv = Hkv; a.P = 0; a.page_size = 1;
  a.scale_log2 = q40::attn_scale_log2(D);
  return q40::launch_branch(a, 0, B, (cudaStream_t)stream);
}

extern "C" int q40_attn_paged(const void* page_tbl, int idx_bytes, int64_t tbl_stride,
                              const int32_t* seq_lens, const void* q, const void* kpool, const void* vpool,
                              void* o, int P, int B, int Lmax, int H, int Hkv, int D, int page_size,
                              void* stream) {
  if (!q || !o) return Q40_E_NULL;
  int rc = check_common(B, H, Hkv, D);
  if (rc) return rc;
  if (Lmax < 0 || P < 0 || page_size <= 0) return Q40_E_SHAPE;
  if (idx_bytes != 2 && idx_bytes != 4) return Q40_E_UNSUPPORTED;
  if (Lmax > 0 && (!page_tbl || !kpool || !vpool || P == 0)) return Q40_E_NULL;
  if (tbl_stride < (Lmax + page_size - 1) / page_size) return Q40_E_SHAPE;
  if (B == 0) return Q40_OK;
  if (!q40_aligned(q, 16) || !q40_aligned(kpool, 16) || !q40_aligned(vpool, 16)) return Q40_E_ALIGN;
  q40::BranchArgs a{};
  a.q = (const __half*)q; a.q_stride = (int64_t)H * D; a.k = (const __half*)kpool; a.v = (const __half*)vpool; a.o = (__half*)o;
  a.tbl = page_tbl; a.tbl_stride = tbl_stride; a.seq_lens = seq_lens;
  a.L = Lmax; a.H = H; a.Hkv = Hkv; a.P = P; a.page_size = page_size;
  a.scale_log2 = q40::attn_scale_log2(D);
  return q40::launch_branch(a, idx_bytes == 2 ? 1 : 2, B, (cudaStream_t)stream);
}
