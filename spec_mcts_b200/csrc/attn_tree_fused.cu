// Decode attention of the KV-shared model as ONE launch: rotary embedding of q and of the new key,
// Q4_0 append of the new key/value, and attention over [shared fp16 prompt | packed Q4_0 suffix |
// the un-quantised new token].  A thread-block cluster of 8 CTAs serves one (branch, head): its
// 128 groups of 8 lanes take the keys round-robin (each lane owns 16 of the 128 head dims), every
// group keeps an fp32 online-softmax state, groups are merged through shared memory inside a
// CTA and the CTAs through distributed shared memory, each rank finishing 16 output dims.
// Meant for small widths (up to about 16 branches), where three separate launches (rotary+append,
// shared-prefix MMA pass, per-branch pass) cost more than the attention itself; larger widths
// use q40_attn_tree_decode, which reads the prompt once for all branches.
//
// Reference: Attention.forward decode branch (hf_model_q40_kv_shared.py:313-317, 330-405).
#include <cooperative_groups.h>
#include <math_constants.h>

#include "q40_common.cuh"

namespace cg = cooperative_groups;

namespace q40 {

constexpr int TF_THREADS = 128;
constexpr int TF_WARPS = TF_THREADS / 32;
constexpr int TF_CLUSTER = 8;
constexpr int TF_KPG = 5;          // keys a group of 8 lanes holds in registers per batch (640 per cluster)

struct TreeFusedArgs {
  __half* qkv;             // [B, W]: q heads, then k heads, then v heads of the new token (un-rotated)
  int64_t W;
  const __half* pk;        // prompt cache [max_p, Hkv, 128]
  const __half* pv;
  int8_t* kq;              // suffix cache [maxB, max_t, Hkv, 64]
  __half* ks;
  int8_t* vq;
  __half* vs;
  const int32_t* pos;
  const int32_t* prefix_len;
  const __half* cos_tbl;   // [n_pos, 64]
  const __half* sin_tbl;
  __half* ao;              // [B, H*128]
  int H, Hkv, max_t, max_p, n_pos;
  void* trace;             // stage timestamps (trace builds only)
};

// One cached key/value row as a lane fetched it: prompt rows are 2 x 16 B of K and of V (this lane's
// 16 dims in fp16); suffix rows are 16 B of K codes, 16 B of V codes and the two scales.
struct TfRaw { uint4 r[4]; };

__device__ __forceinline__ void tf_load(const TreeFusedArgs& a, int key, int plen, int b, int hk, int sub, TfRaw& w) {
  if (key < plen) {
    const int64_t off = ((int64_t)key * a.Hkv + hk) * 128 + sub * 16;
    w.r[0] = __ldg(reinterpret_cast<const uint4*>(a.pk + off));
    w.r[1] = __ldg(reinterpret_cast<const uint4*>(a.pk + off + 8));
    w.r[2] = __ldg(reinterpret_cast<const uint4*>(a.pv + off));
    w.r[3] = __ldg(reinterpret_cast<const uint4*>(a.pv + off + 8));
  } else {
    const int64_t row = ((int64_t)b * a.max_t + (key - plen)) * a.Hkv + hk;
    const int nib_lo = sub >> 2, boff = 16 * (sub & 3);
    w.r[0] = __ldg(reinterpret_cast<const uint4*>(a.kq + row * 64 + boff));
    w.r[1] = __ldg(reinterpret_cast<const uint4*>(a.vq + row * 64 + boff));
    const uint32_t ksb = __half_as_ushort(__ldg(a.ks + row * 2 + nib_lo));
    const uint32_t vsb = __half_as_ushort(__ldg(a.vs + row * 2 + nib_lo));
    w.r[2].x = ksb | (vsb << 16);
  }
}
__device__ __forceinline__ void tf_dec_half(const uint4& lo, const uint4& hi, float (&out)[16]) {
  const __half2* a0 = reinterpret_cast<const __half2*>(&lo);
  const __half2* a1 = reinterpret_cast<const __half2*>(&hi);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(a0[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y;
    f = __half22float2(a1[i]); out[8 + 2 * i] = f.x; out[8 + 2 * i + 1] = f.y;
  }
}
// the lane's 16 codes of a packed row (high nibbles for head dims 0..63, low for 64..127) times the scale
__device__ __forceinline__ void tf_dec_q4(const uint4& bytes, uint32_t scale_bits, int nib_lo, float (&out)[16]) {
  const __half2 sc = __half2half2(__ushort_as_half((unsigned short)scale_bits));
  const uint32_t* wv = reinterpret_cast<const uint32_t*>(&bytes);
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    const uint32_t c = nib_lo ? wv[wi] : (wv[wi] >> 4);
    float2 f = __half22float2(__hmul2(codes_lo_to_h2(c), sc));
    out[4 * wi] = f.x; out[4 * wi + 2] = f.y;
    f = __half22float2(__hmul2(codes_lo_to_h2(c >> 8), sc));
    out[4 * wi + 1] = f.x; out[4 * wi + 3] = f.y;
  }
}
// merge the online-softmax states of lanes `delta` apart (both end up with the merged state)
__device__ __forceinline__ void tf_merge_xor(float& m, float& l, float (&o)[16], int delta) {
  const float m2 = __shfl_xor_sync(0xffffffffu, m, delta), l2 = __shfl_xor_sync(0xffffffffu, l, delta);
  const float M = fmaxf(m, m2);
  const float w1 = (m > -CUDART_INF_F) ? exp2f(m - M) : 0.f, w2 = (m2 > -CUDART_INF_F) ? exp2f(m2 - M) : 0.f;
  l = l * w1 + l2 * w2;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float o2 = __shfl_xor_sync(0xffffffffu, o[i], delta);
    o[i] = o[i] * w1 + o2 * w2;
  }
  m = M;
}

__global__ void __cluster_dims__(TF_CLUSTER, 1, 1) __launch_bounds__(TF_THREADS, 2)
attn_tree_fused_kernel(const TreeFusedArgs a) {
  cg::cluster_group cluster = cg::this_cluster();
  Q40_TRACE_DECL
  Q40_STAMP(0);
  // phase 1 of the cluster barrier only says "this CTA is running" (waited for before the first
  // store into a neighbour's shared memory); phase 2 publishes those stores
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  __shared__ float cta_m[TF_WARPS], cta_l[TF_WARPS];
  __shared__ __align__(16) float cta_o[TF_WARPS * 128];
  __shared__ __align__(16) float recv[TF_CLUSTER][128 / TF_CLUSTER + 4];   // per source rank: this rank's dims, max, sum
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int cs = TF_CLUSTER;
  const int rank = (int)cluster.block_rank();
  const int it = blockIdx.x / TF_CLUSTER;
  const int b = it / a.H, hq = it % a.H;
  const int rep = a.H / a.Hkv, hk = hq / rep;
  const int grp = tid >> 3, sub = tid & 7;
  const unsigned gmask = 0xffu << (lane & 24);
  constexpr int ngroups = (TF_THREADS / 8) * cs;
  const int gidx = rank * (TF_THREADS / 8) + grp;
  const float scale_log2 = (1.0f / sqrtf(128.0f)) * 1.4426950408889634f;
  // positions and the prefix length were written before the previous launch started, and cache
  // rows below `pos` by earlier decode steps: none of this waits for the previous launch
  const int plen = min(max(a.prefix_len[0], 0), a.max_p);
  int pos = a.pos[b];
  pos = min(max(pos, 0), a.n_pos - 1);
  const int slen = min(max(pos - plen, 0), a.max_t);
  // keys: [0, plen) prompt (fp16), [plen, plen + slen) suffix (Q4_0), then the new token
  const int total_keys = plen + slen + 1;
  TfRaw raw[TF_KPG];
#pragma unroll
  for (int i = 0; i < TF_KPG; ++i) {
    const int key = gidx + i * ngroups;
    if (key < total_keys - 1) tf_load(a, key, plen, b, hk, sub, raw[i]);
  }
  Q40_STAMP(1);
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  Q40_STAMP(2);

  // this lane's 16 dims of the rotated, pre-scaled query and of the rotated new key; its 16 dims of v
  float qf[16];
  __align__(16) __half kc[16], vc[16];
  {
    const __half* qp = a.qkv + (int64_t)b * a.W + hq * 128;
    const __half* kp = a.qkv + (int64_t)b * a.W + (a.H + hk) * 128;
    const __half* vp = a.qkv + (int64_t)b * a.W + (a.H + a.Hkv + hk) * 128;
    const int d0 = sub * 16, dp = (d0 + 64) & 127;
    const bool lo_half = d0 < 64;
    __align__(16) __half q1[16], q2[16], k1[16], k2[16], cs_[16], sn_[16];
    *reinterpret_cast<uint4*>(q1) = *reinterpret_cast<const uint4*>(qp + d0);
    *reinterpret_cast<uint4*>(q1 + 8) = *reinterpret_cast<const uint4*>(qp + d0 + 8);
    *reinterpret_cast<uint4*>(q2) = *reinterpret_cast<const uint4*>(qp + dp);
    *reinterpret_cast<uint4*>(q2 + 8) = *reinterpret_cast<const uint4*>(qp + dp + 8);
    *reinterpret_cast<uint4*>(k1) = *reinterpret_cast<const uint4*>(kp + d0);
    *reinterpret_cast<uint4*>(k1 + 8) = *reinterpret_cast<const uint4*>(kp + d0 + 8);
    *reinterpret_cast<uint4*>(k2) = *reinterpret_cast<const uint4*>(kp + dp);
    *reinterpret_cast<uint4*>(k2 + 8) = *reinterpret_cast<const uint4*>(kp + dp + 8);
    *reinterpret_cast<uint4*>(vc) = *reinterpret_cast<const uint4*>(vp + d0);
    *reinterpret_cast<uint4*>(vc + 8) = *reinterpret_cast<const uint4*>(vp + d0 + 8);
    const __half* ct = a.cos_tbl + (int64_t)pos * 64 + (d0 & 63);
    const __half* st = a.sin_tbl + (int64_t)pos * 64 + (d0 & 63);
    *reinterpret_cast<uint4*>(cs_) = *reinterpret_cast<const uint4*>(ct);
    *reinterpret_cast<uint4*>(cs_ + 8) = *reinterpret_cast<const uint4*>(ct + 8);
    *reinterpret_cast<uint4*>(sn_) = *reinterpret_cast<const uint4*>(st);
    *reinterpret_cast<uint4*>(sn_ + 8) = *reinterpret_cast<const uint4*>(st + 8);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      // out = x*cos + rot(x)*sin, rot(x) = -partner for the low half of the head, +partner for the high half
      const __half qr = __hadd_rn(__hmul_rn(q1[i], cs_[i]), __hmul_rn(lo_half ? __hneg(q2[i]) : q2[i], sn_[i]));
      kc[i] = __hadd_rn(__hmul_rn(k1[i], cs_[i]), __hmul_rn(lo_half ? __hneg(k2[i]) : k2[i], sn_[i]));
      qf[i] = __half2float(qr) * scale_log2;
    }
  }
  float mx = -CUDART_INF_F, l = 0.f, o[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i] = 0.f;
  const int nib_lo = sub >> 2;
  Q40_STAMP_DEP(3, __half2float(kc[0]));
  for (int base = 0; base < total_keys; base += TF_KPG * ngroups) {
    if (base > 0) {
#pragma unroll
      for (int i = 0; i < TF_KPG; ++i) {
        const int key = base + gidx + i * ngroups;
        if (key < total_keys - 1) tf_load(a, key, plen, b, hk, sub, raw[i]);
      }
    }
    // the scores of the batch first (independent of one another), then one rescale of the state
    float sd[TF_KPG];
    float bm = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < TF_KPG; ++i) {
      const int key = base + gidx + i * ngroups;
      sd[i] = -CUDART_INF_F;
      if (key < total_keys) {
        float kk[16];
        if (key < plen) {
          tf_dec_half(raw[i].r[0], raw[i].r[1], kk);
        } else if (key < total_keys - 1) {
          tf_dec_q4(raw[i].r[0], raw[i].r[2].x & 0xFFFFu, nib_lo, kk);
        } else {
#pragma unroll
          for (int d = 0; d < 16; ++d) kk[d] = __half2float(kc[d]);
        }
        float sdot = 0.f;
#pragma unroll
        for (int d = 0; d < 16; ++d) sdot = fmaf(qf[d], kk[d], sdot);
        sdot += __shfl_xor_sync(gmask, sdot, 1);
        sdot += __shfl_xor_sync(gmask, sdot, 2);
        sdot += __shfl_xor_sync(gmask, sdot, 4);
        sd[i] = sdot;
        bm = fmaxf(bm, sdot);
      }
    }
    if (base + gidx < total_keys) {          // the group has at least one key in this batch
      const float mnew = fmaxf(mx, bm);
      const float corr = (mx > -CUDART_INF_F) ? exp2f(mx - mnew) : 0.f;
      l *= corr;
#pragma unroll
      for (int d = 0; d < 16; ++d) o[d] *= corr;
#pragma unroll
      for (int i = 0; i < TF_KPG; ++i) {
        const int key = base + gidx + i * ngroups;
        if (key < total_keys) {
          float vv[16];
          if (key < plen) {
            tf_dec_half(raw[i].r[2], raw[i].r[3], vv);
          } else if (key < total_keys - 1) {
            tf_dec_q4(raw[i].r[1], raw[i].r[2].x >> 16, nib_lo, vv);
          } else {
#pragma unroll
            for (int d = 0; d < 16; ++d) vv[d] = __half2float(vc[d]);
          }
          const float pw = exp2f(sd[i] - mnew);
          l += pw;
#pragma unroll
          for (int d = 0; d < 16; ++d) o[d] = fmaf(pw, vv[d], o[d]);
        }
      }
      mx = mnew;
    }
  }
  // Q4_0 append of the new token's rotated key and its value: the first query head of a kv
  // group, rank 0, key group 0 (the 8 lanes hold the whole 128-dim row)
  if (rank == 0 && grp == 0 && (hq % rep) == 0 && (pos - plen) >= 0 && (pos - plen) < a.max_t) {
    float ak = 0.f, av = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      ak = fmaxf(ak, fabsf(__half2float(kc[i])));
      av = fmaxf(av, fabsf(__half2float(vc[i])));
    }
    // a 64-dim group is lanes sub 0..3 (dims 0..63) or 4..7 (dims 64..127)
    ak = fmaxf(ak, __shfl_xor_sync(0xffu, ak, 1)); ak = fmaxf(ak, __shfl_xor_sync(0xffu, ak, 2));
    av = fmaxf(av, __shfl_xor_sync(0xffu, av, 1)); av = fmaxf(av, __shfl_xor_sync(0xffu, av, 2));
    const __half sk = __float2half_rn(__fdiv_rn(ak, 7.0f)), sv = __float2half_rn(__fdiv_rn(av, 7.0f));
    const float fk = __half2float(sk), fv = __half2float(sv);
    uint32_t ck[4] = {0, 0, 0, 0}, cv[4] = {0, 0, 0, 0};     // this lane's 16 codes, one nibble each
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float a = rintf(__half2float(__float2half_rn(__fdiv_rn(__half2float(kc[i]), fk))));
      float c = rintf(__half2float(__float2half_rn(__fdiv_rn(__half2float(vc[i]), fv))));
      const int ia = (fabsf(a) <= 65504.0f) ? (int)a : 0, ic = (fabsf(c) <= 65504.0f) ? (int)c : 0;
      ck[i >> 2] |= (uint32_t)(ia & 0xF) << (8 * (i & 3));
      cv[i >> 2] |= (uint32_t)(ic & 0xF) << (8 * (i & 3));
    }
    // byte d = code(dim d) << 4 | code(dim d + 64): lanes sub and sub + 4 combine
    const int64_t row = ((int64_t)b * a.max_t + (pos - plen)) * a.Hkv + hk;
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      const uint32_t ok_ = __shfl_xor_sync(0xffu, ck[wi], 4), ov_ = __shfl_xor_sync(0xffu, cv[wi], 4);
      if (sub < 4) {
        reinterpret_cast<uint32_t*>(a.kq + row * 64 + 16 * sub)[wi] = (ck[wi] << 4) | ok_;
        reinterpret_cast<uint32_t*>(a.vq + row * 64 + 16 * sub)[wi] = (cv[wi] << 4) | ov_;
      }
    }
    if (sub == 0) { a.ks[row * 2] = sk; a.vs[row * 2] = sv; }
    if (sub == 4) { a.ks[row * 2 + 1] = sk; a.vs[row * 2 + 1] = sv; }
  }

  Q40_STAMP_DEP(4, mx);
  // ---- the four key groups of a warp through shuffles, the eight warps through shared memory ----
  tf_merge_xor(mx, l, o, 8);
  tf_merge_xor(mx, l, o, 16);
  if (lane < 8) {
    if (lane == 0) { cta_m[warp] = mx; cta_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < 16; i += 4)
      *reinterpret_cast<float4*>(&cta_o[warp * 128 + lane * 16 + i]) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
  }
  __syncthreads();
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");     // every CTA of the cluster is running
  constexpr int per = 128 / cs;          // output dims finished by one rank
  if (tid < 128) {
    float Mx = -CUDART_INF_F;
#pragma unroll
    for (int q = 0; q < TF_WARPS; ++q) Mx = fmaxf(Mx, cta_m[q]);
    float Ls = 0.f, acc = 0.f;
    if (Mx > -CUDART_INF_F) {
#pragma unroll
      for (int q = 0; q < TF_WARPS; ++q) {
        const float w = exp2f(cta_m[q] - Mx);
        Ls = fmaf(cta_l[q], w, Ls);
        acc = fmaf(cta_o[q * 128 + tid], w, acc);
      }
    }
    // hand the CTA's partial to the rank that finishes this dim
    float* dst = cluster.map_shared_rank(&recv[rank][0], tid / per);
    dst[tid % per] = acc;
    if (tid % per == 0) { dst[per] = Mx; dst[per + 1] = Ls; }
  }
  Q40_STAMP(5);
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  Q40_STAMP(6);
  if (tid < per) {
    float Mx = -CUDART_INF_F;
#pragma unroll
    for (int r = 0; r < cs; ++r) Mx = fmaxf(Mx, recv[r][per]);
    float Ls = 0.f, acc = 0.f;
#pragma unroll
    for (int r = 0; r < cs; ++r) {
      const float pm = recv[r][per];
      const float w = (pm > -CUDART_INF_F) ? exp2f(pm - Mx) : 0.f;
      Ls = fmaf(recv[r][per + 1], w, Ls);
      acc = fmaf(recv[r][tid], w, acc);
    }
    a.ao[(int64_t)b * (a.H * 128) + hq * 128 + rank * per + tid] = __float2half_rn(Ls > 0.f ? acc / Ls : 0.f);
  }
  Q40_STAMP(7);
  Q40_TRACE_FLUSH(a.trace, 200);
}

}  // namespace q40

extern "C" int q40_attn_tree_fused(void* qkv, int64_t W, const void* pk, const void* pv, void* kq, void* ks,
                                   void* vq, void* vs, const int32_t* pos, const int32_t* prefix_len,
                                   const void* cos_tbl, const void* sin_tbl, int n_pos, void* ao, int B, int H,
                                   int Hkv, int D, int max_t, int max_p, int use_pdl, void* stream) {
  using namespace q40;
  if (!qkv || !pk || !pv || !kq || !ks || !vq || !vs || !pos || !prefix_len || !cos_tbl || !sin_tbl || !ao)
    return Q40_E_NULL;
  if (D != 128) return Q40_E_UNSUPPORTED;
  if (B < 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || max_t <= 0 || max_p <= 0 || n_pos <= 0) return Q40_E_SHAPE;
  if (W < (int64_t)(H + 2 * Hkv) * 128 || W % 8 != 0) return Q40_E_SHAPE;
  if (B == 0) return Q40_OK;
  if (!q40_aligned(qkv, 16) || !q40_aligned(pk, 16) || !q40_aligned(pv, 16) || !q40_aligned(kq, 16) ||
      !q40_aligned(vq, 16) || !q40_aligned(cos_tbl, 16) || !q40_aligned(sin_tbl, 16))
    return Q40_E_ALIGN;
  if ((int64_t)B * H * TF_CLUSTER > 0x7fffffffLL) return Q40_E_SHAPE;
  TreeFusedArgs a{};
  a.qkv = (__half*)qkv; a.W = W; a.pk = (const __half*)pk; a.pv = (const __half*)pv;
  a.kq = (int8_t*)kq; a.ks = (__half*)ks; a.vq = (int8_t*)vq; a.vs = (__half*)vs;
  a.pos = pos; a.prefix_len = prefix_len; a.cos_tbl = (const __half*)cos_tbl; a.sin_tbl = (const __half*)sin_tbl;
#ifdef Q40_TRACE
  a.trace = q40_trace_ptr;
#endif
  a.ao = (__half*)ao; a.H = H; a.Hkv = Hkv; a.max_t = max_t; a.max_p = max_p; a.n_pos = n_pos;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(B * H * TF_CLUSTER), 1, 1);
  cfg.blockDim = dim3(TF_THREADS, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
  cudaError_t e = cudaFuncSetAttribute(attn_tree_fused_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) return (int)e;
  e = cudaLaunchKernelEx(&cfg, attn_tree_fused_kernel, a);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}
