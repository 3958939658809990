// Causal attention of the prompt pass: out[i] = softmax_{j <= i}(q_i . k_j / sqrt(D)) v_j per head, for S
// positions processed at once (hf_model_q40_kv_shared.py:324-329 builds the prompt's K/V, :499-504 the
// triangular mask, :405 calls scaled_dot_product_attention with it).
//
// One CTA per (block of 128 query positions, query head): the query rows are the M dimension of
// mma.m16n8k16 (16 rows per warp, A fragments kept in registers), keys and values of the head's kv head
// (grouped-query attention reads the shared kv head directly, no repeat_interleave) stream through shared
// memory in 64-key tiles (cp.async, double buffered), S = Q K^T and O += P V on the tensor cores with an
// fp32 online softmax in the log2 domain.  Only tiles that reach the diagonal are masked; tiles beyond the
// block's last row are never loaded.  Output is normalised and written as fp16.
#include <math_constants.h>

#include "attn_common.cuh"

namespace q40 {
namespace causal {

constexpr int KT = 64;                       // keys per tile
constexpr int ROW_BYTES = ATTN_D * 2;        // 256 B per key
constexpr int TILE_BYTES = KT * ROW_BYTES;   // 16 KB
constexpr int NWARPS = 8;
constexpr int RB = NWARPS * 16;              // query rows per CTA

struct Args {
  const __half* q;    // position i, head h at q + i * ldq + h * D
  const __half* k;    // position j, kv head g at k + j * ldk + g * D
  const __half* v;
  __half* o;          // position i, head h at o + i * ldo + h * D
  int64_t ldq, ldk, ldv, ldo;
  int S, H, Hkv;
  float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;  // size 0 = write zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// byte offset of 16-byte chunk `chunk` (0..15) of row `row` in a [rows][256 B] tile, XOR-swizzled so
// that the 8 rows of an ldmatrix 8x8 block fall in different bank groups
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * ROW_BYTES + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// grid: (query blocks, H); block: 256 threads
__global__ void __launch_bounds__(NWARPS * 32)
attn_causal_kernel(const Args a) {
  constexpr int D = ATTN_D;
  constexpr int NT = NWARPS * 32;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);     // [stage][K tile | V tile]; the Q rows are staged here first
  const int rblk = blockIdx.x, h = blockIdx.y, hk = h / (a.H / a.Hkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = rblk * RB;
  const int k_end = min(a.S, row0 + RB);     // keys this block can see
  const int ntiles = (k_end + KT - 1) / KT;

  // ---- Q rows -> shared (swizzled) -> A fragments in registers ----
  for (int idx = tid; idx < RB * 16; idx += NT) {
    const int r = idx >> 4, ch = idx & 15;
    const int qi = row0 + r;
    const bool ok = qi < a.S;
    cp_async16(sbase + tile_off(r, ch), a.q + (int64_t)(ok ? qi : 0) * a.ldq + h * D + ch * 8, ok);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qa[8][4];
  {
    const int mi = lane >> 3, r8 = lane & 7;
    const int row = warp * 16 + r8 + (mi & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      ldsm_x4(sbase + tile_off(row, 2 * ks + (mi >> 1)), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
  }
  __syncthreads();  // Q staging area is free again

  auto load_tile = [&](int tile, int stage) {
    const int key0 = tile * KT;
    const uint32_t kdst = sbase + stage * 2 * TILE_BYTES;
    const uint32_t vdst = kdst + TILE_BYTES;
    for (int idx = tid; idx < KT * 16; idx += NT) {
      const int r = idx >> 4, ch = idx & 15;
      const int key = key0 + r;
      const bool ok = key < k_end;
      const int64_t kj = ok ? key : 0;
      cp_async16(kdst + tile_off(r, ch), a.k + kj * a.ldk + hk * D + ch * 8, ok);
      cp_async16(vdst + tile_off(r, ch), a.v + kj * a.ldv + hk * D + ch * 8, ok);
    }
  };

  // query positions of this lane's two rows
  const int qi0 = row0 + warp * 16 + g, qi1 = qi0 + 8;
  const int warp_last = row0 + warp * 16 + 15;          // last query position of the warp
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) oacc[i][j] = 0.f;

  if (ntiles > 0) load_tile(0, 0);
  cp_async_commit();

  for (int tile = 0; tile < ntiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < ntiles) load_tile(tile + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();   // the tile for this iteration has landed
    __syncthreads();
    const int key0 = tile * KT;
    // a warp whose rows all lie before this tile has nothing to add (the barriers are still shared)
    if (key0 <= warp_last) {
      const uint32_t kt = sbase + stage * 2 * TILE_BYTES;
      const uint32_t vt = kt + TILE_BYTES;
      // ---- S = Q K^T for 16 rows x 64 keys ----
      float sacc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sacc[i][j] = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int krow = nt * 8 + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < 8; ks += 2) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(kt + tile_off(krow, 2 * ks + (lane >> 3)), b0, b1, b2, b3);
          mma_f16(sacc[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
          mma_f16(sacc[nt], qa[ks + 1][0], qa[ks + 1][1], qa[ks + 1][2], qa[ks + 1][3], b2, b3);
        }
      }
      // ---- scale, causal mask, online softmax (rows g and g+8 of this warp) ----
      float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = key0 + nt * 8 + 2 * t + (j & 1);
          const int qi = (j >> 1) ? qi1 : qi0;
          const float v = (key <= qi && key < a.S) ? sacc[nt][j] * a.scale_log2 : -CUDART_INF_F;
          sacc[nt][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float mnew = fmaxf(m_run[r], mx[r]);
        // a row with no visible key in this tile and none before keeps everything at zero
        corr[r] = (mnew == -CUDART_INF_F) ? 1.f : exp2f(m_run[r] - mnew);
        m_run[r] = mnew;
        l_run[r] *= corr[r];
      }
      float ls[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float mref = m_run[j >> 1];
          const float p = (mref == -CUDART_INF_F) ? 0.f : exp2f(sacc[nt][j] - mref);
          sacc[nt][j] = p;
          ls[j >> 1] += p;
        }
      }
      l_run[0] += ls[0];   // per-lane partial sums; combined across the quad at the end
      l_run[1] += ls[1];
#pragma unroll
      for (int dt = 0; dt < 16; ++dt) {
        oacc[dt][0] *= corr[0]; oacc[dt][1] *= corr[0];
        oacc[dt][2] *= corr[1]; oacc[dt][3] *= corr[1];
      }
      // ---- O += P V ----
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t a0 = pack_h2(sacc[2 * kk][0], sacc[2 * kk][1]);
        const uint32_t a1 = pack_h2(sacc[2 * kk][2], sacc[2 * kk][3]);
        const uint32_t a2 = pack_h2(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
        const uint32_t a3 = pack_h2(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
        const int vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int dt = 0; dt < 16; dt += 2) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(vt + tile_off(vrow, dt + (lane >> 4)), b0, b1, b2, b3);
          mma_f16(oacc[dt], a0, a1, a2, a3, b0, b1);
          mma_f16(oacc[dt + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();  // all warps are done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // ---- normalise and write rows g and g+8 ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qi = r ? qi1 : qi0;
    if (qi >= a.S) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    __half* dst = a.o + (int64_t)qi * a.ldo + h * D;
#pragma unroll
    for (int dt = 0; dt < 16; ++dt)
      *reinterpret_cast<__half2*>(dst + dt * 8 + 2 * t) = __floats2half2_rn(oacc[dt][2 * r] * inv, oacc[dt][2 * r + 1] * inv);
  }
}

}  // namespace causal
}  // namespace q40

// o[S, H*128] = causal attention of q[S, H*128] over k, v[S, Hkv*128] (position-major rows with the given
// row strides in elements; H % Hkv == 0).  Replaces the masked scaled_dot_product_attention of the
// reference's prompt pass (hf_model_q40_kv_shared.py:375-405, mask :499-504).
extern "C" int q40_attn_causal(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                               void* o, int64_t ldo, int S, int H, int Hkv, int D, void* stream) {
  using namespace q40;
  using namespace q40::causal;
  if (!q || !k || !v || !o) return Q40_E_NULL;
  if (D != ATTN_D) return Q40_E_UNSUPPORTED;
  if (S < 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return Q40_E_SHAPE;
  if (ldq < (int64_t)H * D || ldo < (int64_t)H * D || ldk < (int64_t)Hkv * D || ldv < (int64_t)Hkv * D)
    return Q40_E_SHAPE;
  if (ldq % 8 != 0 || ldk % 8 != 0 || ldv % 8 != 0 || ldo % 2 != 0) return Q40_E_ALIGN;
  if (!q40_aligned(q, 16) || !q40_aligned(k, 16) || !q40_aligned(v, 16) || !q40_aligned(o, 4)) return Q40_E_ALIGN;
  if (S == 0) return Q40_OK;
  Args a{};
  a.q = (const __half*)q; a.k = (const __half*)k; a.v = (const __half*)v; a.o = (__half*)o;
  a.ldq = ldq; a.ldk = ldk; a.ldv = ldv; a.ldo = ldo; a.S = S; a.H = H; a.Hkv = Hkv;
  a.scale_log2 = attn_scale_log2(D);
  const size_t smem = 4 * TILE_BYTES;      // two stages of K and V (also covers the 128 staged Q rows)
  const cudaError_t e = cudaFuncSetAttribute(attn_causal_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return Q40_E_UNSUPPORTED; }
  attn_causal_kernel<<<dim3((S + RB - 1) / RB, H, 1), dim3(NWARPS * 32), smem, (cudaStream_t)stream>>>(a);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}
