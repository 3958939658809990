// Shared-prefix stage of tree/speculative decode attention.
//
// All B branches attend to the same prompt K/V.  Instead of letting every (branch, head)
// CTA re-read the prefix, the queries of all branches (times the GQA group) of one kv head
// are stacked as the M dimension of a tensor-core product: a CTA loads a 64-key tile of the
// prefix once (cp.async, double buffered, 16 KB of K + 16 KB of V) and applies it to up to
// 128 query rows with mma.m16n8k16 (S = Q K^T, online softmax in fp32 in the log2 domain,
// O += P V).  The prefix is split across CTAs flash-decoding style; each CTA writes its
// un-normalised partial (m, l, O) per row to a scratch buffer, and the per-branch kernel
// (attn_branch.cu) folds those partials into the result after walking the branch's private
// suffix pages.  This is the computation the reference's chunk_attn was aiming for
// (triton_kernels.py:1150-1231) and what its model does by materialising
// cat(prompt.expand(B), suffix) for SDPA (hf_model_q40_kv_shared.py:375-376, 405).
//
// Algorithmic traffic: prefix K/V once per (kv head, row block); Q and the partials are
// small next to it.
#include <math_constants.h>

#include "attn_common.cuh"

namespace q40 {

constexpr int PF_KT = 64;                      // keys per tile
constexpr int PF_ROW_BYTES = ATTN_D * 2;       // 256 B per key
constexpr int PF_TILE_BYTES = PF_KT * PF_ROW_BYTES;  // 16 KB

struct PrefixArgs {
  const __half* q;    // branch b, head h at q + b*q_stride + h*D
  int64_t q_stride;
  const __half* pk;   // key t of kv head h at pk + t*key_stride + h*head_stride
  const __half* pv;
  float* pm;          // [nsp][B*H]
  float* pl;
  float* po;          // [nsp][B*H][D]
  int64_t key_stride, head_stride;   // elements between consecutive keys / kv heads of pk, pv
  const int32_t* prefix_len_dev;     // optional device scalar overriding prefix_len (<= prefix_len)
  int B, H, Hkv, prefix_len, keys_per_split;
  float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
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
  return (uint32_t)(row * PF_ROW_BYTES + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// grid: (nsp, Hkv, row blocks); block: NWARPS*32 threads, 16 query rows per warp.
template <int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
attn_prefix_kernel(const PrefixArgs a) {
  constexpr int D = ATTN_D;
  constexpr int RB = NWARPS * 16;
  constexpr int NT = NWARPS * 32;
  extern __shared__ __align__(128) unsigned char smem[];
  // [stage][K tile | V tile]; the Q rows are staged through the same memory first
  const uint32_t sbase = smem_u32(smem);
  asm volatile("griddepcontrol.launch_dependents;");   // a dependent may start prefetching its weights
  asm volatile("griddepcontrol.wait;" ::: "memory");               // ... but nothing of the previous launch is read before it is done

  const int sp = blockIdx.x, hk = blockIdx.y, rblk = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rep = a.H / a.Hkv;
  const int rows = a.B * rep;                 // query rows of this kv head
  const int row0 = rblk * RB;
  const int plen = a.prefix_len_dev ? min(max(a.prefix_len_dev[0], 0), a.prefix_len) : a.prefix_len;
  const int k_begin = sp * a.keys_per_split;
  const int k_end = min(plen, k_begin + a.keys_per_split);
  const int ntiles = (k_end > k_begin) ? (k_end - k_begin + PF_KT - 1) / PF_KT : 0;

  // ---- Q rows -> shared (swizzled) -> A fragments in registers ----
  for (int idx = tid; idx < RB * 16; idx += NT) {
    const int r = idx >> 4, ch = idx & 15;
    const int gr = row0 + r;
    const bool ok = gr < rows;
    const int b = ok ? gr / rep : 0, j = ok ? gr % rep : 0;
    const __half* src = a.q + (int64_t)b * a.q_stride + (hk * rep + j) * D + ch * 8;
    cp_async16(sbase + tile_off(r, ch), src, ok);
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
    const int key0 = k_begin + tile * PF_KT;
    const uint32_t kdst = sbase + stage * 2 * PF_TILE_BYTES;
    const uint32_t vdst = kdst + PF_TILE_BYTES;
    for (int idx = tid; idx < PF_KT * 16; idx += NT) {
      const int r = idx >> 4, ch = idx & 15;
      const int key = key0 + r;
      const bool ok = key < k_end;
      const int64_t off = (int64_t)(ok ? key : k_begin) * a.key_stride + (int64_t)hk * a.head_stride + ch * 8;
      cp_async16(kdst + tile_off(r, ch), a.pk + off, ok);
      cp_async16(vdst + tile_off(r, ch), a.pv + off, ok);
    }
  };

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
    const uint32_t kt = sbase + stage * 2 * PF_TILE_BYTES;
    const uint32_t vt = kt + PF_TILE_BYTES;

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
    // ---- scale, mask the tail, online softmax (rows g and g+8 of this warp) ----
    const int key0 = k_begin + tile * PF_KT;
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = key0 + nt * 8 + 2 * t + (j & 1);
        const float v = (key < k_end) ? sacc[nt][j] * a.scale_log2 : -CUDART_INF_F;
        sacc[nt][j] = v;
        mx[j >> 1] = fmaxf(mx[j >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mnew = fmaxf(m_run[r], mx[r]);   // finite: every tile holds at least one key
      corr[r] = exp2f(m_run[r] - mnew);
      m_run[r] = mnew;
      l_run[r] *= corr[r];
    }
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = exp2f(sacc[nt][j] - m_run[j >> 1]);
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
    __syncthreads();  // all warps are done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // ---- write the partial (m, l, O) of rows g and g+8 ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const int64_t total_rows = (int64_t)a.B * a.H;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int gr = row0 + warp * 16 + g + r * 8;
    if (gr >= rows) continue;
    const int b = gr / rep, j = gr % rep;
    const int64_t ridx = (int64_t)sp * total_rows + (int64_t)b * a.H + hk * rep + j;
    if (t == 0) { a.pm[ridx] = m_run[r]; a.pl[ridx] = l_run[r]; }
    float* dst = a.po + ridx * D;
#pragma unroll
    for (int dt = 0; dt < 16; ++dt)
      *reinterpret_cast<float2*>(dst + dt * 8 + 2 * t) = make_float2(oacc[dt][2 * r], oacc[dt][2 * r + 1]);
  }
}

static int prefix_splits(int B, int H, int Hkv, int prefix_len) {
  const int rep = H / Hkv;
  const int rows = B * rep;
  const int rblocks = (rows + 127) / 128;
  const int tiles = (prefix_len + PF_KT - 1) / PF_KT;
  // CTAs per SM to aim for: two for the 64-row variant (128 threads; measured best for 2048 keys x 64
  // rows), one for the 128-row variant; never round up past whole waves (a 149th CTA doubles the time
  // of one SM)
  const int per_sm = rows <= 64 ? 2 : 1;
  int want = (148 * per_sm) / (Hkv * rblocks);
  if (want < 1) want = 1;
  if (want > tiles) want = tiles;
  if (want < 1) want = 1;
  const int tiles_per = (tiles + want - 1) / want;
  return (tiles + tiles_per - 1) / tiles_per;               // every split is non-empty
}

// pa.prefix_len is the (maximum) prefix length the grid is sized for
static int launch_prefix(PrefixArgs& pa, int nsp, cudaStream_t st) {
  const int tiles = (pa.prefix_len + PF_KT - 1) / PF_KT;
  pa.keys_per_split = ((tiles + nsp - 1) / nsp) * PF_KT;
  const int rep = pa.H / pa.Hkv, rows = pa.B * rep;
  const size_t smem = 4 * PF_TILE_BYTES;  // two stages of K and V (also covers 128 staged Q rows)
  if (rows <= 64) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefix_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = q40_launch_pdl(attn_prefix_kernel<4>, dim3(nsp, pa.Hkv, 1), dim3(128), smem, st, pa);
    if (e != cudaSuccess) return (int)e;
  } else {
    cudaError_t e = cudaFuncSetAttribute(attn_prefix_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = q40_launch_pdl(attn_prefix_kernel<8>, dim3(nsp, pa.Hkv, (rows + 127) / 128), dim3(256), smem, st, pa);
    if (e != cudaSuccess) return (int)e;
  }
  return Q40_OK;
}

}  // namespace q40

extern "C" size_t q40_attn_shared_prefix_workspace_bytes(int B, int H, int D, int prefix_len) {
  if (B <= 0 || H <= 0 || D != q40::ATTN_D || prefix_len <= 0) return 0;
  // the split count depends on Hkv; Hkv = 1 with 128-row blocks gives the largest count
  const int tiles = (prefix_len + q40::PF_KT - 1) / q40::PF_KT;
  const int max_sp = tiles < 296 ? tiles : 296;
  return (size_t)max_sp * B * H * (D + 2) * sizeof(float);
}

extern "C" int q40_attn_shared_prefix(const void* q, const void* prefix_k, const void* prefix_v,
                                      int prefix_len, int64_t prefix_key_stride,
                                      int64_t prefix_head_stride, const void* page_tbl, int idx_bytes,
                                      int64_t tbl_stride, const int32_t* seq_lens, const void* kpool,
                                      const void* vpool, void* o, int P, int B, int Lmax, int H, int Hkv,
                                      int D, int page_size, void* workspace, size_t workspace_bytes,
                                      void* stream) {
  using namespace q40;
  if (!q || !o) return Q40_E_NULL;
  if (D != ATTN_D) return Q40_E_UNSUPPORTED;
  if (B < 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || prefix_len < 0 || Lmax < 0 || P < 0 || page_size <= 0)
    return Q40_E_SHAPE;
  if (idx_bytes != 2 && idx_bytes != 4) return Q40_E_UNSUPPORTED;
  if (prefix_len > 0 && (!prefix_k || !prefix_v)) return Q40_E_NULL;
  if (prefix_len > 0 && (prefix_key_stride % 8 != 0 || prefix_head_stride % 8 != 0)) return Q40_E_ALIGN;
  if (Lmax > 0 && (!page_tbl || !kpool || !vpool || P == 0)) return Q40_E_NULL;
  if (Lmax > 0 && tbl_stride < (Lmax + page_size - 1) / page_size) return Q40_E_SHAPE;
  if (B == 0) return Q40_OK;
  if (!q40_aligned(q, 16) || !q40_aligned(prefix_k, 16) || !q40_aligned(prefix_v, 16) ||
      !q40_aligned(kpool, 16) || !q40_aligned(vpool, 16))
    return Q40_E_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows_total = (int64_t)B * H;

  BranchArgs br{};
  br.q = (const __half*)q; br.q_stride = (int64_t)H * D; br.k = (const __half*)kpool; br.v = (const __half*)vpool; br.o = (__half*)o;
  br.tbl = page_tbl; br.tbl_stride = tbl_stride; br.seq_lens = seq_lens;
  br.L = Lmax; br.H = H; br.Hkv = Hkv; br.P = P; br.page_size = page_size;
  br.scale_log2 = attn_scale_log2(D);

  if (prefix_len > 0) {
    const int nsp = prefix_splits(B, H, Hkv, prefix_len);
    const size_t need = (size_t)nsp * rows_total * (D + 2) * sizeof(float);
    if (!workspace || workspace_bytes < need) return Q40_E_WORKSPACE;
    if (!q40_aligned(workspace, 16)) return Q40_E_ALIGN;
    float* po = (float*)workspace;
    float* pm = po + (size_t)nsp * rows_total * D;
    float* pl = pm + (size_t)nsp * rows_total;
    PrefixArgs pa{};
    pa.q = (const __half*)q; pa.q_stride = (int64_t)H * D; pa.pk = (const __half*)prefix_k; pa.pv = (const __half*)prefix_v;
    pa.pm = pm; pa.pl = pl; pa.po = po;
    pa.key_stride = prefix_key_stride; pa.head_stride = prefix_head_stride;
    pa.B = B; pa.H = H; pa.Hkv = Hkv; pa.prefix_len = prefix_len;
    pa.scale_log2 = br.scale_log2;
    int rc = launch_prefix(pa, nsp, st);
    if (rc != Q40_OK) return rc;
    br.pm = pm; br.pl = pl; br.po = po; br.nsp = nsp;
  }
  // Lmax == 0: the branch kernel only merges the prefix partials
  const int mode = (Lmax == 0) ? 0 : (idx_bytes == 2 ? 1 : 2);
  if (Lmax == 0) { br.seq_lens = nullptr; br.L = 0; }
  return launch_branch(br, mode, B, st);
}

extern "C" int q40_attn_tree_decode(const void* q, int64_t q_stride, const void* prefix_k, const void* prefix_v,
                                    int max_prefix_len, const int32_t* prefix_len_dev,
                                    int64_t prefix_key_stride, int64_t prefix_head_stride,
                                    const void* cache_kq, const void* cache_ks, const void* cache_vq,
                                    const void* cache_vs, int max_t, const int32_t* pos_dev,
                                    const void* cur_k, const void* cur_v, int64_t cur_stride, void* o, int B,
                                    int H, int Hkv, int D, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  using namespace q40;
  if (!q || !o || !prefix_k || !prefix_v || !prefix_len_dev || !pos_dev) return Q40_E_NULL;
  if (!cache_kq || !cache_ks || !cache_vq || !cache_vs) return Q40_E_NULL;
  if ((cur_k == nullptr) != (cur_v == nullptr)) return Q40_E_NULL;
  if (D != ATTN_D) return Q40_E_UNSUPPORTED;
  if (B < 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || max_prefix_len <= 0 || max_t <= 0) return Q40_E_SHAPE;
  if (prefix_key_stride % 8 != 0 || prefix_head_stride % 8 != 0 || cur_stride % 8 != 0 || q_stride % 8 != 0)
    return Q40_E_ALIGN;
  if (q_stride < (int64_t)H * D) return Q40_E_SHAPE;
  if (B == 0) return Q40_OK;
  if (!q40_aligned(q, 16) || !q40_aligned(prefix_k, 16) || !q40_aligned(prefix_v, 16) ||
      !q40_aligned(cache_kq, 16) || !q40_aligned(cache_vq, 16) || !q40_aligned(cur_k, 16) ||
      !q40_aligned(cur_v, 16))
    return Q40_E_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows_total = (int64_t)B * H;
  const int nsp = prefix_splits(B, H, Hkv, max_prefix_len);
  const size_t need = (size_t)nsp * rows_total * (D + 2) * sizeof(float);
  if (!workspace || workspace_bytes < need) return Q40_E_WORKSPACE;
  if (!q40_aligned(workspace, 16)) return Q40_E_ALIGN;
  float* po = (float*)workspace;
  float* pm = po + (size_t)nsp * rows_total * D;
  float* pl = pm + (size_t)nsp * rows_total;
  PrefixArgs pa{};
  pa.q = (const __half*)q; pa.q_stride = q_stride; pa.pk = (const __half*)prefix_k; pa.pv = (const __half*)prefix_v;
  pa.pm = pm; pa.pl = pl; pa.po = po;
  pa.key_stride = prefix_key_stride; pa.head_stride = prefix_head_stride;
  pa.prefix_len_dev = prefix_len_dev;
  pa.B = B; pa.H = H; pa.Hkv = Hkv; pa.prefix_len = max_prefix_len;
  pa.scale_log2 = attn_scale_log2(D);
  int rc = launch_prefix(pa, nsp, st);
  if (rc != Q40_OK) return rc;
  BranchArgs br{};
  br.q = (const __half*)q; br.q_stride = q_stride; br.o = (__half*)o;
  br.H = H; br.Hkv = Hkv; br.L = max_t;
  br.scale_log2 = pa.scale_log2;
  br.pm = pm; br.pl = pl; br.po = po; br.nsp = nsp;
  br.kq = (const int8_t*)cache_kq; br.ksc = (const __half*)cache_ks;
  br.vq = (const int8_t*)cache_vq; br.vsc = (const __half*)cache_vs;
  br.pos = pos_dev; br.prefix_len = prefix_len_dev; br.max_t = max_t;
  br.cur_k = (const __half*)cur_k; br.cur_v = (const __half*)cur_v; br.cur_stride = cur_stride;
  return launch_branch(br, 3, B, st);
}
