// One decode step of the Q4_0 model (up to 8 branches) as a single persistent kernel.
//
// Why: at batch 1 a layer is seven short, dependent kernels, and each of them pays a launch, a
// DRAM-latency ramp and a reduction tail that are long next to the ~1.4-7 us its weights take
// to stream.  Here all CTAs stay resident for the whole step (2 per SM, in thread-block
// clusters of 16 or 8) and walk the same static phase list
//     embed | per layer: [wq,wk,wv] . attention . wo . [w1,w3] . w2 | final norm
// separated by grid-wide barriers.  Weights do not depend on activations, so every warp keeps
// queueing cp.async copies of its next 16-row steps — across item, phase and layer boundaries —
// into its lane-private ring while it waits at a barrier: the HBM stream does not stop at
// the dependencies.
//
// A matmul item is one 128-byte span of the packed rows (256 output features); the CTAs of a
// cluster split K, sum through distributed shared memory and finish disjoint column slices
// (RMSNorm prologue, residual / SiLU-mul epilogues as in q40_gemv_fused.cu, same arithmetic
// and rounding points).  An attention item is one (branch, head): the cluster's CTAs split
// the keys (shared fp16 prompt, packed Q4_0 suffix, the un-quantised new token), merge their
// online-softmax states through distributed shared memory, and the head's rotary embedding
// and Q4_0 cache append happen in the same place.
//
// Every wait on another CTA is bounded (iteration limit, then an error word is set and the
// kernel carries on to its end); data exchanged between CTAs is read with L1-bypassing loads.
//
// Reference semantics: Transformer.forward / TransformerBlock.forward / Attention.forward
// decode branch / FeedForward.forward (hf_model_q40_kv_shared.py:303-409, 431-436, 456-510).
#include <cooperative_groups.h>
#include <math_constants.h>

#include "q40_common.cuh"

namespace cg = cooperative_groups;

namespace q40 {

constexpr int DS_WARPS = 8;
constexpr int DS_THREADS = DS_WARPS * 32;
constexpr int DS_DEPTH = 2;                        // ring slots per warp
constexpr int DS_SLOT_W = 4 * 32 * 16;
constexpr int DS_SLOT_BYTES = DS_SLOT_W + 4 * 32 * 4;
constexpr int DS_SPAN_BYTES = 128;
constexpr int DS_SPAN_COLS = 256;
constexpr int DS_XS_PAD = 16;
constexpr unsigned DS_SPIN_LIMIT = 1u << 21;

struct DsLayer {            // device pointers of one layer (all packed as 64-bit words by the host)
  const uint8_t* w[7];      // wq wk wv wo w1 w3 w2 : packed [K, N/2]
  const __half* s[7];       // scales [K, N/64]
  const __half* attn_norm;
  const __half* ffn_norm;
  const __half* pk;         // prompt cache [maxP, Hkv, 128]
  const __half* pv;
  int8_t* kq;               // suffix cache [maxB, maxT, Hkv, 64]
  __half* ks;               // [maxB, maxT, Hkv, 2]
  int8_t* vq;
  __half* vs;
};

struct DsParams {
  const DsLayer* layers;
  int n_layers, M, dim, H, Hkv, hidden, vocab, max_t, max_p, n_pos;
  float eps;
  const __half* emb;
  const __half* final_norm;
  const int64_t* tokens;
  const int32_t* pos;
  const int32_t* prefix_len;
  const __half* cos_tbl;
  const __half* sin_tbl;
  // state (global scratch owned by the caller)
  __half* h;        // [M, dim] residual stream
  __half* qkv;      // [M, (H + 2 Hkv) * 128]
  __half* ao;       // [M, H * 128]
  __half* g;        // [M, hidden]
  __half* xn;       // [M, dim] final normalised hidden state (input of the lm_head)
  float* ss_a;      // [M, 1024] sum-of-squares partials written by wo (and by the embedding)
  float* ss_f;      // [M, 1024] ... written by w2
  unsigned int* bar;   // zeroed by the host before the launch
  int* err;
  int rps_max;      // largest rows-per-split over all phases (sizes the activation staging)
  unsigned long long* trace;   // optional: CTA 0 stores the global timer after every grid barrier
};

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ds_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ds_cp16(uint32_t dst, const void* src, bool ok) {
  const int sz = ok ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void ds_cp4(uint32_t dst, const void* src, bool ok) {
  const int sz = ok ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ unsigned ds_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// L1-bypassing loads for data another CTA wrote during this launch
__device__ __forceinline__ uint4 ds_ld16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float ds_ldf(const float* p) { return __ldcg(p); }
__device__ __forceinline__ __half ds_ldh(const __half* p) {
  return __ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(p)));
}

__device__ __forceinline__ int ds_span_col(int span, int lc) {
  const int cb = span * DS_SPAN_BYTES + (lc & (DS_SPAN_BYTES - 1));
  return 128 * (cb >> 6) + (cb & 63) + ((lc >> 7) ? 64 : 0);
}

// All CTAs of the grid meet here.  `gen` counts barriers since the launch.
__device__ __forceinline__ void ds_grid_barrier(const DsParams& p, unsigned& gen) {
  __syncthreads();
  ++gen;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(p.bar, 1u);
    const unsigned target = gen * gridDim.x;
    unsigned spins = 0;
    while (ds_ld_acquire(p.bar) < target) {
      // give up after the limit, or at once when an earlier barrier already gave up somewhere
      if (++spins > DS_SPIN_LIMIT || *reinterpret_cast<volatile int*>(p.err) != 0) { atomicExch(p.err, 2); break; }
      __nanosleep(64);
    }
    __threadfence();
    if (p.trace && blockIdx.x == 0) {
      unsigned long long tm;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm));
      p.trace[gen] = tm;
    }
  }
  __syncthreads();
}

// fine-grained profiling aid: CTA 0, thread 0 stamps the timer into trace[slot]
#define DS_STAMP(slot)                                                           \
  do {                                                                           \
    if (p.trace && blockIdx.x == 0 && threadIdx.x == 0 && layer == 1) {          \
      unsigned long long tm__;                                                   \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm__));                   \
      p.trace[(slot)] = tm__;                                                    \
    }                                                                            \
  } while (0)

// --------------------------------------------------------------------------------- weight stream
enum { PH_QKV = 0, PH_ATTN = 1, PH_WO = 2, PH_W13 = 3, PH_W2 = 4, PH_COUNT = 5 };

struct ItemPos { int layer, ph, it; };

struct Stream {       // what one lane needs to queue a step of an item
  const uint8_t* wstep;
  const __half* sstep;
  int64_t w_ld, s_ld;   // bytes / elements per k row
  int my_steps;         // steps of this warp in the item
  bool col_ok;
};

struct Geo {          // per-kernel constants derived from DsParams
  int cs, ncl, cluster_id, rank;
  int spans_q, spans_kv, spans_dim, spans_hid;
};

__device__ __forceinline__ int ds_items(const Geo& g, int ph) {
  switch (ph) {
    case PH_QKV: return g.spans_q + 2 * g.spans_kv;
    case PH_WO: return g.spans_dim;
    case PH_W13: return g.spans_hid;       // (w1, w3) pairs
    case PH_W2: return g.spans_dim;
    default: return 0;
  }
}

// next matmul item of this cluster after `a` (a.it may be -1 - ncl to mean "before the first")
__device__ __forceinline__ bool ds_next_item(const DsParams& p, const Geo& g, ItemPos& a) {
  a.it += g.ncl;
  while (a.layer < p.n_layers) {
    if (a.ph != PH_ATTN && a.it < ds_items(g, a.ph)) return true;
    a.it = g.cluster_id;
    if (++a.ph == PH_COUNT) { a.ph = 0; ++a.layer; }
  }
  return false;
}

// K rows, split count and split index of a phase for this CTA
__device__ __forceinline__ void ds_split(const DsParams& p, const Geo& g, int ph, int& K, int& nsplit, int& split,
                                         int& rps) {
  K = (ph == PH_W2) ? p.hidden : ((ph == PH_WO) ? p.H * 128 : p.dim);
  nsplit = (ph == PH_W13) ? g.cs / 2 : g.cs;
  split = (ph == PH_W13) ? (g.rank >> 1) : g.rank;
  rps = ((K + nsplit - 1) / nsplit + 15) / 16 * 16;
}

__device__ __forceinline__ Stream ds_stream(const DsParams& p, const Geo& g, const ItemPos& a, int warp, int lane) {
  Stream st;
  const DsLayer& L = p.layers[a.layer];
  int mat, span = a.it, N;
  if (a.ph == PH_QKV) {
    if (span < g.spans_q) { mat = 0; N = p.H * 128; }
    else if (span < g.spans_q + g.spans_kv) { mat = 1; span -= g.spans_q; N = p.Hkv * 128; }
    else { mat = 2; span -= g.spans_q + g.spans_kv; N = p.Hkv * 128; }
  } else if (a.ph == PH_WO) { mat = 3; N = p.dim; }
  else if (a.ph == PH_W13) { mat = 4 + (g.rank & 1); N = p.hidden; }
  else { mat = 6; N = p.dim; }
  int K, nsplit, split, rps;
  ds_split(p, g, a.ph, K, nsplit, split, rps);
  const int kb = split * rps, ke = min(K, kb + rps);
  const int nsteps = (ke > kb) ? (ke - kb) / 16 : 0;
  st.my_steps = (nsteps > warp) ? (nsteps - warp + DS_WARPS - 1) / DS_WARPS : 0;
  st.w_ld = N / 2;
  st.s_ld = N / 64;
  const int gq = lane >> 2, t = lane & 3;
  const int colbyte = span * DS_SPAN_BYTES + 16 * gq;
  st.col_ok = colbyte < st.w_ld;
  const int cb = st.col_ok ? colbyte : 0;
  st.wstep = L.w[mat] + (int64_t)(kb + warp * 16 + 4 * t) * st.w_ld + cb;
  st.sstep = L.s[mat] + (int64_t)(kb + warp * 16 + 4 * t) * st.s_ld + 2 * (cb >> 6);
  return st;
}

struct Ring {           // per-warp bookkeeping of the cp.async ring (identical in all lanes)
  uint32_t base;        // shared address of this warp's slots + lane * 16
  unsigned issued, consumed, committed;
  unsigned grp0, grp1;  // commit index of the group that filled slot 0 / 1 (DS_DEPTH == 2)
};

__device__ __forceinline__ void ds_issue(Ring& r, const Stream& st, int j, int lane) {
  const unsigned slot = r.issued % DS_DEPTH;
  const uint32_t b = r.base + slot * DS_SLOT_BYTES;
  const uint8_t* wp = st.wstep + (int64_t)j * (DS_WARPS * 16) * st.w_ld;
  const __half* sp = st.sstep + (int64_t)j * (DS_WARPS * 16) * st.s_ld;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    ds_cp16(b + q * 512, wp + q * st.w_ld, st.col_ok);
    ds_cp4(b + DS_SLOT_W - lane * 12 + q * 128, sp + q * st.s_ld, st.col_ok);
  }
  asm volatile("cp.async.commit_group;");
  if (slot == 0) r.grp0 = r.committed; else r.grp1 = r.committed;
  ++r.committed;
  ++r.issued;
}

// queue as many steps as the ring has room for: first the current item's, then the next item's
__device__ __forceinline__ void ds_fill(Ring& r, const Stream& cur, int& cur_issued, const Stream& nxt,
                                        int& nxt_issued, bool nxt_valid, int lane) {
  while (r.issued - r.consumed < DS_DEPTH) {
    if (cur_issued < cur.my_steps) ds_issue(r, cur, cur_issued++, lane);
    else if (nxt_valid && nxt_issued < nxt.my_steps) ds_issue(r, nxt, nxt_issued++, lane);
    else break;
  }
}

// --------------------------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(DS_THREADS, 2)
decode_step_kernel(const DsParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, t = lane & 3;

  Geo g;
  g.cs = (int)cluster.num_blocks();
  g.ncl = gridDim.x / g.cs;
  g.cluster_id = blockIdx.x / g.cs;
  g.rank = (int)cluster.block_rank();
  g.spans_q = (p.H * 128 / 2 + DS_SPAN_BYTES - 1) / DS_SPAN_BYTES;
  g.spans_kv = (p.Hkv * 128 / 2 + DS_SPAN_BYTES - 1) / DS_SPAN_BYTES;
  g.spans_dim = (p.dim / 2 + DS_SPAN_BYTES - 1) / DS_SPAN_BYTES;
  g.spans_hid = (p.hidden / 2 + DS_SPAN_BYTES - 1) / DS_SPAN_BYTES;

  // shared memory carve-up
  const int xs_ld = p.rps_max + DS_XS_PAD;
  unsigned char* ring_mem = smem;                                                  // DS_WARPS*DEPTH slots
  __half* xs = reinterpret_cast<__half*>(smem + DS_WARPS * DS_DEPTH * DS_SLOT_BYTES);   // [8][xs_ld]
  __half* wn = xs + 8 * xs_ld;                                                     // [rps_max]
  float* s_inv = reinterpret_cast<float*>(wn + p.rps_max);                         // [16]
  float4* slab = reinterpret_cast<float4*>(s_inv + 16);                            // [4][16][32] float4
  float* cta_part = reinterpret_cast<float*>(slab + 4 * 16 * 32);                  // [8][256]
  // attention scratch aliases the slabs
  float* at_m = reinterpret_cast<float*>(slab);           // [32 groups]
  float* at_l = at_m + 32;
  float* at_o = at_l + 32;                                 // [32][128]
  float* at_part = cta_part;                               // CTA partial: m, l, o[128] (130 floats)

  Ring ring;
  ring.base = (uint32_t)__cvta_generic_to_shared(ring_mem) + warp * (DS_DEPTH * DS_SLOT_BYTES) + lane * 16;
  ring.issued = ring.consumed = ring.committed = 0;
  ring.grp0 = ring.grp1 = 0;
  static_assert(DS_DEPTH == 2, "the ring bookkeeping below is written for two slots");

  // the first two matmul items of this cluster, and the head of the weight stream
  ItemPos cur_pos{0, 0, g.cluster_id - g.ncl};
  bool cur_valid = ds_next_item(p, g, cur_pos);
  ItemPos nxt_pos = cur_pos;
  bool nxt_valid = cur_valid && ds_next_item(p, g, nxt_pos);
  Stream cur = cur_valid ? ds_stream(p, g, cur_pos, warp, lane) : Stream{};
  Stream nxt = nxt_valid ? ds_stream(p, g, nxt_pos, warp, lane) : Stream{};
  if (!cur_valid) cur.my_steps = 0;
  int cur_issued = 0, nxt_issued = 0;
  ds_fill(ring, cur, cur_issued, nxt, nxt_issued, nxt_valid, lane);

  unsigned gen = 0;
  if (p.trace && blockIdx.x == 0 && tid == 0) p.trace[399] = gridDim.x;   // resident CTAs (profiling aid)
  const int M = p.M;
  const int W = (p.H + 2 * p.Hkv) * 128;
  const int cnt_a = g.spans_dim * g.cs;      // partial count of the sums of squares (wo / w2 / embed)
  const float scale_log2 = (1.0f / sqrtf(128.0f)) * 1.4426950408889634f;

  // ------------------------------------------------------------------ embedding
  for (int m = blockIdx.x; m < M; m += gridDim.x) {
    int64_t tok = p.tokens[m];
    tok = tok < 0 ? 0 : (tok >= p.vocab ? p.vocab - 1 : tok);
    const __half* src = p.emb + tok * p.dim;
    float s = 0.f;
    for (int i = tid * 8; i < p.dim; i += DS_THREADS * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + i);
      *reinterpret_cast<uint4*>(p.h + (int64_t)m * p.dim + i) = v;
      const __half2* vh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(vh[j]);
        s = fmaf(f.x, f.x, s);
        s = fmaf(f.y, f.y, s);
      }
    }
    s = warp_sum(s);
    if (lane == 0) s_inv[warp] = s;
    __syncthreads();
    for (int i = tid; i < cnt_a; i += DS_THREADS) {
      float tot = 0.f;
      if (i == 0)
        for (int w = 0; w < DS_WARPS; ++w) tot += s_inv[w];
      p.ss_f[(int64_t)m * 1024 + i] = tot;
    }
    __syncthreads();
  }
  ds_grid_barrier(p, gen);

  // ------------------------------------------------------------------ layers
  for (int layer = 0; layer < p.n_layers; ++layer) {
    const DsLayer& L = p.layers[layer];
    for (int ph = 0; ph < PH_COUNT; ++ph) {
      if (ph == PH_ATTN) {
        // ====================== attention: one (branch, head) per cluster ======================
        DS_STAMP(400 + 16);
        const int plen = min(max(p.prefix_len[0], 0), p.max_p);
        const int rep = p.H / p.Hkv;
        const int grp = tid >> 3, sub = tid & 7;          // 32 key groups of 8 lanes per CTA
        const unsigned gmask = 0xffu << (lane & 24);
        const int ngroups = 32 * g.cs;                     // over the whole cluster
        const int gidx = g.rank * 32 + grp;
        for (int it = g.cluster_id; it < M * p.H; it += g.ncl) {
          const int b = it / p.H, hq = it % p.H, hk = hq / rep;
          int pos = p.pos[b];
          pos = min(max(pos, 0), p.n_pos - 1);
          const int slen = min(max(pos - plen, 0), p.max_t);
          // this lane's 16 dims of the rotated, pre-scaled query, and of the rotated new key
          float qf[16];
          __half kc[16], vc[16];
          {
            const __half* qp = p.qkv + (int64_t)b * W + hq * 128;
            const __half* kp = p.qkv + (int64_t)b * W + (p.H + hk) * 128;
            const __half* vp = p.qkv + (int64_t)b * W + (p.H + p.Hkv + hk) * 128;
            const int d0 = sub * 16, dp = (d0 + 64) & 127;     // partner half for the rotation
            const bool lo_half = d0 < 64;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const __half c = p.cos_tbl[(int64_t)pos * 64 + ((d0 + i) & 63)];
              const __half s = p.sin_tbl[(int64_t)pos * 64 + ((d0 + i) & 63)];
              const __half q1 = ds_ldh(qp + d0 + i), q2 = ds_ldh(qp + dp + i);
              const __half k1 = ds_ldh(kp + d0 + i), k2 = ds_ldh(kp + dp + i);
              // out = x*cos + rot(x)*sin, rot(x) = -partner for the low half, +partner for the high half
              const __half qr = __hadd_rn(__hmul_rn(q1, c), __hmul_rn(lo_half ? __hneg(q2) : q2, s));
              kc[i] = __hadd_rn(__hmul_rn(k1, c), __hmul_rn(lo_half ? __hneg(k2) : k2, s));
              vc[i] = ds_ldh(vp + d0 + i);
              qf[i] = __half2float(qr) * scale_log2;
            }
          }
          if (it == g.cluster_id) DS_STAMP(400 + 17);
          float mx = -CUDART_INF_F, l = 0.f, o[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = 0.f;
          // keys: [0, plen) prompt (fp16), [plen, plen + slen) suffix (Q4_0), then the new token
          const int total_keys = plen + slen + 1;
          for (int key = gidx; key < total_keys; key += ngroups) {
            float kv_k[16], kv_v[16];
            if (key < plen) {
              const int64_t off = ((int64_t)key * p.Hkv + hk) * 128 + sub * 16;
              const uint4 k0 = __ldg(reinterpret_cast<const uint4*>(L.pk + off));
              const uint4 k1 = __ldg(reinterpret_cast<const uint4*>(L.pk + off + 8));
              const uint4 v0 = __ldg(reinterpret_cast<const uint4*>(L.pv + off));
              const uint4 v1 = __ldg(reinterpret_cast<const uint4*>(L.pv + off + 8));
              const __half2* a0 = reinterpret_cast<const __half2*>(&k0);
              const __half2* a1 = reinterpret_cast<const __half2*>(&k1);
              const __half2* c0 = reinterpret_cast<const __half2*>(&v0);
              const __half2* c1 = reinterpret_cast<const __half2*>(&v1);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                float2 f = __half22float2(a0[i]); kv_k[2 * i] = f.x; kv_k[2 * i + 1] = f.y;
                f = __half22float2(a1[i]); kv_k[8 + 2 * i] = f.x; kv_k[8 + 2 * i + 1] = f.y;
                f = __half22float2(c0[i]); kv_v[2 * i] = f.x; kv_v[2 * i + 1] = f.y;
                f = __half22float2(c1[i]); kv_v[8 + 2 * i] = f.x; kv_v[8 + 2 * i + 1] = f.y;
              }
            } else if (key < plen + slen) {
              const int64_t row = ((int64_t)b * p.max_t + (key - plen)) * p.Hkv + hk;
              const int nib_lo = sub >> 2, boff = 16 * (sub & 3);
              const uint4 kb4 = __ldg(reinterpret_cast<const uint4*>(L.kq + row * 64 + boff));
              const uint4 vb4 = __ldg(reinterpret_cast<const uint4*>(L.vq + row * 64 + boff));
              const __half2 ksc = __half2half2(L.ks[row * 2 + nib_lo]);
              const __half2 vsc = __half2half2(L.vs[row * 2 + nib_lo]);
              const uint32_t* kw = reinterpret_cast<const uint32_t*>(&kb4);
              const uint32_t* vw = reinterpret_cast<const uint32_t*>(&vb4);
#pragma unroll
              for (int wi = 0; wi < 4; ++wi) {
                const uint32_t a = nib_lo ? kw[wi] : (kw[wi] >> 4);
                const uint32_t c = nib_lo ? vw[wi] : (vw[wi] >> 4);
                float2 f = __half22float2(__hmul2(codes_lo_to_h2(a), ksc));
                kv_k[4 * wi] = f.x; kv_k[4 * wi + 2] = f.y;
                f = __half22float2(__hmul2(codes_lo_to_h2(a >> 8), ksc));
                kv_k[4 * wi + 1] = f.x; kv_k[4 * wi + 3] = f.y;
                f = __half22float2(__hmul2(codes_lo_to_h2(c), vsc));
                kv_v[4 * wi] = f.x; kv_v[4 * wi + 2] = f.y;
                f = __half22float2(__hmul2(codes_lo_to_h2(c >> 8), vsc));
                kv_v[4 * wi + 1] = f.x; kv_v[4 * wi + 3] = f.y;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) { kv_k[i] = __half2float(kc[i]); kv_v[i] = __half2float(vc[i]); }
            }
            float sdot = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) sdot = fmaf(qf[i], kv_k[i], sdot);
            sdot += __shfl_xor_sync(gmask, sdot, 1);
            sdot += __shfl_xor_sync(gmask, sdot, 2);
            sdot += __shfl_xor_sync(gmask, sdot, 4);
            const float mnew = fmaxf(mx, sdot);
            const float corr = exp2f(mx - mnew), pw = exp2f(sdot - mnew);
            l = l * corr + pw;
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = fmaf(pw, kv_v[i], o[i] * corr);
            mx = mnew;
          }
          // Q4_0 append of the new token's rotated key and its value: the first query head of a kv
          // group, rank 0, key group 0 (the 8 lanes hold the whole 128-dim row)
          if (g.rank == 0 && grp == 0 && (hq % rep) == 0 && (pos - plen) >= 0 && (pos - plen) < p.max_t) {
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
            const int64_t row = ((int64_t)b * p.max_t + (pos - plen)) * p.Hkv + hk;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              const uint32_t ok_ = __shfl_xor_sync(0xffu, ck[wi], 4), ov_ = __shfl_xor_sync(0xffu, cv[wi], 4);
              if (sub < 4) {
                reinterpret_cast<uint32_t*>(L.kq + row * 64 + 16 * sub)[wi] = (ck[wi] << 4) | ok_;
                reinterpret_cast<uint32_t*>(L.vq + row * 64 + 16 * sub)[wi] = (cv[wi] << 4) | ov_;
              }
            }
            if (sub == 0) { L.ks[row * 2] = sk; L.vs[row * 2] = sv; }
            if (sub == 4) { L.ks[row * 2 + 1] = sk; L.vs[row * 2 + 1] = sv; }
          }
          if (it == g.cluster_id) DS_STAMP(400 + 18);
          // merge the 32 groups of this CTA, then the CTAs of the cluster
          if (sub == 0) { at_m[grp] = mx; at_l[grp] = l; }
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<float4*>(&at_o[grp * 128 + sub * 16 + i]) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
          __syncthreads();
          if (tid < 128) {
            float Mx = -CUDART_INF_F;
            for (int q = 0; q < 32; ++q) Mx = fmaxf(Mx, at_m[q]);
            float Ls = 0.f, acc = 0.f;
            if (Mx > -CUDART_INF_F)
              for (int q = 0; q < 32; ++q) {
                const float w = exp2f(at_m[q] - Mx);
                Ls = fmaf(at_l[q], w, Ls);
                acc = fmaf(at_o[q * 128 + tid], w, acc);
              }
            at_part[2 + tid] = acc;
            if (tid == 0) { at_part[0] = Mx; at_part[1] = Ls; }
          }
          cluster.sync();
          if (it == g.cluster_id) DS_STAMP(400 + 19);
          {
            // rank r finishes dims [r*per, (r+1)*per)
            const int per = 128 / g.cs;
            if (tid < per) {
              const int d = g.rank * per + tid;
              float pm[16], pl[16], po[16];
#pragma unroll
              for (int r = 0; r < 16; ++r) {
                if (r < g.cs) {
                  const float* rp = cluster.map_shared_rank(at_part, r);
                  pm[r] = rp[0]; pl[r] = rp[1]; po[r] = rp[2 + d];
                } else { pm[r] = -CUDART_INF_F; pl[r] = 0.f; po[r] = 0.f; }
              }
              float Mx = -CUDART_INF_F;
#pragma unroll
              for (int r = 0; r < 16; ++r) Mx = fmaxf(Mx, pm[r]);
              float Ls = 0.f, acc = 0.f;
#pragma unroll
              for (int r = 0; r < 16; ++r) {
                const float w = (pm[r] > -CUDART_INF_F) ? exp2f(pm[r] - Mx) : 0.f;
                Ls = fmaf(pl[r], w, Ls);
                acc = fmaf(po[r], w, acc);
              }
              p.ao[(int64_t)b * (p.H * 128) + hq * 128 + d] = __float2half_rn(Ls > 0.f ? acc / Ls : 0.f);
            }
          }
          cluster.sync();
          if (it == g.cluster_id) DS_STAMP(400 + 20);
        }
        DS_STAMP(400 + 21);
        ds_grid_barrier(p, gen);
        continue;
      }

      // ====================== matmul phase ======================
      int K, nsplit, split, rps;
      ds_split(p, g, ph, K, nsplit, split, rps);
      const int kb = split * rps, ke = min(K, kb + rps);
      const bool has_items = g.cluster_id < ds_items(g, ph);
      DS_STAMP(400 + ph * 16 + 0);
      if (has_items) {
        // ---- activations of this CTA's k range (same for all its items of the phase) ----
        const __half* src;
        int64_t ld;
        const __half* nw = nullptr;
        const float* ssin = nullptr;
        if (ph == PH_QKV) { src = p.h; ld = p.dim; nw = L.attn_norm; ssin = p.ss_f; }
        else if (ph == PH_WO) { src = p.ao; ld = p.H * 128; }
        else if (ph == PH_W13) { src = p.h; ld = p.dim; nw = L.ffn_norm; ssin = p.ss_a; }
        else { src = p.g; ld = p.hidden; }
        const int chunks = rps / 8;
        for (int idx = tid; idx < 8 * chunks; idx += DS_THREADS) {
          const int m = idx / chunks, kk = (idx % chunks) * 8;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (m < M && kb + kk < ke) v = ds_ld16(src + (int64_t)m * ld + kb + kk);
          *reinterpret_cast<uint4*>(xs + m * xs_ld + kk) = v;
        }
        if (nw) {
          for (int idx = tid; idx < chunks; idx += DS_THREADS) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (kb + idx * 8 < ke) v = *reinterpret_cast<const uint4*>(nw + kb + idx * 8);
            *reinterpret_cast<uint4*>(wn + idx * 8) = v;
          }
          for (int m = warp; m < M; m += DS_WARPS) {
            float s = 0.f;
            for (int i = lane; i < cnt_a; i += 32) s += ds_ldf(ssin + (int64_t)m * 1024 + i);
            s = warp_sum(s);
            if (lane == 0) s_inv[m] = rsqrtf(s / (float)K + p.eps);
          }
        }
        __syncthreads();
        if (nw) {
          for (int idx = tid; idx < M * chunks; idx += DS_THREADS) {
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
      }

      DS_STAMP(400 + ph * 16 + 1);
      for (int it = g.cluster_id; it < ds_items(g, ph); it += g.ncl) {
        // `cur` describes exactly this item (the stream is walked in the same order)
        float acc[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        const __half* xlane = xs + gq * xs_ld + 4 * t;
        for (int j = 0; j < cur.my_steps; ++j) {
          const unsigned slot = ring.consumed % DS_DEPTH;
          // groups complete in order: allow as many to stay pending as were committed after ours
          if (ring.committed - 1 - (slot == 0 ? ring.grp0 : ring.grp1) >= 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
          else asm volatile("cp.async.wait_group 0;" ::: "memory");
          const unsigned char* sb = ring_mem + (warp * DS_DEPTH + slot) * DS_SLOT_BYTES;
          uint4 w[4];
          uint32_t sc[4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            w[r] = *reinterpret_cast<const uint4*>(sb + (r * 32 + lane) * 16);
            sc[r] = *reinterpret_cast<const uint32_t*>(sb + DS_SLOT_W + (r * 32 + lane) * 4);
          }
          const int step = warp + j * DS_WARPS;
          const uint2 xv = *reinterpret_cast<const uint2*>(xlane + step * 16);
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
              ds_mma(acc[wi * 4 + b], a0, a1, a2, a3, xv.x, xv.y);
            }
          }
          ++ring.consumed;
          ds_fill(ring, cur, cur_issued, nxt, nxt_issued, nxt_valid, lane);
        }
        if (it == g.cluster_id) DS_STAMP(400 + ph * 16 + 2);
        // this item's stream is exhausted: the following item becomes current, and the one after it
        // may start to prefetch while this item is reduced
        const int span = (ph == PH_QKV)
                             ? (it < g.spans_q ? it : (it < g.spans_q + g.spans_kv ? it - g.spans_q
                                                                                   : it - g.spans_q - g.spans_kv))
                             : it;
        cur = nxt; cur_issued = nxt_issued; cur_valid = nxt_valid; cur_pos = nxt_pos;
        if (!cur_valid) cur.my_steps = 0;
        nxt_pos = cur_pos;
        nxt_valid = cur_valid && ds_next_item(p, g, nxt_pos);
        if (nxt_valid) nxt = ds_stream(p, g, nxt_pos, warp, lane);
        nxt_issued = 0;
        ds_fill(ring, cur, cur_issued, nxt, nxt_issued, nxt_valid, lane);

        if (it == g.cluster_id) DS_STAMP(400 + ph * 16 + 3);
        // ---- sum the 8 warps: 4-7 store, 0-3 add, then the CTA partial ----
        if (warp >= 4) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            slab[((warp - 4) * 16 + i) * 32 + lane] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        }
        __syncthreads();
        if (warp < 4) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float4 v = slab[(warp * 16 + i) * 32 + lane];
            v.x += acc[i][0]; v.y += acc[i][1]; v.z += acc[i][2]; v.w += acc[i][3];
            slab[(warp * 16 + i) * 32 + lane] = v;
          }
        }
        __syncthreads();
        {
          const float* sl = reinterpret_cast<const float*>(slab);
          for (int idx = tid; idx < M * DS_SPAN_COLS; idx += DS_THREADS) {
            const int m = idx / DS_SPAN_COLS, lc = idx % DS_SPAN_COLS;
            const int c = lc & 127, is_lo = lc >> 7;
            const int fg = c >> 4, tb = c & 15;
            const int fl = fg * 4 + (m >> 1);
            const int off = ((tb * 32 + fl) << 2) + (m & 1) + 2 * is_lo;
            cta_part[idx] = sl[off] + sl[off + 16 * 32 * 4] + sl[off + 2 * 16 * 32 * 4] + sl[off + 3 * 16 * 32 * 4];
          }
        }
        if (it == g.cluster_id) DS_STAMP(400 + ph * 16 + 4);
        cluster.sync();
        if (it == g.cluster_id) DS_STAMP(400 + ph * 16 + 5);
        {
          const int nranks = g.cs;
          const int slice = DS_SPAN_COLS / nranks;
          const bool silu = (ph == PH_W13);
          const int npart = silu ? nranks / 2 : nranks;
          // destination and geometry of this item
          __half* out;
          int64_t ldo;
          int N;
          if (ph == PH_QKV) {
            ldo = W;
            if (it < g.spans_q) { out = p.qkv; N = p.H * 128; }
            else if (it < g.spans_q + g.spans_kv) { out = p.qkv + p.H * 128; N = p.Hkv * 128; }
            else { out = p.qkv + (p.H + p.Hkv) * 128; N = p.Hkv * 128; }
          } else if (ph == PH_W13) { out = p.g; ldo = p.hidden; N = p.hidden; }
          else { out = p.h; ldo = p.dim; N = p.dim; }
          float* ssout = (ph == PH_WO) ? p.ss_a : p.ss_f;
          for (int m = warp; m < M; m += DS_WARPS) {
            float ssq = 0.f;
            for (int cidx = lane; cidx < slice; cidx += 32) {
              const int lc = g.rank * slice + cidx;
              const int idx = m * DS_SPAN_COLS + lc;
              float v0 = 0.f, v1 = 0.f;
              if (silu) {
                float t0[8], t1[8];
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                  t0[r] = (r < npart) ? *cluster.map_shared_rank(cta_part + idx, 2 * r) : 0.f;
                  t1[r] = (r < npart) ? *cluster.map_shared_rank(cta_part + idx, 2 * r + 1) : 0.f;
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
              const int n = ds_span_col(span, lc);
              if (n < N) {
                if (ph == PH_QKV) {
                  out[(int64_t)m * ldo + n] = __float2half_rn(v0);
                } else if (silu) {
                  const float a1 = __half2float(__float2half_rn(v0));
                  const __half sg = __float2half_rn(a1 / (1.0f + expf(-a1)));
                  out[(int64_t)m * ldo + n] = __hmul_rn(sg, __float2half_rn(v1));
                } else {
                  const __half hn = __hadd_rn(ds_ldh(p.h + (int64_t)m * p.dim + n), __float2half_rn(v0));
                  out[(int64_t)m * ldo + n] = hn;
                  const float f = __half2float(hn);
                  ssq = fmaf(f, f, ssq);
                }
              }
            }
            if (ph == PH_WO || ph == PH_W2) {
              ssq = warp_sum(ssq);
              if (lane == 0) ssout[(int64_t)m * 1024 + span * nranks + g.rank] = ssq;
            }
          }
        }
        if (it == g.cluster_id) DS_STAMP(400 + ph * 16 + 6);
        cluster.sync();
        if (it == g.cluster_id) DS_STAMP(400 + ph * 16 + 7);
      }
      DS_STAMP(400 + ph * 16 + 8);
      ds_grid_barrier(p, gen);
      DS_STAMP(400 + ph * 16 + 9);
    }
  }

  // ------------------------------------------------------------------ final RMSNorm -> xn
  for (int m = blockIdx.x; m < M; m += gridDim.x) {
    if (warp == 0) {
      float s = 0.f;
      for (int i = lane; i < cnt_a; i += 32) s += ds_ldf(p.ss_f + (int64_t)m * 1024 + i);
      s = warp_sum(s);
      if (lane == 0) s_inv[0] = rsqrtf(s / (float)p.dim + p.eps);
    }
    __syncthreads();
    const float inv = s_inv[0];
    for (int i = tid * 8; i < p.dim; i += DS_THREADS * 8) {
      uint4 v = ds_ld16(p.h + (int64_t)m * p.dim + i);
      const uint4 wv = *reinterpret_cast<const uint4*>(p.final_norm + i);
      __half2* vh = reinterpret_cast<__half2*>(&v);
      const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(vh[j]);
        vh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);
      }
      *reinterpret_cast<uint4*>(p.xn + (int64_t)m * p.dim + i) = v;
    }
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

static size_t ds_smem_bytes(int rps_max) {
  return (size_t)DS_WARPS * DS_DEPTH * DS_SLOT_BYTES + (size_t)8 * (rps_max + DS_XS_PAD) * 2 + (size_t)rps_max * 2 +
         64 + (size_t)4 * 16 * 32 * 16 + (size_t)8 * 256 * 4;
}

}  // namespace q40

// One whole decode step (1 <= M <= 8 branches) as a single persistent launch.  `layers` is a device
// array of n_layers records of 22 pointers each (see DsLayer); all other pointers are device
// buffers owned by the caller; `bar` and `err` are device words the entry zeroes on the stream before
// the launch.  Leaves the final normalised hidden state in `xn` (the caller applies the lm_head).
extern "C" int q40_decode_step(const void* layers, int n_layers, int M, int dim, int H, int Hkv, int hidden,
                               int vocab, int max_t, int max_p, int n_pos, float eps, const void* emb,
                               const void* final_norm, const int64_t* tokens, const int32_t* pos,
                               const int32_t* prefix_len, const void* cos_tbl, const void* sin_tbl, void* h,
                               void* qkv, void* ao, void* g, void* xn, float* ss_a, float* ss_f,
                               unsigned int* bar, int* err, int max_cluster, unsigned long long* trace, void* stream) {
  using namespace q40;
  if (!layers || !emb || !final_norm || !tokens || !pos || !prefix_len || !cos_tbl || !sin_tbl || !h || !qkv ||
      !ao || !g || !xn || !ss_a || !ss_f || !bar || !err)
    return Q40_E_NULL;
  if (M < 1 || M > 8 || n_layers < 1 || H % Hkv != 0) return Q40_E_SHAPE;
  if (dim % 256 != 0 || hidden % 256 != 0 || (H * 128) % 256 != 0 || (Hkv * 128) % 128 != 0) return Q40_E_SHAPE;
  if (max_cluster != 8 && max_cluster != 16) return Q40_E_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const int cs = max_cluster;
  if ((dim / 2 / DS_SPAN_BYTES) * cs > 1024) return Q40_E_SHAPE;         // sum-of-squares partial slots
  auto rps_of = [](int K, int ns) { return ((K + ns - 1) / ns + 15) / 16 * 16; };
  int rps_max = rps_of(dim, cs);
  if (rps_of(H * 128, cs) > rps_max) rps_max = rps_of(H * 128, cs);
  if (rps_of(dim, cs / 2) > rps_max) rps_max = rps_of(dim, cs / 2);
  if (rps_of(hidden, cs) > rps_max) rps_max = rps_of(hidden, cs);
  const size_t smem = ds_smem_bytes(rps_max);
  if (smem > 113 * 1024) return Q40_E_SHAPE;
  cudaError_t e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  if (cs > 8) {
    e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
  }
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(DS_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = cs;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  // all clusters must be resident at once (they meet at grid barriers): ask how many fit
  cfg.gridDim = dim3(cs * 16, 1, 1);
  int ncl = 0;
  e = cudaOccupancyMaxActiveClusters(&ncl, decode_step_kernel, &cfg);
  if (e != cudaSuccess || ncl < 1) { (void)cudaGetLastError(); return Q40_E_UNSUPPORTED; }
  if (ncl > 16) ncl = 16;
  cfg.gridDim = dim3(cs * ncl, 1, 1);
  e = cudaMemsetAsync(bar, 0, sizeof(unsigned int), st);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemsetAsync(err, 0, sizeof(int), st);
  if (e != cudaSuccess) return (int)e;
  DsParams p{};
  p.layers = (const DsLayer*)layers;
  p.n_layers = n_layers; p.M = M; p.dim = dim; p.H = H; p.Hkv = Hkv; p.hidden = hidden; p.vocab = vocab;
  p.max_t = max_t; p.max_p = max_p; p.n_pos = n_pos; p.eps = eps;
  p.emb = (const __half*)emb; p.final_norm = (const __half*)final_norm;
  p.tokens = tokens; p.pos = pos; p.prefix_len = prefix_len;
  p.cos_tbl = (const __half*)cos_tbl; p.sin_tbl = (const __half*)sin_tbl;
  p.h = (__half*)h; p.qkv = (__half*)qkv; p.ao = (__half*)ao; p.g = (__half*)g; p.xn = (__half*)xn;
  p.ss_a = ss_a; p.ss_f = ss_f; p.bar = bar; p.err = err; p.rps_max = rps_max; p.trace = trace;
  e = cudaLaunchKernelEx(&cfg, decode_step_kernel, p);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}
