// One sampling step of the token tree search on the device: temperature, top-k, softmax, multinomial
// draws with replacement (counted per candidate), the sorted unique tokens with their counts, the
// branch bookkeeping (first unique token stays on the branch, the others fork new branches while there
// is room), terminal detection, and the copy of the forked branches' Q4_0 suffix cache rows.
//
// Reference: mcts.search, the body of its token loop (mcts.py:104-172), detectTerminal (mcts.py:14-28)
// and Attention.fork (hf_model_q40_kv_shared.py:282-297), where all of this is a Python loop over the
// live branches with a host synchronisation per branch (torch.multinomial, torch.unique).
//
// Conventions that make the result a function of the inputs alone (the reference leaves them to the
// library): candidates are ordered by (scaled logit descending, token id ascending); draw u in [0, 1)
// selects the first candidate j whose running probability sum exceeds u * (sum of all 32); sums run
// in candidate order in fp32.
#include "q40_common.cuh"

namespace q40 {
namespace tree {

constexpr int TOPK_MAX = 32;
constexpr int THREADS = 1024;     // one CTA per branch: 32 warps hide the latency of the division per element

// monotone map float -> uint32
__device__ __forceinline__ uint32_t fkey(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct SampleParams {
  const __half* logits;    // [B, ld]
  int64_t ld;
  int V, top_k;
  float temp;              // > 0: fixed temperature (scaled logits rounded to fp16, as fp16 / python float);
                           // <= 0: per-branch divisor slope * (count - 1) + 0.1 in fp32, scaled logits stay fp32
  float slope;             // (|temp| - 0.1) / (batch - 1), rounded to fp32 by the caller
  const int32_t* counts;   // [B] particles on each branch = number of draws
  const float* draws;      // [B, draws_ld] uniform numbers in [0, 1)
  int64_t draws_ld;
  int32_t* n_unique;       // [B]
  int32_t* uni_tok;        // [B, 32] ascending token ids
  int32_t* uni_cnt;        // [B, 32]
  float* probs_out;        // [B, 32] candidate probabilities in candidate order (optional)
  int32_t* cand_out;       // [B, 32] candidate token ids in candidate order (optional)
  int use_cache;           // 4 V bytes of dynamic shared memory hold the row's order keys
};

constexpr int EQ_LIST = 128;     // ties with the k-th largest value that are ranked from a list; more fall back to a scan

__global__ void __launch_bounds__(THREADS) sample_kernel(const SampleParams p) {
  __shared__ unsigned int hist[256];
  __shared__ uint32_t s_prefix, s_need;
  __shared__ uint32_t c_key[64];
  __shared__ int c_idx[64];
  __shared__ int c_n, c_eq_taken;
  __shared__ float s_val[TOPK_MAX], s_p[TOPK_MAX], s_cdf[TOPK_MAX];
  __shared__ int s_tok[TOPK_MAX];
  __shared__ unsigned int s_hist[TOPK_MAX];
  const int b = blockIdx.x, tid = threadIdx.x;
  const int k = min(p.top_k, min(p.V, TOPK_MAX));
  const int cnt = p.counts[b];
  const bool fixed = p.temp > 0.f;
  const float tdiv = fixed ? p.temp : __fadd_rn(__fmul_rn(p.slope, (float)(cnt - 1)), 0.1f);
  const __half* row = p.logits + (int64_t)b * p.ld;
  auto scaled = [&](int i) {
    const float x = __fdiv_rn(__half2float(row[i]), tdiv);
    return fixed ? __half2float(__float2half_rn(x)) : x;
  };
  // the order keys of the whole row, computed once (a division per element) and kept in shared memory when
  // the row fits (use_cache: 4 V bytes were granted at launch); the passes below read them from there
  extern __shared__ uint32_t key_cache[];
  const bool cached = p.use_cache != 0;
  if (cached) {
    for (int i = tid; i < p.V; i += THREADS) key_cache[i] = fkey(scaled(i));
    __syncthreads();
  }
  auto key_of = [&](int i) { return cached ? key_cache[i] : fkey(scaled(i)); };

  // ---- the k-th largest key by radix selection, most significant byte first ----
  if (tid == 0) { s_prefix = 0; s_need = (uint32_t)k; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    // fp16 logits of one row share a handful of leading bytes, so the lanes of a warp mostly hit the same bin:
    // one shared-memory atomic per distinct bin and warp (match_any) instead of one per element
    for (int base = 0; base < p.V; base += THREADS) {
      const int i = base + tid;
      uint32_t bin = 0xFFFFFFFFu;
      if (i < p.V) {
        const uint32_t key = key_of(i);
        if ((key & mask) == prefix) bin = (key >> shift) & 0xFF;
      }
      if (pass == 0) {
        const unsigned peers = __match_any_sync(0xffffffffu, bin);
        if (bin != 0xFFFFFFFFu && (tid & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], (unsigned)__popc(peers));
      } else if (bin != 0xFFFFFFFFu) {
        atomicAdd(&hist[bin], 1u);          // later passes: few keys left, spread over the bins
      }
    }
    __syncthreads();
    if (tid < 32) {
      // the highest bin b with count(bins > b) < need <= count(bins >= b): lane l owns bins 8l .. 8l + 7;
      // suffix sums across the lanes by shuffles instead of one thread walking 256 counters
      const uint32_t need0 = s_need;
      uint32_t mine[8], tot = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { mine[j] = hist[8 * tid + j]; tot += mine[j]; }
      uint32_t above = 0;                 // keys in the bins of higher lanes
      for (int l = 31; l > 0; --l) {
        const uint32_t v = __shfl_sync(0xffffffffu, tot, l);
        if (tid < l) above += v;
      }
      // the lane whose bins contain the threshold: above < need0 <= above + tot (lane 0 takes the rest)
      const bool has = (above < need0 && need0 <= above + tot) || (tid == 0 && need0 > above + tot);
      if (has) {
        uint32_t need = need0 - above;
        int j = 7;
        for (; j > 0; --j) {
          if (mine[j] >= need) break;
          need -= mine[j];
        }
        s_prefix = prefix | ((uint32_t)(8 * tid + j) << shift);
        s_need = need;                    // how many keys equal to the final threshold are taken
      }
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int eq_take = (int)s_need;
  // ---- collect: every key above the threshold, and the eq_take smallest token ids among the equal ones ----
  __shared__ int e_n, e_idx[EQ_LIST];
  if (tid == 0) { c_n = 0; c_eq_taken = 0; e_n = 0; }
  __syncthreads();
  for (int i = tid; i < p.V; i += THREADS) {
    const uint32_t key = key_of(i);
    if (key > thr) {
      const int s = atomicAdd(&c_n, 1);
      c_key[s] = key; c_idx[s] = i;
    } else if (key == thr) {
      const int s = atomicAdd(&e_n, 1);          // ties with the threshold are rare: list them
      if (s < EQ_LIST) e_idx[s] = i;
    }
  }
  __syncthreads();
  if (e_n <= EQ_LIST) {
    // the eq_take smallest token ids of the list (rank by counting smaller ids), no scan over the row
    if (tid < e_n) {
      const int mi = e_idx[tid];
      int rank = 0;
      for (int j = 0; j < e_n; ++j) rank += e_idx[j] < mi ? 1 : 0;
      if (rank < eq_take) {
        const int s = atomicAdd(&c_n, 1);
        c_key[s] = thr; c_idx[s] = mi;
      }
    }
    __syncthreads();
    if (tid == 0) c_eq_taken = eq_take;
    __syncthreads();
  }
  // equal keys in ascending token order: blocks of THREADS consecutive ids, ranked by ballot inside a block
  for (int base = 0; base < p.V && c_eq_taken < eq_take; base += THREADS) {
    const int i = base + tid;
    const bool eq = i < p.V && key_of(i) == thr;
    __shared__ int warp_cnt[THREADS / 32];
    const unsigned bal = __ballot_sync(0xffffffffu, eq);
    if ((tid & 31) == 0) warp_cnt[tid >> 5] = __popc(bal);
    __syncthreads();
    int before = c_eq_taken;
    for (int w = 0; w < (tid >> 5); ++w) before += warp_cnt[w];
    before += __popc(bal & ((1u << (tid & 31)) - 1));
    if (eq && before < eq_take) {
      const int s = atomicAdd(&c_n, 1);
      c_key[s] = thr; c_idx[s] = i;
    }
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < THREADS / 32; ++w) tot += warp_cnt[w];
      c_eq_taken = min(eq_take, c_eq_taken + tot);
    }
    __syncthreads();
  }
  // ---- order the k candidates: value descending, token id ascending (rank sort) ----
  if (tid < k) {
    const uint32_t mk = c_key[tid];
    const int mi = c_idx[tid];
    int rank = 0;
    for (int j = 0; j < k; ++j) rank += (c_key[j] > mk || (c_key[j] == mk && c_idx[j] < mi)) ? 1 : 0;
    s_val[rank] = scaled(mi);
    s_tok[rank] = mi;
  }
  if (tid < TOPK_MAX) s_hist[tid] = 0;
  __syncthreads();
  // ---- softmax over the candidates and its running sum, in candidate order ----
  if (tid == 0) {
    const float m = s_val[0];
    float s = 0.f;
    for (int j = 0; j < k; ++j) { s_p[j] = expf(s_val[j] - m); s += s_p[j]; }
    float c = 0.f;
    for (int j = 0; j < k; ++j) {
      float pj = s_p[j] / s;
      if (fixed) pj = __half2float(__float2half_rn(pj));      // the softmax of an fp16 tensor is fp16
      s_p[j] = pj;
      c += pj;
      s_cdf[j] = c;
    }
  }
  __syncthreads();
  // ---- draws ----
  const float total = s_cdf[k - 1];
  for (int i = tid; i < cnt; i += THREADS) {
    const float target = p.draws[(int64_t)b * p.draws_ld + i] * total;
    int j = 0;
    while (j < k - 1 && !(target < s_cdf[j])) ++j;
    atomicAdd(&s_hist[j], 1u);
  }
  __syncthreads();
  // ---- unique tokens in ascending order with their counts ----
  if (tid < k) {
    if (p.probs_out) p.probs_out[b * TOPK_MAX + tid] = s_p[tid];
    if (p.cand_out) p.cand_out[b * TOPK_MAX + tid] = s_tok[tid];
    if (s_hist[tid] > 0) {
      int rank = 0;
      for (int j = 0; j < k; ++j) rank += (s_hist[j] > 0 && s_tok[j] < s_tok[tid]) ? 1 : 0;
      p.uni_tok[b * TOPK_MAX + rank] = s_tok[tid];
      p.uni_cnt[b * TOPK_MAX + rank] = (int)s_hist[tid];
    }
  }
  if (tid == 0) {
    int n = 0;
    for (int j = 0; j < k; ++j) n += s_hist[j] > 0 ? 1 : 0;
    p.n_unique[b] = n;
  }
}

struct ForkParams {
  const int32_t* n_unique;   // [curr]
  const int32_t* uni_tok;    // [curr, 32]
  const int32_t* uni_cnt;
  int64_t* results;          // [batch, max_new]
  int max_new, step, batch;
  int32_t* counts;           // [batch] particles per branch (output_counts[1])
  int32_t* last_tok;         // [batch] (output_counts[0])
  uint8_t* alive;            // [batch] results_mask
  int32_t* results_len;      // [batch]
  int32_t* end_state;        // [batch] terminal-sequence matcher state
  const int64_t* term_seq;   // [term_len]
  int term_len;
  int64_t eos;
  int32_t* curr;             // [1] live branch count in, out
  int32_t* fork_src;         // [batch] for every branch created in this step: the branch it copies
  int32_t* n_forks;          // [1]
  int32_t* fork_base;        // [1] index of the first branch created in this step
  uint8_t* batch_stats;      // [max_new]
  int32_t* all_done;         // [1]
};

constexpr int FORK_MAX_BRANCHES = 1024;     // branches whose bookkeeping is staged in shared memory

__global__ void __launch_bounds__(THREADS) fork_kernel(const ForkParams p) {
  __shared__ int s_curr0, s_curr1, s_dead;
  __shared__ short s_nu[FORK_MAX_BRANCHES], s_start[FORK_MAX_BRANCHES], s_forks[FORK_MAX_BRANCHES];
  const int tid = threadIdx.x;
  // ---- who forks how often (mcts.py:127-154): the order of the branches decides who gets the room.  The
  // inputs are staged in shared memory by all threads, the sequential walk touches shared memory only, and
  // the results are written back by all threads (a single thread walking global memory costs ~1.5 us per
  // branch) ----
  const int curr_in = *p.curr;
  for (int i = tid; i < curr_in; i += THREADS) s_nu[i] = p.alive[i] ? (short)p.n_unique[i] : (short)0;
  __syncthreads();
  if (tid == 0) {
    int curr = curr_in;
    for (int i = 0; i < curr_in; ++i) {
      int forks = 0;
      if (s_nu[i] > 0) {
        forks = min((int)s_nu[i] - 1, p.batch - curr);
        if (forks < 0 || curr >= p.batch) forks = 0;
      }
      s_start[i] = (short)curr;
      s_forks[i] = (short)forks;
      curr += forks;
    }
    s_curr0 = curr_in; s_curr1 = curr; s_dead = 0;
    *p.curr = curr;
    *p.n_forks = curr - curr_in;
    *p.fork_base = curr_in;
    p.batch_stats[p.step] = (uint8_t)curr;
  }
  __syncthreads();
  for (int i = tid; i < curr_in; i += THREADS) {
    if (s_nu[i] == 0) continue;                 // not alive
    const int32_t tok0 = p.uni_tok[i * TOPK_MAX];
    p.last_tok[i] = tok0;
    p.counts[i] = p.uni_cnt[i * TOPK_MAX];
    p.results[(int64_t)i * p.max_new + p.step] = tok0;
    const int start = s_start[i], forks = s_forks[i];
    for (int j = 0; j < forks; ++j) {
      p.fork_src[start + j] = i;
      p.last_tok[start + j] = p.uni_tok[i * TOPK_MAX + 1 + j];
      p.counts[start + j] = p.uni_cnt[i * TOPK_MAX + 1 + j];
    }
  }
  __threadfence_block();
  __syncthreads();
  const int curr0 = s_curr0, curr1 = s_curr1;
  // ---- the new branches inherit the token history of their origin, then take their own token ----
  for (int nb = curr0; nb < curr1; ++nb) {
    const int src = p.fork_src[nb];
    for (int t = tid; t < p.step; t += THREADS)
      p.results[(int64_t)nb * p.max_new + t] = p.results[(int64_t)src * p.max_new + t];
    // (the row's own mask, length and terminal-matcher state are kept, as in the reference, where only
    // `results` and the counts are copied: rows that are not live yet count steps like live ones)
    if (tid == 0) p.results[(int64_t)nb * p.max_new + p.step] = p.last_tok[nb];
  }
  __syncthreads();
  // ---- per branch: mask the token of finished branches, terminal detection, lengths (mcts.py:158-165) ----
  for (int i = tid; i < p.batch; i += THREADS) {
    const bool alive = p.alive[i] != 0;
    int64_t tok = p.results[(int64_t)i * p.max_new + p.step];
    if (!alive) { tok = 0; p.results[(int64_t)i * p.max_new + p.step] = 0; }
    int st = p.end_state[i];
    const int m = (st >= 0 && st < p.term_len && p.term_seq[st] == tok) ? 1 : 0;
    st = (st + m) * m;
    const bool end = (st == p.term_len) || (tok == p.eos);
    st = end ? 0 : st;
    p.end_state[i] = st;
    p.results_len[i] += alive ? 1 : 0;
    p.alive[i] = (alive && !end) ? 1 : 0;
    if (!(alive && !end)) atomicAdd(&s_dead, 1);
  }
  __syncthreads();
  // the reference stops when the number of finished rows equals the live branch count (mcts.py:174)
  if (tid == 0) *p.all_done = (s_dead == curr1) ? 1 : 0;
}

// Copy the Q4_0 suffix rows [0, len) of branch fork_src[nb] to branch nb for every layer, for the branches
// fork_base .. fork_base + n_forks - 1 created by the step.  Rows are `row_bytes` long, a branch holds
// `rows_per_branch` of them, a layer `branches` branches.
__global__ void __launch_bounds__(256)
fork_copy_kernel(uint8_t* cache, int64_t layer_stride, int64_t branch_stride, int64_t copy_bytes, int n_layers,
                 const int32_t* fork_src, const int32_t* n_forks, const int32_t* fork_base, int max_forks) {
  const int f = blockIdx.y, layer = blockIdx.z;
  if (f >= *n_forks || f >= max_forks) return;
  const int dst_b = *fork_base + f, src_b = fork_src[dst_b];
  const uint4* s = reinterpret_cast<const uint4*>(cache + layer * layer_stride + src_b * branch_stride);
  uint4* d = reinterpret_cast<uint4*>(cache + layer * layer_stride + dst_b * branch_stride);
  const int64_t n16 = copy_bytes / 16;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x)
    d[i] = s[i];
}

}  // namespace tree
}  // namespace q40

// Sampling of one step for B live branches.  See include/q40b200.h.
extern "C" int q40_tree_sample(const void* logits, int64_t ld, int B, int V, int top_k, float temp, float slope,
                               const int32_t* counts, const float* draws, int64_t draws_ld, int32_t* n_unique,
                               int32_t* uni_tok, int32_t* uni_cnt, float* probs_out, int32_t* cand_out, void* stream) {
  using namespace q40::tree;
  if (!logits || !counts || !draws || !n_unique || !uni_tok || !uni_cnt) return Q40_E_NULL;
  if (B < 0 || V < 1 || top_k < 1 || ld < V) return Q40_E_SHAPE;
  if (B == 0) return Q40_OK;
  SampleParams p{};
  p.logits = (const __half*)logits; p.ld = ld; p.V = V; p.top_k = top_k; p.temp = temp; p.slope = slope;
  p.counts = counts; p.draws = draws; p.draws_ld = draws_ld; p.n_unique = n_unique; p.uni_tok = uni_tok;
  p.uni_cnt = uni_cnt; p.probs_out = probs_out; p.cand_out = cand_out;
  // the row's order keys in dynamic shared memory when they fit beside the static arrays
  size_t smem = 0;
  if ((size_t)V * 4 <= 200 * 1024) {
    smem = (size_t)V * 4;
    if (smem > 40 * 1024 &&
        cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      (void)cudaGetLastError();
      smem = 0;
    }
  }
  p.use_cache = smem ? 1 : 0;
  sample_kernel<<<B, THREADS, smem, (cudaStream_t)stream>>>(p);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}

// Branch bookkeeping of one step (one CTA; the order of the branches is part of the semantics).
extern "C" int q40_tree_fork(const int32_t* n_unique, const int32_t* uni_tok, const int32_t* uni_cnt, int64_t* results,
                             int max_new, int step, int batch, int32_t* counts, int32_t* last_tok, uint8_t* alive,
                             int32_t* results_len, int32_t* end_state, const int64_t* term_seq, int term_len,
                             int64_t eos, int32_t* curr, int32_t* fork_src, int32_t* n_forks, int32_t* fork_base,
                             uint8_t* batch_stats, int32_t* all_done, void* stream) {
  using namespace q40::tree;
  if (!n_unique || !uni_tok || !uni_cnt || !results || !counts || !last_tok || !alive || !results_len || !end_state ||
      !curr || !fork_src || !n_forks || !fork_base || !batch_stats || !all_done || (term_len > 0 && !term_seq))
    return Q40_E_NULL;
  if (batch < 1 || max_new < 1 || step < 0 || step >= max_new || term_len < 0) return Q40_E_SHAPE;
  if (batch > FORK_MAX_BRANCHES) return Q40_E_UNSUPPORTED;
  ForkParams p{};
  p.n_unique = n_unique; p.uni_tok = uni_tok; p.uni_cnt = uni_cnt; p.results = results; p.max_new = max_new;
  p.step = step; p.batch = batch; p.counts = counts; p.last_tok = last_tok; p.alive = alive;
  p.results_len = results_len; p.end_state = end_state; p.term_seq = term_seq; p.term_len = term_len; p.eos = eos;
  p.curr = curr; p.fork_src = fork_src; p.n_forks = n_forks; p.fork_base = fork_base; p.batch_stats = batch_stats;
  p.all_done = all_done;
  fork_kernel<<<1, THREADS, 0, (cudaStream_t)stream>>>(p);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}

// Suffix-cache copy for the branches the step created: `cache` is one of the model's cache tensors
// [n_layers, branches, ...]; copy_bytes (a multiple of 16) of every new branch are copied from its origin.
extern "C" int q40_tree_fork_copy(void* cache, int64_t layer_stride, int64_t branch_stride, int64_t copy_bytes,
                                  int n_layers, const int32_t* fork_src, const int32_t* n_forks,
                                  const int32_t* fork_base, int max_forks, void* stream) {
  using namespace q40::tree;
  if (!cache || !fork_src || !n_forks || !fork_base) return Q40_E_NULL;
  if (copy_bytes < 0 || copy_bytes % 16 != 0 || n_layers < 1 || max_forks < 0) return Q40_E_SHAPE;
  if (!q40_aligned(cache, 16) || layer_stride % 16 != 0 || branch_stride % 16 != 0) return Q40_E_ALIGN;
  if (copy_bytes == 0 || max_forks == 0) return Q40_OK;
  int gx = (int)((copy_bytes / 16 + 255) / 256);
  if (gx > 64) gx = 64;
  if (gx < 1) gx = 1;
  fork_copy_kernel<<<dim3(gx, max_forks, n_layers), 256, 0, (cudaStream_t)stream>>>(
      (uint8_t*)cache, layer_stride, branch_stride, copy_bytes, n_layers, fork_src, n_forks, fork_base, max_forks);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}
