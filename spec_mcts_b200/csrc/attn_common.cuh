// Declarations shared by the attention kernels.
#pragma once
#include "q40_common.cuh"

namespace q40 {

constexpr int ATTN_D = 128;  // head dim of every supported model (CodeLlama 7B/70B)

inline float attn_scale_log2(int D) { return (1.0f / sqrtf((float)D)) * 1.4426950408889634f; }

struct BranchArgs {
  const __half* q;        // branch b, head h at q + b*q_stride + h*D
  int64_t q_stride;
  const __half* k;        // contiguous: [B,Hkv,L,D]; paged: pool [Hkv,P,D]
  const __half* v;
  __half* o;              // [B, H, D]
  const void* tbl;        // page table or nullptr
  int64_t tbl_stride;
  const int32_t* seq_lens;  // per-branch length or nullptr (= L)
  int L, H, Hkv, P, page_size;
  // optional partial results of a prefix pass over rows (b, h), log2 domain, un-normalised
  const float* pm;        // [nsp][B*H]
  const float* pl;        // [nsp][B*H]
  const float* po;        // [nsp][B*H][128]
  int nsp;
  float scale_log2;       // 1/sqrt(D) * log2(e)
  // Q4_0 suffix cache (mode 3): packed rows [B, max_t, Hkv, 64] + scales [B, max_t, Hkv, 2];
  // the branch's suffix length is pos[b] - prefix_len[0] (device values)
  const int8_t* kq;
  const __half* ksc;
  const int8_t* vq;
  const __half* vsc;
  const int32_t* pos;
  const int32_t* prefix_len;
  int max_t;
  // optional un-quantised K/V of the token being decoded, [B, Hkv*D] rows of stride cur_stride
  const __half* cur_k;
  const __half* cur_v;
  int64_t cur_stride;
};

// defined in attn_branch.cu; mode 0 contiguous, 1 paged/int16 ids, 2 paged/int32 ids, 3 Q4_0 cache
int launch_branch(const BranchArgs& a, int mode, int B, cudaStream_t st);

}  // namespace q40
