/*
 * q40b200 — C ABI of the B200 (sm_100a) kernels for the Q4_0 decode hot path.
 *
 * Conventions for every entry point
 *   - all data pointers are DEVICE pointers owned by the caller; nothing is allocated,
 *     freed or retained across the boundary;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = legacy default
 *     stream) and the call returns without synchronising the host;
 *   - return value: 0 = enqueued, negative = argument error (Q40_E_*), positive = the
 *     cudaError_t of a failed launch;  q40_strerror() turns either into text;
 *   - "half" means IEEE binary16 stored as 2 bytes; Q4_0 here is the reference's format:
 *     signed 4-bit codes in [-8,7], one fp16 scale per `group` consecutive elements
 *     (group = 64 is the reference's fixed choice, 32 is also accepted), two groups
 *     (2j, 2j+1) packed into one row of `group` bytes: byte i = code[2j][i] << 4 |
 *     code[2j+1][i] & 0xF.
 *
 * Each declaration cites the reference interface it stands in for, as file:line of the
 * reference project (hongyihuang/spec-mcts).
 */
#ifndef Q40B200_H
#define Q40B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q40_OK 0
#define Q40_E_NULL (-1)      /* a required pointer is NULL                         */
#define Q40_E_SHAPE (-2)     /* a size violates a divisibility or range rule       */
#define Q40_E_ALIGN (-3)     /* a pointer or stride is not aligned as documented   */
#define Q40_E_WORKSPACE (-4) /* workspace missing or smaller than *_workspace_bytes */
#define Q40_E_UNSUPPORTED (-5)

const char* q40_strerror(int status);
/* Library/ABI version, bumped when a signature changes. */
int q40_abi_version(void);

/* ---- Q4_0 pack / unpack ------------------------------------------------------------ */

/* w[n] fp16 (row-major, any logical shape) -> q[n/2] bytes viewed as [n/(2*group), group],
 * s[n/group] fp16.  Bit-exact with quantize_q40 for fp16 input: scale = fp16(absmax/7),
 * code = int8(rint(fp16(w/scale))), non-finite quotient -> 0.
 * n % (2*group) == 0; w, q 16-byte aligned.
 * Replaces: quantize_q40 (triton_kernels.py:12-41) and, with correct rounding,
 * triton_q_int40 (triton_kernels.py:109-152). */
int q40_quantize(const void* w, void* q, void* s, int64_t n, int group, void* stream);

/* Same packer applied to n_rows separate rows of row_len fp16 elements each; row r is
 * read at w + r*w_row_stride (elements) and written at q + r*q_row_stride (bytes) and
 * s + r*s_row_stride (elements), so the new token rows of a strided KV cache can be
 * quantised in place.  row_len % (2*group) == 0, strides keep 16-byte alignment.
 * Replaces the intent of triton_q_int40_sliced (triton_kernels.py:154-200) and the
 * per-step re-quantisation in Attention.forward (hf_model_q40_kv_shared.py:365-371). */
int q40_quantize_rows(const void* w, int64_t w_row_stride, void* q, int64_t q_row_stride,
                      void* s, int64_t s_row_stride, int64_t n_rows, int row_len, int group,
                      void* stream);

/* q, s -> out[n] fp16, out = fp16(code * scale).  Bit-exact with dequantize_q40.
 * Replaces: dequantize_q40 (triton_kernels.py:43-56), triton_deq_int40 (:58-107). */
int q40_dequantize(const void* q, const void* s, void* out, int64_t n, int group, void* stream);

/* ---- fused dequant-matmul ------------------------------------------------------------ */

/* Workspace (bytes) that q40_gemm_kn / q40_gemm_nk need for this problem; the buffer
 * must be zero-filled once when it is created (the kernels leave it zeroed) and must not
 * be shared by calls that can overlap on the GPU. */
size_t q40_gemm_workspace_bytes(int M, int N, int K);

/* C[M,N] = A[M,K] @ deq(B)[K,N], B quantised from a row-major [K,N] matrix (groups along
 * N; the on-disk orientation): bw viewed as [K, N/2] bytes, bs as [K, N/group] fp16.
 * fp16 in, fp32 accumulate, fp16 out.  lda/ldc in elements.  N % (2*group) == 0.
 * Up to 16 rows run a split-K kernel that sums its partials through the workspace (any shape);
 * for group 64, N % 128 == 0 and K % 16 == 0 the cluster-reduced launch q40_gemv_fused (mode 0, one
 * matrix) computes the same product without a workspace and 1.2-2x faster, and is what the Python
 * matmul_q40 of this repository calls for such shapes.
 * Replaces: matmul_q40 (triton_kernels.py:357-500), called by LinearQ4_0.forward
 * (hf_model_q40_kv_shared.py:228-236). */
int q40_gemm_kn(const void* a, int64_t lda, const void* bw, const void* bs, void* c,
                int64_t ldc, int M, int N, int K, int group, void* workspace,
                size_t workspace_bytes, void* stream);

/* The tensor-core form q40_gemm_kn selects for M > 16 (group 64, K % 64 == 0, N % 128 == 0, even ldc, lda % 8 == 0):
 * tcgen05.mma with the 128 output features of a packed block as the MMA M dimension and the
 * batch as N, accumulator in tensor memory, split-K over a thread-block cluster.  `err` is a
 * device int (zeroed by the caller) that the kernel sets to 1 if one of its bounded waits
 * expired, in which case the output is undefined; through q40_gemm_kn it is the last int of the
 * first 4096 bytes of the workspace.
 * Replaces: matmul_q40 (triton_kernels.py:357-500) at batch 100 and for the prompt pass. */
int q40_gemm_kn_tc(const void* a, int64_t lda, const void* bw, const void* bs, void* c, int64_t ldc,
                   int M, int N, int K, int* err, void* stream);

/* q40_gemm_kn_tc for up to three weight matrices that share the activations and K (wq, wk, wv of a
 * layer) in one launch: the feature tiles of all matrices form one grid, so that small matrices
 * do not pay a launch each.  bw/bs/c/ldc/n_cols are host arrays of nmat entries read during the
 * call; every n_cols[i] % 128 == 0 and ldc[i] even.  use_pdl != 0 launches with programmatic stream
 * serialization: the first weight blocks are requested while the previous launch on the stream
 * drains, so that launch must not be the one that writes the weights.  No counterpart in the reference (its model
 * issues one matmul_q40 per projection, hf_model_q40_kv_shared.py:313-315). */
int q40_gemm_kn_tc_multi(int nmat, const void* a, int64_t lda, const void* const* bw,
                         const void* const* bs, void* const* c, const int64_t* ldc, const int* n_cols,
                         int M, int K, int* err, int use_pdl, void* stream);

/* The same operation on TILED copies of the weights (q40_relayout_tiled; N_i % 256 == 0, K % 64 == 0),
 * so that a caller that already holds tiled copies for the narrow decode path needs no second format:
 * the weight stream of a CTA is one contiguous run fetched by 1-D bulk copies, the activations arrive by
 * tiled TMA copies (a tensor map over `a` is encoded per call), both into a 3..6 stage ring; A operand
 * value fp16(code * scale) as in the reference (triton_kernels.py:444-445), written to tensor memory.  Batches
 * above 128 rows run as consecutive launches of 128 rows.  Results are bit-identical from run to run.  Same
 * `err` and `use_pdl` rules as q40_gemm_kn_tc_multi; Q40_E_UNSUPPORTED when the driver offers no tensor-map
 * encoder. */
int q40_gemm_tiled_tc_multi(int nmat, const void* a, int64_t lda, const void* const* bw_tiled, void* const* c,
                            const int64_t* ldc, const int* n_cols, int M, int K, int* err, int use_pdl,
                            void* stream);

/* q40_gemm_kn without a caller-provided workspace, for hosts that cannot allocate device
 * memory themselves (all HBM already handed to their own planner, or a plug-in that only
 * receives input and output buffers).  The split-K scratch is a fixed array inside the library
 * (q40_gemm_kn_static_max_workspace() bytes, 8 MiB, held on every GPU that loads the library);
 * a problem whose q40_gemm_workspace_bytes() exceeds it returns Q40_E_WORKSPACE.  The first
 * call on a device looks up the array's device address and should precede any stream
 * capture.  Calls share the array, so calls that overlap on the GPU race; calls on one
 * stream are safe (host threads may make the first call on a device concurrently).  The array of the
 * CURRENT device is used: make the device of `stream` current before the call.  No allocation is made
 * by this entry point or anything it calls.
 * This entry point has no counterpart in the reference. */
int q40_gemm_kn_static(const void* a, int64_t lda, const void* bw, const void* bs, void* c,
                       int64_t ldc, int M, int N, int K, int group, void* stream);
size_t q40_gemm_kn_static_max_workspace(void);
/* Above 16 rows q40_gemm_kn_static runs the tcgen05 kernel, whose bounded waits report expiry in a
 * word inside the library's array: this copies that word to *host_out (0 = every call since the last
 * clear completed its waits; non-zero = at least one output is undefined), optionally clears it, and
 * waits for `stream`.  It is this library's status read-back for the entry points that own no
 * caller-visible workspace; with a caller-owned workspace the same word is the int at byte 4092 of the
 * workspace (q40_gemm_kn) or the `err` argument (q40_gemm_kn_tc), and q40_gemv_stream reports in the
 * first int of its workspace.  No counterpart in the reference. */
int q40_gemm_kn_static_error(int* host_out, int clear, void* stream);

/* Y[M,N] = X[M,K] @ deq(W)[N,K]^T, W quantised from a row-major [N,K] matrix (groups
 * along K): wq viewed as [N*K/(2*group), group], ws as [N*K/group].  K % (2*group) == 0.
 * Replaces: dequantize_q40 + F.linear in LinearQ4_0.forward (quantize.py:235-246,
 * hf_model_q40.py:222-233). */
int q40_gemm_nk(const void* x, int64_t ldx, const void* wq, const void* ws, void* y,
                int64_t ldy, int M, int N, int K, int group, void* workspace,
                size_t workspace_bytes, void* stream);

/* Decode-step form of q40_gemm_kn (group 64, 1 <= M <= 16, K % 16 == 0, every N % 128 == 0):
 * one launch computes out[i] = X @ deq(B_i) for nmat (1..3) matrices that share the
 * activations, with the element-wise neighbours of the matmul folded in.  mode:
 *   0  X = a                                   out[i] = fp16(acc)
 *   1  X = RMSNorm(a) (a = residual stream, weight norm_w, eps; the row sums of squares are the
 *      sums of ss_in[m][0..ss_in_count), as written by a mode-2 launch)      out[i] = fp16(acc)
 *   2  nmat == 1: out = fp16(h_in + fp16(acc)) (h_in may alias out), and
 *      ss_out[m][0..ss_out_count) receives partial sums of out^2 (ss_out_count must equal
 *      q40_gemv_fused_ss_count(N, K, max_cluster))
 *   3  nmat == 2 (w1, w3), prologue as mode 1:  out[0] = fp16(fp16(silu(fp16(acc1))) * fp16(acc3))
 * Split-K partials are summed inside a thread-block cluster (max_cluster = 8, or 16 where the
 * device allows non-portable cluster sizes); no workspace.  With use_pdl != 0 the kernel is
 * launched with programmatic stream serialization: it prefetches weights before waiting for
 * the preceding kernel on the stream, so the preceding kernel must not be one whose output
 * buffers this launch's *weights* alias (they never do).
 * Replaces: LinearQ4_0.forward chains of TransformerBlock.forward
 * (hf_model_q40_kv_shared.py:228-236, 313, 409, 431-436, 456-467) together with RMSNorm
 * (:123-134), the residual adds (:463-466) and F.silu(w1 x) * w3 x (:434). */
int q40_gemv_fused(int mode, int nmat, const void* const* bw, const void* const* bs, void* const* out,
                   const int* n_cols, int64_t ldc, const void* a, int64_t lda, int M, int K,
                   const void* norm_w, const float* ss_in, int ss_in_count, float eps, const void* h_in,
                   int64_t ldh, float* ss_out, int ss_out_count, int max_cluster, int use_pdl,
                   void* stream);
int q40_gemv_fused_ss_count(int N, int K, int max_cluster);

/* Tiled copy of a packed [K, N] matrix for q40_gemv_tiled (N % 256 == 0, K % 16 == 0): a one-time
 * device pass that rearranges codes and scales (none is changed) so that the decode matmul needs
 * about one instruction per weight.  `out` has q40_tiled_bytes(N, K) bytes (= packed + scales).
 * No counterpart in the reference (its Triton kernel reads the checkpoint layout directly). */
size_t q40_tiled_bytes(int N, int K);
int q40_relayout_tiled(const void* bw, const void* bs, void* out, int N, int K, void* stream);

/* q40_gemv_fused on tiled copies (same modes, arguments and results up to rounding: the scale is
 * applied to the activations, fp16(scale*x), instead of to the weight; the RMSNorm of modes 1 and 3
 * keeps the reference's rounding points; 1 <= M <= 16; every N % 256 == 0).  bw[i] are the tiled
 * streams; bs is ignored and may be NULL. */
int q40_gemv_tiled(int mode, int nmat, const void* const* bw, const void* const* bs, void* const* out,
                   const int* n_cols, int64_t ldc, const void* a, int64_t lda, int M, int K,
                   const void* norm_w, const float* ss_in, int ss_in_count, float eps, const void* h_in,
                   int64_t ldh, float* ss_out, int ss_out_count, int max_cluster, int use_pdl,
                   void* stream);
int q40_gemv_tiled_ss_count(int N, int K, int max_cluster);

/* The decode matmul as one byte-balanced wave (stream-K): the same modes and results as
 * q40_gemv_tiled on the same tiled copies, except that modes 1 and 3 keep the reference's RMSNorm
 * rounding points (fp16(fp16(float(a) / rms) * norm_w) is the operand).  One CTA per SM at most, each
 * streaming an equal contiguous share of the launch's weight bytes through a shared-memory ring filled
 * by 1-D bulk copies; the partial sums of a 256-column span meet in `workspace` and the CTA that
 * arrives last adds them in a fixed order, so results are reproducible run to run.
 * workspace: q40_gemv_stream_workspace_bytes(M, sum of n_cols, K) bytes, 16-byte aligned, zero-filled
 * once by the caller (the kernels leave its counters zeroed); launches that share it must be ordered on
 * one stream.  Its first int is a status word: non-zero after a launch means a bounded wait inside the
 * kernel expired and the outputs of that launch are undefined.  ss_out_count must be
 * q40_gemv_stream_ss_count(N) = N / 256.  smem_budget: shared memory per CTA in bytes (0 = 100 KiB up to
 * 4 rows, which lets the CTAs of two consecutive launches share an SM, 200 KiB above).  1 <= M <= 16, every N % 256 == 0.
 * Replaces: the same reference lines as q40_gemv_fused. */
size_t q40_gemv_stream_workspace_bytes(int M, int total_cols, int K);
int q40_gemv_stream(int mode, int nmat, const void* const* bw_tiled, void* const* out, const int* n_cols,
                    int64_t ldc, const void* a, int64_t lda, int M, int K, const void* norm_w,
                    const float* ss_in, int ss_in_count, float eps, const void* h_in, int64_t ldh,
                    float* ss_out, int ss_out_count, void* workspace, size_t workspace_bytes,
                    int smem_budget, int use_pdl, void* stream);
int q40_gemv_stream_ss_count(int N);

/* Tail of a decode step in one launch: logits[M, V] = fp16(RMSNorm(h; norm_w, eps) @ w^T) for the fp16
 * lm_head w [V, K] (row-major), 1 <= M <= 16, K % 128 == 0.  ss_in [M, ss_count] are partial sums of
 * squares of the rows of h as a mode-2 matmul launch leaves them (NULL: computed here).  If tok_out is
 * given, the arg-max of every row of the fp16 logits (ties: the smaller index) is written to tok_out[m]
 * (int64) and pos[m] (int32, may be NULL) is advanced by one — greedy decoding without the host.
 * `scratch`: q40_lm_head_scratch_bytes() bytes, 8-byte aligned, zero-filled once (left zeroed);
 * required with tok_out.
 * Replaces: self.norm + self.output of Transformer.forward (hf_model_q40_kv_shared.py:508-510) and the
 * arg-max a greedy harness applies to its result. */
int q40_lm_head(const void* h, int64_t ldh, const float* ss_in, int ss_count, const void* norm_w, float eps,
                const void* w, int V, int K, void* logits, int64_t ldl, int M, int64_t* tok_out,
                int32_t* pos, void* scratch, int use_pdl, void* stream);
size_t q40_lm_head_scratch_bytes(void);

/* ---- token tree search: one sampling step on the device ----------------------------------- */

/* For each of B live branches: scaled logits (temp > 0: fp16(logit / temp), as the reference's
 * fp16 tensor / python float; temp <= 0: logit / (slope * (counts[b] - 1) + 0.1) in fp32, the
 * reference's per-branch temperature by particle count, slope = (|temp| - 0.1) / (batch - 1)), the
 * top_k (<= 32) candidates ordered by (value descending, token id ascending), their softmax (rounded to
 * fp16 when temp > 0), counts[b] draws with replacement — draws[b, i] in [0, 1) selects the first
 * candidate whose running fp32 probability sum exceeds draws[b, i] times the total — and the distinct
 * sampled tokens in ascending order with their multiplicities: n_unique[b], uni_tok[b, 0..], uni_cnt[b, 0..]
 * (rows of 32).  probs_out / cand_out (rows of 32, may be NULL) receive the candidate list.
 * Replaces: mcts.search's per-branch temperature / torch.topk / F.softmax / torch.multinomial /
 * torch.unique sequence (mcts.py:110-131). */
int q40_tree_sample(const void* logits, int64_t ld, int B, int V, int top_k, float temp, float slope,
                    const int32_t* counts, const float* draws, int64_t draws_ld, int32_t* n_unique,
                    int32_t* uni_tok, int32_t* uni_cnt, float* probs_out, int32_t* cand_out, void* stream);

/* Branch bookkeeping of token `step` for the *curr live branches, in branch order: the first distinct
 * token stays on its branch, each further one creates a branch while fewer than `batch` exist (token
 * history copied from the origin, counts and last token set, fork_src[new] = origin); then, for all
 * `batch` rows, tokens of finished rows are zeroed, the terminal-sequence matcher and the end-of-
 * sequence test run, lengths and the alive mask are updated, batch_stats[step] = live branches and
 * *all_done = (finished rows == live branches).  *n_forks / *fork_base describe the branches created.
 * Replaces: mcts.search's fork / bookkeeping block and detectTerminal (mcts.py:133-176, 14-28). */
int q40_tree_fork(const int32_t* n_unique, const int32_t* uni_tok, const int32_t* uni_cnt, int64_t* results,
                  int max_new, int step, int batch, int32_t* counts, int32_t* last_tok, uint8_t* alive,
                  int32_t* results_len, int32_t* end_state, const int64_t* term_seq, int term_len,
                  int64_t eos, int32_t* curr, int32_t* fork_src, int32_t* n_forks, int32_t* fork_base,
                  uint8_t* batch_stats, int32_t* all_done, void* stream);

/* For the *n_forks branches created by q40_tree_fork: copy copy_bytes (a multiple of 16) of branch
 * fork_src[b] to branch b in every layer of a cache tensor [n_layers, branches, ...] with the given
 * byte strides.  max_forks bounds the grid (the count itself stays on the device).
 * Replaces: Attention.fork / Transformer.fork (hf_model_q40_kv_shared.py:282-297, 512-516). */
int q40_tree_fork_copy(void* cache, int64_t layer_stride, int64_t branch_stride, int64_t copy_bytes, int n_layers,
                       const int32_t* fork_src, const int32_t* n_forks, const int32_t* fork_base, int max_forks,
                       void* stream);

/* ---- decode attention (one query token per branch) ---------------------------------- */

/* q[B,H,D], k/v[B,Hkv,L,D] contiguous fp16 -> o[B,H,D]; scale 1/sqrt(D); D == 128;
 * H % Hkv == 0.  fp32 online softmax.
 * Replaces: flash_attn (triton_kernels.py:559-647). */
int q40_attn_decode(const void* q, const void* k, const void* v, void* o, int B, int L, int H,
                    int Hkv, int D, void* stream);

/* Paged decode attention.  kpool/vpool [Hkv, P, D] fp16 hold P token slots per kv head.
 * page_tbl[B, tbl_stride] (idx_bytes = 2: int16, 4: int32) lists page ids; token t of
 * branch b is slot page_tbl[b][t / page_size] * page_size + t % page_size.  seq_lens[B]
 * int32 gives each branch's length, or NULL = every branch has length Lmax.
 * page_size = 1 with an int16 table is the reference's layout.
 * Replaces: page_flash_attn (triton_kernels.py:700-789). */
int q40_attn_paged(const void* page_tbl, int idx_bytes, int64_t tbl_stride, const int32_t* seq_lens,
                   const void* q, const void* kpool, const void* vpool, void* o, int P, int B,
                   int Lmax, int H, int Hkv, int D, int page_size, void* stream);

/* Bytes of fp32 scratch q40_attn_shared_prefix needs (partial max / sum / output of each
 * prefix split).  No initialisation required. */
size_t q40_attn_shared_prefix_workspace_bytes(int B, int H, int D, int prefix_len);

/* Shared-prefix decode attention: all B branches attend to the same prefix (key t of kv
 * head h at prefix_k + t*prefix_key_stride + h*prefix_head_stride, in elements; strides are
 * multiples of 8; the prefix is read once per CTA and applied to every branch)
 * and then to their private paged suffix (arguments as q40_attn_paged, lengths = suffix
 * lengths, may be 0).  Result is attention over cat(prefix, suffix_b).
 * Replaces: chunk_attn (triton_kernels.py:1150-1231) and the materialised
 * cat(prompt.expand(B), suffix) + SDPA in Attention.forward
 * (hf_model_q40_kv_shared.py:375-376, 405). */
int q40_attn_shared_prefix(const void* q, const void* prefix_k, const void* prefix_v,
                           int prefix_len, int64_t prefix_key_stride, int64_t prefix_head_stride,
                           const void* page_tbl, int idx_bytes,
                           int64_t tbl_stride, const int32_t* seq_lens, const void* kpool,
                           const void* vpool, void* o, int P, int B, int Lmax, int H, int Hkv,
                           int D, int page_size, void* workspace, size_t workspace_bytes,
                           void* stream);

/* One decode step of the KV-shared model's attention, replayable from a CUDA graph because
 * every length is read from device memory (branch b's queries start at q + b*q_stride
 * elements): all B branches attend to the shared fp16 prompt
 * cache (first *prefix_len_dev <= max_prefix_len keys), then to their own Q4_0 suffix cache
 * (packed rows cache_kq/cache_vq [maxB, max_t, Hkv, 64] bytes with scales cache_ks/cache_vs
 * [maxB, max_t, Hkv, 2] fp16; branch b holds pos_dev[b] - *prefix_len_dev tokens), and
 * finally, if cur_k/cur_v are given, to the un-quantised K/V of the token being decoded
 * (rows of cur_stride elements, [B, Hkv*D]).  Workspace as q40_attn_shared_prefix sized for
 * max_prefix_len.
 * Replaces: the decode branch of Attention.forward (hf_model_q40_kv_shared.py:330-405):
 * dequantise the whole suffix, overwrite the new position, cat with the expanded prompt, SDPA. */
int q40_attn_tree_decode(const void* q, int64_t q_stride, const void* prefix_k, const void* prefix_v,
                         int max_prefix_len, const int32_t* prefix_len_dev,
                         int64_t prefix_key_stride, int64_t prefix_head_stride,
                         const void* cache_kq, const void* cache_ks, const void* cache_vq,
                         const void* cache_vs, int max_t, const int32_t* pos_dev, const void* cur_k,
                         const void* cur_v, int64_t cur_stride, void* o, int B, int H, int Hkv, int D,
                         void* workspace, size_t workspace_bytes, void* stream);

/* q40_rope_kv_append + q40_attn_tree_decode as one launch for small widths (a cluster of 8 CTAs
 * per (branch, head) splits the keys; no workspace): qkv [B, W] holds the new token's q heads, k
 * heads and v heads (un-rotated, W >= (H + 2 Hkv) * 128); the rotated key and the value are
 * appended to the Q4_0 suffix cache at slot (b, pos[b] - *prefix_len) and the attention output is
 * written to ao [B, H*128].  Caches and tables as in the two calls it replaces.  use_pdl != 0
 * launches with programmatic stream serialization: cached keys are fetched while the previous
 * launch (the one that writes qkv) drains; pos, prefix_len and cache rows below pos must then
 * have been complete before that previous launch started.
 * Replaces: the decode branch of Attention.forward (hf_model_q40_kv_shared.py:313-317, 330-405). */
int q40_attn_tree_fused(void* qkv, int64_t W, const void* pk, const void* pv, void* kq, void* ks, void* vq,
                        void* vs, const int32_t* pos, const int32_t* prefix_len, const void* cos_tbl,
                        const void* sin_tbl, int n_pos, void* ao, int B, int H, int Hkv, int D, int max_t,
                        int max_p, int use_pdl, void* stream);

/* Rotary embedding of the new token's q [B, H*D] and k [B, Hkv*D] in place (position
 * pos_dev[b], tables cos/sin [n_pos, D/2] fp16) and Q4_0 append of the rotated k and of v to
 * the suffix cache at slot (b, pos_dev[b] - *prefix_len_dev); k and v stay un-quantised in
 * their buffers for this step's attention.  Strides in elements.  D == 128.
 * Replaces: apply_rotary_emb (hf_model_q40_kv_shared.py:166-203, 317) and the quantise-and-
 * store of the new rows (:365-371). */
int q40_rope_kv_append(void* q, int64_t q_stride, void* k, int64_t k_stride, const void* v,
                       int64_t v_stride, const int32_t* pos_dev, const int32_t* prefix_len_dev,
                       const void* cos_tbl, const void* sin_tbl, int n_pos, void* cache_kq,
                       void* cache_ks, void* cache_vq, void* cache_vs, int B, int H, int Hkv, int D,
                       int max_t, void* stream);

/* h[r,:] = emb[tokens[r], :] (fp16 table [vocab, dim], int64 ids, ids clamped into the table)
 * and the row's sum of squares as ss[r][0] (ss[r][1..ss_count) = 0): the first producer of the
 * residual stream in the form q40_gemv_fused mode 1/3 consumes.
 * Replaces: tok_embeddings lookup in Transformer.forward (hf_model_q40_kv_shared.py:495-498). */
int q40_embed_rows(const void* emb, const int64_t* tokens, void* h, float* ss, int ss_count, int rows,
                   int dim, int vocab, void* stream);

/* ---- epilogue math with the reference's rounding points ------------------------------ */

/* y[r,:] = fp16(fp16(x32 * rsqrt(mean(x32^2) + eps)) * w); if `residual` is non-NULL the
 * row is first replaced by h = fp16(x + residual), which is also written to h_out.
 * Replaces: RMSNorm.forward (hf_model_q40_kv_shared.py:123-134) and the residual adds of
 * TransformerBlock.forward (:463-466). */
int q40_rmsnorm(const void* x, const void* residual, const void* w, void* y, void* h_out,
                int rows, int dim, float eps, void* stream);

/* In-place rotary embedding of x[rows, n_heads, D] with per-row positions pos[rows] (int32)
 * and fp16 tables cos/sin [n_pos, D/2]: out = fp16(fp16(x*cos) + fp16(rot(x)*sin)),
 * rot(x) = cat(-x[D/2:], x[:D/2]).
 * Replaces: apply_rotary_emb / rotate_half (hf_model_q40_kv_shared.py:166-203). */
int q40_rope(void* x, const int32_t* pos, const void* cos_tbl, const void* sin_tbl, int rows,
             int n_heads, int D, int64_t row_stride, void* stream);

/* y = fp16(fp16(silu(a)) * b), n elements.
 * Replaces: F.silu(w1(x)) * w3(x) in FeedForward.forward (hf_model_q40_kv_shared.py:434). */
int q40_silu_mul(const void* a, const void* b, void* y, int64_t n, void* stream);

/* Causal attention of the prompt pass: o[S, H*128] = softmax over j <= i of q_i . k_j / sqrt(128), times v, per head,
 * for S positions at once; q / o rows hold H heads, k / v rows Hkv heads (H % Hkv == 0, grouped-query heads
 * read their kv head directly); ld* are row strides in elements.  Replaces the masked
 * scaled_dot_product_attention of hf_model_q40_kv_shared.py:375-405 (mask built at :499-504). */
int q40_attn_causal(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, void* o,
                    int64_t ldo, int S, int H, int Hkv, int D, void* stream);

/* ---- tensor-parallel all-reduce fused with residual add and RMSNorm (no counterpart in the reference beyond
 * the torch.distributed all_reduce after wo and w2, hf_model_q40_kv_shared.py:258-261) ----
 * One process per GPU.  Every rank allocates one buffer (q40_tp_alloc: cudaMalloc + zero fill + CUDA IPC handle of
 * 64 bytes), hands the handle to the other ranks by any host channel, and maps theirs (q40_tp_open).
 * q40_tp_layout gives {offset of the receive areas, total bytes} for (world <= 8, max_rows, dim); a receive
 * area is [2][world][max_rows][dim / 4] lines of 16 bytes {2 fp16, flag, 2 fp16, flag}.
 * q40_tp_allreduce_norm, called by all ranks in the same order:
 *   h[rows, dim] += fp16(sum over ranks of partial[rows, dim], fp32, rank order); xn = RMSNorm(h) * norm_w
 * (norm_w / xn may be NULL).  The kernel pushes its partial rows into the peers' buffers with plain 16-byte
 * stores that carry the call's sequence number as their flags (no fences), waits for the peers' lines at
 * most `wait_cycles` SM cycles (<= 0: 2^31) and reduces locally; a wait that expires sets the status word
 * (q40_tp_status: 1 + the missing rank) and the launch still ends.  `bufs` is a
 * host array of `world` device pointers (own buffer at [rank]).  Capturable in a CUDA graph: the call's
 * sequence number lives in the buffer. */
int q40_tp_layout(int world, int max_rows, int dim, size_t* out2);
int q40_tp_alloc(size_t bytes, void** ptr, void* handle64);
int q40_tp_open(const void* handle64, void** ptr);
int q40_tp_close(void* ptr);
int q40_tp_free(void* ptr);
int q40_tp_allreduce_norm(const void* partial, int64_t ldp, void* h, const void* norm_w, void* xn, int rows, int dim,
                          float eps, int rank, int world, void* const* bufs, int max_rows, long long wait_cycles,
                          void* stream);
int q40_tp_status(void* own_buf, int* host_out, int clear, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q40B200_H */
