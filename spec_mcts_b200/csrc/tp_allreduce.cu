// Tensor-parallel all-reduce fused with the residual add and the next RMSNorm, over peer-mapped buffers.
//
// The reference sums the partial outputs of the row-parallel projections (wo, w2) with one
// torch.distributed all_reduce each (hf_model_q40_kv_shared.py:258-261) and then adds the residual and
// normalises in separate operations.  A decode step of the 70B geometry has 160 such reductions of at most
// a megabyte: latency, not bandwidth.  Here one kernel per reduction does all three steps, one CTA per
// batch row:
//   1. PUSH: the CTA stores its row of this rank's partial output into every peer's receive area with plain
//      16-byte global stores through NVLink (no loads from a peer, no bulk or tensor copies).  Every 16-byte
//      store is a self-validating line {data, flag, data, flag} with flag = the call's sequence number (the
//      "LL" scheme of collective libraries): the receiver needs no fence and the sender no flag store after a
//      fence — a system-scope fence costs about 5 us on this GPU, two of them more than the whole transfer;
//   2. REDUCE locally, waiting per line and bounded: a thread spins on its own lines until both flags show the
//      sequence number; when the limit in cycles expires the kernel records a status word and goes on, so the
//      launch always ends.  fp32 sum of the ranks' fp16 partials in rank order (the same order on every rank,
//      so all ranks hold bit-identical residual streams), one rounding to fp16, fp16 residual add, RMSNorm
//      with the reference's rounding points (hf_model_q40_kv_shared.py:129-134).
// Two ranks exchange whole rows in one shot as described.  More than two ranks work in two shots, so that a
// rank sends 2 (world - 1) / world rows' worth instead of world - 1: rank j receives column slice j of every
// peer's partial row, sums it (rank order, fp32), adds the residual and pushes the finished slice to everybody;
// every rank then holds the same finished row and normalises it.  (One shot at 8 ranks: 64 us per 1 MiB
// reduction, slower than the library's 50 us.)
// Receive areas are double-buffered by the parity of the sequence number: a rank can be at most one call
// ahead of a peer, because it cannot finish call k + 1 before that peer has pushed call k + 1, which the peer
// does only after it has consumed call k.  The sequence number lives in the rank's own buffer and is
// advanced by the last CTA of a launch, so CUDA-graph replays need no host-side argument.
//
// The buffers are plain cudaMalloc allocations shared between the ranks' processes with CUDA IPC handles.
// No counterpart in the reference beyond the all_reduce call it replaces.
#include <cstdio>
#include <cstring>

#include "q40_common.cuh"

namespace q40 {
namespace tp {

constexpr int MAX_WORLD = 8;
constexpr int THREADS = 256;
constexpr size_t HEADER_BYTES = 256;      // [0] sequence number, [1] finished CTAs, [2] status

// receive area: [2 slots][world][max_rows][dim / 4 lines of 16 bytes], a line = 4 fp16 values and two flags
struct Layout {
  size_t recv_off, total;
};
static inline Layout make_layout(int world, int max_rows, int dim) {
  Layout l;
  l.recv_off = HEADER_BYTES;
  l.total = l.recv_off + (size_t)2 * world * max_rows * dim * 4;
  return l;
}

struct Params {
  unsigned char* bufs[MAX_WORLD];   // every rank's buffer as mapped into this process (own at [rank])
  const __half* partial;            // [rows, ldp] this rank's partial output
  int64_t ldp;
  __half* h;                        // [rows, dim] residual stream, updated in place
  const __half* norm_w;             // [dim] or null: no normalised output
  __half* xn;                       // [rows, dim]
  int rows, dim, rank, world, max_rows;
  float eps;
  long long wait_cycles;
  size_t recv_off;
};

__device__ __forceinline__ void st_line(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(THREADS)
allreduce_norm_kernel(const Params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* row = reinterpret_cast<__half*>(smem_raw);     // [dim]
  __shared__ float red[THREADS / 32];
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");      // the partial output comes from the previous launch
  const int r = blockIdx.x, tid = threadIdx.x;
  unsigned char* own = p.bufs[p.rank];
  int* hdr = reinterpret_cast<int*>(own);
  const int seq = *reinterpret_cast<volatile int*>(hdr) + 1;
  const int slot = seq & 1;
  const size_t row_lines = (size_t)p.dim / 4;
  const __half* mine = p.partial + (int64_t)r * p.ldp;

  float ss = 0.f;
  __half* hr = p.h + (int64_t)r * p.dim;
  const long long t0 = clock64();
  bool gave_up = false;
  // a peer line: spin (bounded) until both flags show this call's sequence number
  auto wait_lines = [&](const uint4* src, int q) -> uint4 {
    uint4 l0 = ld_line(src), l1 = ld_line(src + 1);
    unsigned spins = 0;
    while (!gave_up && !(l0.y == (uint32_t)seq && l0.w == (uint32_t)seq && l1.y == (uint32_t)seq && l1.w == (uint32_t)seq)) {
      if ((++spins & 63u) == 0 && clock64() - t0 > p.wait_cycles) {
        atomicExch(hdr + 2, 1 + q);     // status: 1 + the rank that did not arrive
        gave_up = true;
        break;
      }
      l0 = ld_line(src);
      l1 = ld_line(src + 1);
    }
    return make_uint4(l0.x, l0.z, l1.x, l1.z);
  };
  auto push_lines = [&](uint4* dst, uint4 v) {
    st_line(dst, make_uint4(v.x, (uint32_t)seq, v.y, (uint32_t)seq));
    st_line(dst + 1, make_uint4(v.z, (uint32_t)seq, v.w, (uint32_t)seq));
  };
  auto add8 = [](float (&acc)[8], uint4 v) {
    const __half2* vh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(vh[j]);
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  };
  // residual add of 8 columns (fp16 add, one rounding), sum of squares, store to h and to the row buffer
  auto finish8 = [&](int i, const float (&acc)[8]) -> uint4 {
    uint4 hv = *reinterpret_cast<const uint4*>(hr + i);
    __half2* hh = reinterpret_cast<__half2*>(&hv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      hh[j] = __hadd2(hh[j], __floats2half2_rn(acc[2 * j], acc[2 * j + 1]));
      const float2 f = __half22float2(hh[j]);
      ss = fmaf(f.x, f.x, ss);
      ss = fmaf(f.y, f.y, ss);
    }
    *reinterpret_cast<uint4*>(hr + i) = hv;
    *reinterpret_cast<uint4*>(row + i) = hv;
    return hv;
  };

  if (p.world <= 2) {
    // ================= one shot: every rank gets every rank's whole row =================
    // ---- 1. push this rank's row into every peer's receive area [slot][this rank][row] ----
    for (int q = 0; q < p.world; ++q) {
      if (q == p.rank) continue;
      uint4* dst = reinterpret_cast<uint4*>(p.bufs[q] + p.recv_off) +
                   (((size_t)slot * p.world + p.rank) * p.max_rows + r) * row_lines;
      for (int i = tid * 8; i < p.dim; i += THREADS * 8)
        push_lines(dst + i / 4, *reinterpret_cast<const uint4*>(mine + i));
    }
    // ---- 2. fp32 sum in rank order (waiting, bounded, for each peer line), one rounding, residual add ----
    const uint4* recv = reinterpret_cast<const uint4*>(own + p.recv_off);
    for (int i = tid * 8; i < p.dim; i += THREADS * 8) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int q = 0; q < p.world; ++q) {
        const uint4 v = (q == p.rank)
            ? *reinterpret_cast<const uint4*>(mine + i)
            : wait_lines(recv + (((size_t)slot * p.world + q) * p.max_rows + r) * row_lines + i / 4, q);
        add8(acc, v);
      }
      finish8(i, acc);
    }
  } else {
    // ================= two shots: rank j sums columns [j dim / world, (j + 1) dim / world) of every row and
    // hands the finished slice (residual already added) to everybody =================
    // areas: scatter [slot][source rank][row][slice lines], then gather with the same shape
    const int ls = p.dim / p.world;                         // slice length in columns (a multiple of 8)
    const size_t slice_lines = (size_t)ls / 4;
    const size_t area_lines = (size_t)2 * p.world * p.max_rows * slice_lines;
    auto scatter_of = [&](unsigned char* buf) { return reinterpret_cast<uint4*>(buf + p.recv_off); };
    auto gather_of = [&](unsigned char* buf) { return reinterpret_cast<uint4*>(buf + p.recv_off) + area_lines; };
    const size_t my_src = (((size_t)slot * p.world + p.rank) * p.max_rows + r) * slice_lines;   // as a source in a peer's area
    const int chunks = ls / 8;
    // ---- 1. push slice q of this rank's partial row to rank q ----
    for (int e = tid; e < (p.world - 1) * chunks; e += THREADS) {
      int q = e / chunks;
      const int c = e % chunks;
      if (q >= p.rank) ++q;
      push_lines(scatter_of(p.bufs[q]) + my_src + 2 * c, *reinterpret_cast<const uint4*>(mine + q * ls + 8 * c));
    }
    // ---- 2. own slice: fp32 sum in rank order, one rounding, residual add; push the result to every peer ----
    const uint4* sc_in = scatter_of(own);
    for (int c = tid; c < chunks; c += THREADS) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      const int i = p.rank * ls + 8 * c;
      for (int q = 0; q < p.world; ++q) {
        const uint4 v = (q == p.rank)
            ? *reinterpret_cast<const uint4*>(mine + i)
            : wait_lines(sc_in + (((size_t)slot * p.world + q) * p.max_rows + r) * slice_lines + 2 * c, q);
        add8(acc, v);
      }
      const uint4 hv = finish8(i, acc);
      for (int q = 0; q < p.world; ++q)
        if (q != p.rank) push_lines(gather_of(p.bufs[q]) + my_src + 2 * c, hv);
    }
    // ---- 3. the other ranks' finished slices ----
    const uint4* ga_in = gather_of(own);
    for (int e = tid; e < (p.world - 1) * chunks; e += THREADS) {
      int q = e / chunks;
      const int c = e % chunks;
      if (q >= p.rank) ++q;
      const uint4 hv = wait_lines(ga_in + (((size_t)slot * p.world + q) * p.max_rows + r) * slice_lines + 2 * c, q);
      const int i = q * ls + 8 * c;
      const __half2* hh = reinterpret_cast<const __half2*>(&hv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(hh[j]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
      *reinterpret_cast<uint4*>(hr + i) = hv;
      *reinterpret_cast<uint4*>(row + i) = hv;
    }
  }
  if (p.norm_w != nullptr) {
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < THREADS / 32; ++i) tot += red[i];
    const float inv = rsqrtf(tot / (float)p.dim + p.eps);
    for (int i = tid * 8; i < p.dim; i += THREADS * 8) {
      uint4 v = *reinterpret_cast<const uint4*>(row + i);
      const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + i);
      __half2* vh = reinterpret_cast<__half2*>(&v);
      const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(vh[j]);
        vh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);   // round to fp16, then * weight in fp16
      }
      *reinterpret_cast<uint4*>(p.xn + (int64_t)r * p.dim + i) = v;
    }
  }
  // ---- the last CTA advances the sequence number (every CTA has read it by then) ----
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(hdr + 1, 1) == (int)gridDim.x - 1) {
      hdr[1] = 0;
      *reinterpret_cast<volatile int*>(hdr) = seq;
      __threadfence();
    }
  }
}

}  // namespace tp
}  // namespace q40

extern "C" int q40_tp_layout(int world, int max_rows, int dim, size_t* out2) {
  if (!out2) return Q40_E_NULL;
  if (world < 1 || world > q40::tp::MAX_WORLD || max_rows < 1 || dim < 8 || dim % 8 != 0) return Q40_E_SHAPE;
  const q40::tp::Layout l = q40::tp::make_layout(world, max_rows, dim);
  out2[0] = l.recv_off; out2[1] = l.total;
  return Q40_OK;
}

// A zero-filled device buffer of `bytes` on the current device and its 64-byte inter-process handle.
extern "C" int q40_tp_alloc(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64) return Q40_E_NULL;
  if (bytes == 0) return Q40_E_SHAPE;
  void* d = nullptr;
  cudaError_t e = cudaMalloc(&d, bytes);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  e = cudaMemset(d, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
  if (e != cudaSuccess) { (void)cudaGetLastError(); cudaFree(d); return (int)e; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  memcpy(handle64, &h, 64);
  *ptr = d;
  return Q40_OK;
}
extern "C" int q40_tp_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return Q40_E_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* d = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  *ptr = d;
  return Q40_OK;
}
extern "C" int q40_tp_close(void* ptr) {
  if (!ptr) return Q40_E_NULL;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  return Q40_OK;
}
extern "C" int q40_tp_free(void* ptr) {
  if (!ptr) return Q40_E_NULL;
  const cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  return Q40_OK;
}

// h[rows, dim] += sum over ranks of partial (fp32 sum in rank order, rounded once); xn = RMSNorm(h) * norm_w when
// norm_w is given.  `bufs`: host array of `world` device pointers, every rank's buffer of q40_tp_layout(...).total
// bytes as mapped into this process (own buffer at [rank]).  All ranks make the same sequence of calls.
// wait_cycles: limit of the wait for a peer's row in SM cycles (<= 0: about one second).
extern "C" int q40_tp_allreduce_norm(const void* partial, int64_t ldp, void* h, const void* norm_w, void* xn, int rows,
                                     int dim, float eps, int rank, int world, void* const* bufs, int max_rows,
                                     long long wait_cycles, void* stream) {
  using namespace q40::tp;
  if (!partial || !h || !bufs) return Q40_E_NULL;
  if (norm_w && !xn) return Q40_E_NULL;
  if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world) return Q40_E_SHAPE;
  if (rows < 1 || rows > max_rows || dim < 8 || dim % 8 != 0 || ldp < dim || ldp % 8 != 0) return Q40_E_SHAPE;
  if (world > 2 && dim % (8 * world) != 0) return Q40_E_SHAPE;      // column slices of whole 16-byte chunks
  if (!q40_aligned(partial, 16) || !q40_aligned(h, 16) || (norm_w && !q40_aligned(norm_w, 16)) ||
      (xn && !q40_aligned(xn, 16)))
    return Q40_E_ALIGN;
  Params p{};
  for (int i = 0; i < world; ++i) {
    if (!bufs[i] || !q40_aligned(bufs[i], 256)) return Q40_E_NULL;
    p.bufs[i] = (unsigned char*)bufs[i];
  }
  const Layout l = make_layout(world, max_rows, dim);
  p.partial = (const __half*)partial; p.ldp = ldp; p.h = (__half*)h; p.norm_w = (const __half*)norm_w; p.xn = (__half*)xn;
  p.rows = rows; p.dim = dim; p.rank = rank; p.world = world; p.max_rows = max_rows; p.eps = eps;
  p.wait_cycles = wait_cycles > 0 ? wait_cycles : (1ll << 31);
  p.recv_off = l.recv_off;
  const size_t smem = (size_t)dim * 2;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(allreduce_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return Q40_E_UNSUPPORTED; }
  }
  const cudaError_t e2 = q40_launch_pdl(allreduce_norm_kernel, dim3(rows), dim3(THREADS), smem, (cudaStream_t)stream, p);
  if (e2 != cudaSuccess) return (int)e2;
  return Q40_OK;
}

// Copies the status word of this rank's buffer to the host (0 = every wait was met; 1 + r = rank r did not
// arrive in time in some call) and optionally clears it.  Synchronises the stream.
extern "C" int q40_tp_status(void* own_buf, int* host_out, int clear, void* stream) {
  if (!own_buf || !host_out) return Q40_E_NULL;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(host_out, (char*)own_buf + 8, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess && clear) e = cudaMemsetAsync((char*)own_buf + 8, 0, sizeof(int), st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return (int)e;
  return Q40_OK;
}
