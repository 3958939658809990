// Q4_0 packer and unpacker (bit-exact with the reference's torch functions).
//
// Format, restated from the reference's quantize_q40 / dequantize_q40
// (triton_kernels.py:12-56): the tensor is read row-major as groups of G elements;
// scale[g] = fp16(absmax/7) ; code = int8(rint(fp16(w/scale))) ; groups (2j, 2j+1) share a
// packed row of G bytes: byte i = code[2j][i] << 4 | code[2j+1][i] & 0xF.
//
// Both kernels are pure streaming kernels (HBM-bound): 16-byte loads and stores, one
// thread handles 8 consecutive elements of an even group and the matching 8 of the odd
// group so that it can emit 8 finished bytes on its own.
#include "q40_common.cuh"

namespace q40 {

// ---------------------------------------------------------------------------------------
// quantise: rows of `row_len` elements; a "pair" is 2*G consecutive elements of a row.
// G/8 threads cooperate on one pair (absmax via shuffles inside that lane group).
// ---------------------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __half* __restrict__ w, int64_t w_row_stride, uint8_t* __restrict__ q,
                     int64_t q_row_stride, __half* __restrict__ s, int64_t s_row_stride,
                     int64_t n_rows, int pairs_per_row) {
  constexpr int TPP = G / 8;  // threads per pair
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t pair = gtid / TPP;
  const int sub = (int)(gtid % TPP);
  const int64_t total_pairs = n_rows * (int64_t)pairs_per_row;
  const bool live = pair < total_pairs;
  const int64_t row = live ? pair / pairs_per_row : 0;
  const int pj = live ? (int)(pair % pairs_per_row) : 0;

  const __half* src = w + row * w_row_stride + (int64_t)pj * 2 * G + sub * 8;
  uint4 e = make_uint4(0, 0, 0, 0), o = make_uint4(0, 0, 0, 0);
  if (live) {
    e = *reinterpret_cast<const uint4*>(src);      // 8 elements of the even group
    o = *reinterpret_cast<const uint4*>(src + G);  // the same positions of the odd group
  }
  const __half2* eh = reinterpret_cast<const __half2*>(&e);
  const __half2* oh = reinterpret_cast<const __half2*>(&o);
  float me = 0.f, mo = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 a = __half22float2(eh[i]), b = __half22float2(oh[i]);
    me = fmaxf(me, fmaxf(fabsf(a.x), fabsf(a.y)));   // fmaxf drops NaN like torch.max would not,
    mo = fmaxf(mo, fmaxf(fabsf(b.x), fabsf(b.y)));   // but NaN inputs are outside the format
  }
#pragma unroll
  for (int off = TPP / 2; off > 0; off >>= 1) {
    me = fmaxf(me, __shfl_xor_sync(0xffffffffu, me, off));
    mo = fmaxf(mo, __shfl_xor_sync(0xffffffffu, mo, off));
  }
  // scale = fp16(absmax / 7): fp32 division, one rounding to fp16
  const __half se = __float2half_rn(__fdiv_rn(me, 7.0f));
  const __half so = __float2half_rn(__fdiv_rn(mo, 7.0f));
  const float fe = __half2float(se), fo = __half2float(so);

  uint32_t out[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = __half2float(reinterpret_cast<const __half*>(&e)[i]);
    const float b = __half2float(reinterpret_cast<const __half*>(&o)[i]);
    // quotient rounded to fp16 first (the format's double rounding), then to integer, ties even
    float qa = __half2float(__float2half_rn(__fdiv_rn(a, fe)));
    float qb = __half2float(__float2half_rn(__fdiv_rn(b, fo)));
    qa = rintf(qa);
    qb = rintf(qb);
    // NaN (0/0) and inf (x/0) become 0, as the x86 float->int conversion makes them
    int ia = (fabsf(qa) <= 65504.0f) ? (int)qa : 0;
    int ib = (fabsf(qb) <= 65504.0f) ? (int)qb : 0;
    ia = (int)(int8_t)ia;  // wrap like a cast to int8
    ib = (int)(int8_t)ib;
    const uint32_t byte = (uint32_t)(((ia << 4) | (ib & 0xF)) & 0xFF);
    out[i >> 2] |= byte << (8 * (i & 3));
  }
  if (live) {
    uint8_t* dst = q + row * q_row_stride + (int64_t)pj * G + sub * 8;
    *reinterpret_cast<uint2*>(dst) = make_uint2(out[0], out[1]);
    if (sub == 0) {
      __half* sd = s + row * s_row_stride + (int64_t)pj * 2;
      *reinterpret_cast<__half2*>(sd) = __halves2half2(se, so);
    }
  }
}

// ---------------------------------------------------------------------------------------
// dequantise: one thread = 16 packed bytes -> 16 values of the even group + 16 of the odd.
// ---------------------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint8_t* __restrict__ q, const __half* __restrict__ s,
                  __half* __restrict__ out, int64_t n_bytes) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t byte0 = t * 16;
  if (byte0 >= n_bytes) return;
  const int64_t prow = byte0 / G;      // packed row = pair index
  const int i0 = (int)(byte0 % G);
  const uint4 p = *reinterpret_cast<const uint4*>(q + byte0);
  const __half2 sc = *reinterpret_cast<const __half2*>(s + 2 * prow);
  const __half2 s_hi = __half2half2(__low2half(sc));
  const __half2 s_lo = __half2half2(__high2half(sc));
  const uint32_t wds[4] = {p.x, p.y, p.z, p.w};
  uint32_t hi[8], lo[8];
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    const uint32_t w0 = wds[wi];       // bytes b0 b1 b2 b3
    const uint32_t w1 = w0 >> 8;       // bytes b1 b2 b3 -
    // half2 results hold (b0,b2) and (b1,b3); put them back in byte order with prmt
    const __half2 l02 = __hmul2(codes_lo_to_h2(w0), s_lo);
    const __half2 l13 = __hmul2(codes_lo_to_h2(w1), s_lo);
    const __half2 h02 = __hmul2(codes_hi_to_h2(w0), s_hi);
    const __half2 h13 = __hmul2(codes_hi_to_h2(w1), s_hi);
    lo[wi * 2 + 0] = prmt(h2_as_u32(l02), h2_as_u32(l13), 0x5410);  // (b0, b1)
    lo[wi * 2 + 1] = prmt(h2_as_u32(l02), h2_as_u32(l13), 0x7632);  // (b2, b3)
    hi[wi * 2 + 0] = prmt(h2_as_u32(h02), h2_as_u32(h13), 0x5410);
    hi[wi * 2 + 1] = prmt(h2_as_u32(h02), h2_as_u32(h13), 0x7632);
  }
  __half* oe = out + prow * 2 * G + i0;  // even group
  __half* oo = oe + G;                   // odd group
  reinterpret_cast<uint4*>(oe)[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  reinterpret_cast<uint4*>(oe)[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
  reinterpret_cast<uint4*>(oo)[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  reinterpret_cast<uint4*>(oo)[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
}

}  // namespace q40

extern "C" int q40_quantize_rows(const void* w, int64_t w_row_stride, void* q, int64_t q_row_stride,
                                 void* s, int64_t s_row_stride, int64_t n_rows, int row_len,
                                 int group, void* stream) {
  if (!w || !q || !s) return Q40_E_NULL;
  if (group != 64 && group != 32) return Q40_E_UNSUPPORTED;
  if (n_rows < 0 || row_len < 0 || row_len % (2 * group) != 0) return Q40_E_SHAPE;
  if (n_rows == 0 || row_len == 0) return Q40_OK;
  if (!q40_aligned(w, 16) || !q40_aligned(q, 8) || !q40_aligned(s, 4)) return Q40_E_ALIGN;
  if (w_row_stride % 8 != 0 || q_row_stride % 8 != 0 || s_row_stride % 2 != 0) return Q40_E_ALIGN;
  const int pairs_per_row = row_len / (2 * group);
  const int64_t threads = n_rows * (int64_t)pairs_per_row * (group / 8);
  const int block = 256;
  const int64_t grid = (threads + block - 1) / block;
  if (grid > 0x7fffffffLL) return Q40_E_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (group == 64)
    q40::quantize_rows_kernel<64><<<(unsigned)grid, block, 0, st>>>(
        (const __half*)w, w_row_stride, (uint8_t*)q, q_row_stride, (__half*)s, s_row_stride, n_rows,
        pairs_per_row);
  else
    q40::quantize_rows_kernel<32><<<(unsigned)grid, block, 0, st>>>(
        (const __half*)w, w_row_stride, (uint8_t*)q, q_row_stride, (__half*)s, s_row_stride, n_rows,
        pairs_per_row);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}

extern "C" int q40_quantize(const void* w, void* q, void* s, int64_t n, int group, void* stream) {
  if (group != 64 && group != 32) return Q40_E_UNSUPPORTED;
  if (n < 0 || n % (2 * group) != 0) return Q40_E_SHAPE;
  // one "row" per pair of groups keeps every index within int range
  return q40_quantize_rows(w, 2 * group, q, group, s, 2, n / (2 * group), 2 * group, group, stream);
}

extern "C" int q40_dequantize(const void* q, const void* s, void* out, int64_t n, int group,
                              void* stream) {
  if (!q || !s || !out) return Q40_E_NULL;
  if (group != 64 && group != 32) return Q40_E_UNSUPPORTED;
  if (n < 0 || n % (2 * group) != 0) return Q40_E_SHAPE;
  if (n == 0) return Q40_OK;
  if (!q40_aligned(q, 16) || !q40_aligned(out, 16) || !q40_aligned(s, 4)) return Q40_E_ALIGN;
  const int64_t n_bytes = n / 2;
  const int64_t threads = n_bytes / 16;
  const int block = 256;
  const int64_t grid = (threads + block - 1) / block;
  if (grid > 0x7fffffffLL) return Q40_E_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (group == 64)
    q40::dequantize_kernel<64><<<(unsigned)grid, block, 0, st>>>((const uint8_t*)q, (const __half*)s,
                                                              (__half*)out, n_bytes);
  else
    q40::dequantize_kernel<32><<<(unsigned)grid, block, 0, st>>>((const uint8_t*)q, (const __half*)s,
                                                              (__half*)out, n_bytes);
  Q40_LAUNCH_CHECK();
  return Q40_OK;
}
