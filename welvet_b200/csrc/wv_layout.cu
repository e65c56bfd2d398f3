// Upload-time re-layout (wire -> device planes), the bit-exact unpack kernel and the
// shape-agnostic GEMV used for matrices whose rows do not start on a chunk boundary.
//
// Everything that defines a dequantised weight lives in wv_dequant(): it restates the
// reference's Unpack formulas (quant/q4_0.go:47-79, q4_1.go:51-76, q5_0.go:47-68,
// q5_1.go:48-70, q8_0.go:46-66, kquant.go:178-188, iq.go:169-180, ternary.go:53-62,
// binary.go:49-84, affine_g64.go:121-175, core/floatconv.go:21-46) with one explicitly
// rounded float32 operation per Go operation. This translation unit is compiled with
// --fmad=false and uses the _rn intrinsics anyway, so no multiply-add is ever contracted:
// amd64 Go rounds each float32 operation separately and the unpack result must match it
// bit for bit.
#include "wv_common.cuh"

__constant__ float c_iq4nl[16] = WV_IQ4NL_GRID;

// ---------------------------------------------------------------- wire readers
__device__ __forceinline__ unsigned read_bits(const uint8_t* p, size_t nbytes, long long bitoff, int nbits) {
  size_t by = (size_t)(bitoff >> 3);
  unsigned v = 0;
  if (by < nbytes) v = p[by];
  if (by + 1 < nbytes) v |= (unsigned)p[by + 1] << 8;
  return (v >> (bitoff & 7)) & ((1u << nbits) - 1u);
}
__device__ __forceinline__ float read_f32(const uint8_t* p) {
  unsigned u = (unsigned)p[0] | ((unsigned)p[1] << 8) | ((unsigned)p[2] << 16) | ((unsigned)p[3] << 24);
  return __uint_as_float(u);
}

// Stored code of flat weight i, read from the wire layout of Raw.
__device__ __forceinline__ unsigned wire_code(int format, const WvFmtInfo fi, const uint8_t* raw, size_t nraw, long long i) {
  const int bits = fi.bits_lo + fi.bits_hi;
  unsigned c;
  if (fi.kind == WK_CLASSIC) {
    long long blk = i >> 5; int j = (int)(i & 31);
    size_t off = (size_t)blk * fi.wire_block + (fi.has_min ? 8 : 4);
    if (off + (size_t)(bits * 4) > nraw) return 0;
    c = read_bits(raw + off, (size_t)bits * 4, (long long)j * bits, bits);
    if (format == WV_Q4_0) c ^= 8u;
    if (format == WV_Q8_0) c ^= 0x80u;
    return c;
  }
  if (fi.kind == WK_KQUANT) {
    long long sb = i >> 8; int idx = (int)(i & 255);
    size_t off = (size_t)sb * fi.wire_block + (fi.has_min ? 40 : 24);
    if (off + (size_t)(bits * 32) > nraw) return 0;
    return read_bits(raw + off, (size_t)bits * 32, (long long)idx * bits, bits);
  }
  c = read_bits(raw, nraw, i * bits, bits);
  if (format == WV_TERNARY && c == 3u) c = 1u;  // both decode to 0 (ternary.go:53-62)
  return c;
}

// One thread per 32-weight chunk: gathers its codes from the wire and writes the planes
// and the per-chunk parameters.
__global__ void relayout_kernel(WvDevBlob b, const uint8_t* __restrict__ raw, size_t nraw) {
  const WvFmtInfo fi = wv_fmt_info(b.format);
  const int BL = fi.bits_lo, BH = fi.bits_hi;
  long long ch = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= b.nchunks) return;
  uint32_t* lo = const_cast<uint32_t*>(b.lo);
  uint32_t* hi = const_cast<uint32_t*>(b.hi);
  unsigned low[8] = {0, 0, 0, 0, 0, 0, 0, 0}, hiw[2] = {0, 0};
  const int cpw = 32 / BL;
  for (int j = 0; j < 32; j++) {
    unsigned c = wire_code(b.format, fi, raw, nraw, ch * 32 + j);
    low[j / cpw] |= (c & ((1u << BL) - 1u)) << (BL * (j % cpw));
    if (BH) {
      int k = wv_k_of(BL, j), m = wv_m_of(BL, j);
      hiw[wv_hi_word(BH, k)] |= (c >> BL) << wv_hi_bit(BH, k, m);
    }
  }
  for (int w = 0; w < BL; w++) lo[ch * BL + w] = low[w];
  for (int w = 0; w < BH; w++) hi[ch * BH + w] = hiw[w];
  if (fi.kind == WK_CLASSIC) {
    size_t off = (size_t)ch * fi.wire_block;
    float* p0 = const_cast<float*>(b.p0);
    float* p1 = const_cast<float*>(b.p1);
    bool ok = off + fi.wire_block <= nraw;
    p0[ch] = ok ? read_f32(raw + off) : 1.0f;
    if (fi.has_min) p1[ch] = ok ? read_f32(raw + off + 4) : 0.0f;
  } else if (fi.kind == WK_KQUANT) {
    long long sb = ch >> 3; int cc = (int)(ch & 7);
    size_t off = (size_t)sb * fi.wire_block;
    bool ok = off + fi.wire_block <= nraw;
    if (cc == 0) {
      float2* kd = reinterpret_cast<float2*>(const_cast<float*>(b.p0));
      kd[sb] = ok ? make_float2(read_f32(raw + off), read_f32(raw + off + 4)) : make_float2(1.f, 0.f);
    }
    // A zero scale byte decodes as d/255 (kquant.go:180-182), which is exactly what byte 1
    // decodes to (d*1/255), so it is stored as 1 and the GEMV needs no special case.
    unsigned s0 = ok ? raw[off + 8 + 2 * cc] : 1, s1 = ok ? raw[off + 8 + 2 * cc + 1] : 1;
    if (s0 == 0) s0 = 1;
    if (s1 == 0) s1 = 1;
    if (fi.has_min) {
      unsigned m0 = ok ? raw[off + 24 + 2 * cc] : 0, m1 = ok ? raw[off + 24 + 2 * cc + 1] : 0;
      const_cast<uint32_t*>(b.km)[ch] = s0 | (s1 << 8) | (m0 << 16) | (m1 << 24);
    } else {
      reinterpret_cast<uint16_t*>(const_cast<uint32_t*>(b.km))[ch] = (uint16_t)(s0 | (s1 << 8));
    }
  }
}

int wv_launch_relayout(const WvDevBlob& dst, const uint8_t* d_raw, size_t nraw, cudaStream_t st) {
  if (dst.nchunks <= 0) return WV_OK;
  const int nt = 128;
  long long nb = (dst.nchunks + nt - 1) / nt;
  relayout_kernel<<<(unsigned)nb, nt, 0, st>>>(dst, d_raw, nraw);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}

// ---------------------------------------------------------------- dequant (bit-exact)
__device__ __forceinline__ float f16_bits_to_f32(unsigned h) {  // core/floatconv.go:21-36
  unsigned sign = (h & 0x8000u) << 16, expo = (h >> 10) & 0x1fu, mant = h & 0x3ffu;
  if (expo == 0) {
    if (mant == 0) return __uint_as_float(sign);
    float d = __fmul_rn((float)mant, 5.9604644775390625e-08f);  // mant / 1024 / 16384, exact
    return __uint_as_float(sign | __float_as_uint(d));
  }
  if (expo == 31) return __uint_as_float(sign | 0x7f800000u | (mant << 13));
  return __uint_as_float(sign | ((expo - 15 + 127) << 23) | (mant << 13));
}

__device__ __forceinline__ float wv_dequant(const WvDevBlob& b, const WvFmtInfo fi, long long i) {
  if (fi.kind == WK_NONE) {
    if (b.dtype == WV_DT_F32) return __uint_as_float(b.lo[i]);
    unsigned h = reinterpret_cast<const uint16_t*>(b.lo)[i];
    return b.dtype == WV_DT_F16 ? f16_bits_to_f32(h) : __uint_as_float(h << 16);
  }
  unsigned u = wv_dev_code(b, fi.bits_lo, fi.bits_hi, i);
  switch (fi.kind) {
  case WK_CLASSIC: {
    float scale = b.p0[i >> 5];
    if (fi.has_min) return __fadd_rn(b.p1[i >> 5], __fmul_rn((float)u, scale));
    return __fmul_rn((float)((int)u - fi.mid), scale);
  }
  case WK_KQUANT: {
    float2 dd = reinterpret_cast<const float2*>(b.p0)[i >> 8];
    int g = (int)((i & 255) >> 4);
    long long ch = i >> 5;
    unsigned su, mu = 0;
    if (fi.has_min) { unsigned km = b.km[ch]; su = (km >> (8 * (g & 1))) & 0xffu; mu = (km >> (16 + 8 * (g & 1))) & 0xffu; }
    else { unsigned km = reinterpret_cast<const uint16_t*>(b.km)[ch]; su = (km >> (8 * (g & 1))) & 0xffu; }
    float sc = __fdiv_rn(__fmul_rn(dd.x, (float)su), 255.0f);
    if (sc == 0.0f) sc = __fdiv_rn(dd.x, 255.0f);
    if (fi.has_min) {
      float mn = __fdiv_rn(__fmul_rn(dd.y, (float)(int)(signed char)mu), 127.0f);
      return __fadd_rn(mn, __fmul_rn((float)u, sc));
    }
    return __fmul_rn(sc, (float)((int)u - fi.mid));
  }
  case WK_IQ: {
    float scale = b.p0[i / fi.pgroup];
    if (fi.table) return __fmul_rn(scale, c_iq4nl[u & 15]);
    if (fi.sign) return (u & 1) ? scale : -scale;
    return __fmul_rn(scale, __fsub_rn((float)u, (float)fi.mid + 0.5f));
  }
  case WK_TERNARY: {
    float scale = b.p0[i >> 4];
    return u == 0 ? -scale : (u == 2 ? scale : 0.0f);
  }
  case WK_BINARY: {
    float scale = b.p0[i / b.group];
    return (u & 1) ? scale : -scale;
  }
  case WK_AFFINE: {
    long long g = i / b.group;
    return __fadd_rn(__fmul_rn(b.p0[g], (float)u), b.p1[g]);
  }
  }
  return 0.0f;
}

__global__ void unpack_kernel(WvDevBlob b, float* __restrict__ out) {
  const WvFmtInfo fi = wv_fmt_info(b.format);
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < b.n; i += stride) out[i] = wv_dequant(b, fi, i);
}

int wv_launch_unpack(const WvDevBlob& b, float* d_out, cudaStream_t st) {
  long long nb = (b.n + 255) / 256;
  if (nb > 148 * 32) nb = 148 * 32;
  unpack_kernel<<<(unsigned)nb, 256, 0, st>>>(b, d_out);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}

// quant.DecodeRow (quant/decode_row.go:7-38): one output row of the matrix as float32, the same values Unpack gives
// for that row. Rows are counted within the rows this device holds.
__global__ void unpack_rows_kernel(WvDevBlob b, long long first, long long count, float* __restrict__ out) {
  const WvFmtInfo fi = wv_fmt_info(b.format);
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) out[i] = wv_dequant(b, fi, first + i);
}
int wv_launch_unpack_rows(const WvDevBlob& b, int row, int nrows, float* d_out, cudaStream_t st) {
  const long long count = (long long)nrows * b.cols;
  long long nb = (count + 255) / 256;
  if (nb > 148 * 32) nb = 148 * 32;
  if (nb < 1) return WV_OK;
  unpack_rows_kernel<<<(unsigned)nb, 256, 0, st>>>(b, (long long)row * b.cols, count, d_out);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}

// ---------------------------------------------------------------- ragged-shape GEMV
// One warp per output row, lanes stride over columns, exact dequant + f32 multiply-add,
// shuffle reduction. Used only when rows are not chunk aligned (cols % 32*J != 0); the
// config shapes all take the chunked kernels in wv_gemv.cu.
__global__ void gemv_ragged_kernel(WvDevBlob b, const float* __restrict__ x, float* __restrict__ y,
                                   int batch, int row_begin, int row_end) {
  const WvFmtInfo fi = wv_fmt_info(b.format);
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int nwarps = (gridDim.x * blockDim.x) >> 5;
  int nrows = row_end - row_begin;
  for (long long item = warp; item < (long long)nrows * batch; item += nwarps) {
    int bi = (int)(item / nrows), r = row_begin + (int)(item % nrows);
    const float* xb = x + (long long)bi * b.cols;
    float acc = 0.0f;
    for (int c = lane; c < b.cols; c += 32) acc = fmaf(wv_dequant(b, fi, (long long)r * b.cols + c), xb[c], acc);
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[(long long)bi * b.rows + r] = acc;
  }
}

int wv_launch_gemv_ragged(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end,
                          cudaStream_t st) {
  long long items = (long long)(row_end - row_begin) * batch;
  if (items <= 0) return WV_OK;
  long long nb = (items + 7) / 8;
  if (nb > 148 * 8) nb = 148 * 8;
  gemv_ragged_kernel<<<(unsigned)nb, 256, 0, st>>>(b, dx, dy, batch, row_begin, row_end);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}
