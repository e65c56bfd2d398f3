// Device helpers shared by the GEMV kernels: per-chunk weight fragments, the f32 chunk math
// (IQ4_NL) and the integer-dot chunk math (every other packed format).
#pragma once
#include "wv_common.cuh"
#include <cuda_fp16.h>
#include <cuda_runtime.h>

static __constant__ float c_grid4nl[16] = WV_IQ4NL_GRID;

// ------------------------------------------------------------------ fragments
template <int F> struct FragT {
  static constexpr WvFmtInfo fi = wv_fmt_info(F);
  static constexpr int BL = fi.bits_lo, BH = fi.bits_hi;
  // number of 32-bit parameter registers per chunk-row
  static constexpr int NP =
      fi.kind == WK_KQUANT ? 3 : ((fi.has_min || fi.pgroup == 16) ? 2 : 1);
  uint32_t lo[BL];
  uint32_t hi[BH ? BH : 1];
  uint32_t pr[NP];
};

template <int N> __device__ __forceinline__ void ldg_words(uint32_t (&dst)[N], const uint32_t* p) {
  if constexpr (N == 1) { dst[0] = __ldg(p); }
  else if constexpr (N == 2) { uint2 v = __ldg(reinterpret_cast<const uint2*>(p)); dst[0] = v.x; dst[1] = v.y; }
  else if constexpr (N == 4) { uint4 v = __ldg(reinterpret_cast<const uint4*>(p)); dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w; }
  else if constexpr (N == 8) {
    uint4 v = __ldg(reinterpret_cast<const uint4*>(p)), u = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w; dst[4] = u.x; dst[5] = u.y; dst[6] = u.z; dst[7] = u.w;
  }
}

// cg = global chunk index (row * chunks_per_row + chunk)
template <int F> __device__ __forceinline__ void load_frag(FragT<F>& f, const WvDevBlob& b, long long cg) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  ldg_words<FragT<F>::BL>(f.lo, b.lo + cg * FragT<F>::BL);
  if constexpr (fi.bits_hi == 1) f.hi[0] = __ldg(b.hi + cg);
  if constexpr (fi.bits_hi == 2) { uint2 v = __ldg(reinterpret_cast<const uint2*>(b.hi) + cg); f.hi[0] = v.x; f.hi[1] = v.y; }
  if constexpr (fi.kind == WK_KQUANT) {
    float2 dd = __ldg(reinterpret_cast<const float2*>(b.p0) + (cg >> 3));
    f.pr[0] = __float_as_uint(dd.x); f.pr[1] = __float_as_uint(dd.y);
    if constexpr (fi.has_min) f.pr[2] = __ldg(b.km + cg);
    else f.pr[2] = __ldg(reinterpret_cast<const unsigned short*>(b.km) + cg);
  } else if constexpr (fi.kind == WK_CLASSIC) {
    f.pr[0] = __float_as_uint(__ldg(b.p0 + cg));
    if constexpr (fi.has_min) f.pr[1] = __float_as_uint(__ldg(b.p1 + cg));
  } else if constexpr (fi.kind == WK_BINARY) {
    f.pr[0] = __float_as_uint(__ldg(b.p0 + (cg * 32) / b.group));
  } else if constexpr (fi.kind == WK_AFFINE) {
    long long g = (cg * 32) / b.group;
    f.pr[0] = __float_as_uint(__ldg(b.p0 + g)); f.pr[1] = __float_as_uint(__ldg(b.p1 + g));
  } else if constexpr (fi.pgroup == 16) {  // IQ *_XS/_S, ternary: two scales per chunk
    float2 s = __ldg(reinterpret_cast<const float2*>(b.p0) + cg);
    f.pr[0] = __float_as_uint(s.x); f.pr[1] = __float_as_uint(s.y);
  } else {  // IQ with one scale per 32
    f.pr[0] = __float_as_uint(__ldg(b.p0 + cg));
  }
}

// ------------------------------------------------------------------ chunk dot
// s0 / s1 = sum over the first / second 16 weights of (code - MID) * x (1-bit planes put
// everything in s0). xr[k] holds the four activations matching byte lanes 0..3 of group k.
template <int F>
__device__ __forceinline__ void chunk_dot(const FragT<F>& f, const float4 (&xr)[8], const float* tbl, float& s0, float& s1) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi, SPW = 8 / BL;
  constexpr unsigned MASK = 0x01010101u * ((1u << BL) - 1u);
  constexpr unsigned MASKH = BH ? (0x01010101u * ((1u << BH) - 1u)) << BL : 0u;
  const float magic = 8388608.0f + (float)fi.mid;
  float2 a0 = make_float2(0.f, 0.f), a1 = a0, b0 = a0, b1 = a0;
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const int w = k / SPW, s = k % SPW;
    unsigned bytes = (f.lo[w] >> (BL * s)) & MASK;
    if constexpr (BH > 0) {
      const int hw = (k * BH) >> 3, sh = (k * BH) & 7;
      unsigned hv = f.hi[hw];
      hv = sh >= BL ? (hv >> (sh - BL)) : (hv << (BL - sh));
      bytes |= hv & MASKH;
    }
    float2 q01, q23;
    if constexpr (fi.table) {
      q01.x = tbl[(bytes & 0xffu) * 32]; q01.y = tbl[((bytes >> 8) & 0xffu) * 32];
      q23.x = tbl[((bytes >> 16) & 0xffu) * 32]; q23.y = tbl[(bytes >> 24) * 32];
    } else {
      q01.x = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7650)) - magic;
      q01.y = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7651)) - magic;
      q23.x = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7652)) - magic;
      q23.y = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7653)) - magic;
    }
    const float2 x01 = make_float2(xr[k].x, xr[k].y), x23 = make_float2(xr[k].z, xr[k].w);
    if (BL == 1 || k < 4) { a0 = __ffma2_rn(q01, x01, a0); a1 = __ffma2_rn(q23, x23, a1); }
    else { b0 = __ffma2_rn(q01, x01, b0); b1 = __ffma2_rn(q23, x23, b1); }
  }
  s0 = (a0.x + a0.y) + (a1.x + a1.y);
  s1 = (b0.x + b0.y) + (b1.x + b1.y);
}

__device__ __forceinline__ float u8f(unsigned v, int byte) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650 + byte)) - 8388608.0f;
}

// Contribution of one chunk-row to its output row.
template <int F>
__device__ __forceinline__ float chunk_value(const FragT<F>& f, const float4 (&xr)[8], float2 sx, const float* tbl) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  float s0, s1;
  chunk_dot<F>(f, xr, tbl, s0, s1);
  if constexpr (fi.kind == WK_KQUANT) {
    const float d = __uint_as_float(f.pr[0]) * (1.0f / 255.0f);
    float a0 = d * u8f(f.pr[2], 0), a1 = d * u8f(f.pr[2], 1);
    if (a0 == 0.0f) a0 = d;  // kquant.go:180-182: a zero group scale decodes as d/255
    if (a1 == 0.0f) a1 = d;
    float v = a0 * s0 + a1 * s1;
    if constexpr (fi.has_min) {
      const float dm = __uint_as_float(f.pr[1]) * (1.0f / 127.0f);
      const unsigned mb = f.pr[2] ^ 0x80800000u;  // int8 -> biased uint8
      v += dm * ((u8f(mb, 2) - 128.0f) * sx.x + (u8f(mb, 3) - 128.0f) * sx.y);
    }
    return v;
  } else if constexpr (fi.kind == WK_CLASSIC || fi.kind == WK_AFFINE) {
    float v = __uint_as_float(f.pr[0]) * (s0 + s1);
    if constexpr (fi.has_min) v += __uint_as_float(f.pr[1]) * (sx.x + sx.y);
    return v;
  } else if constexpr (fi.kind == WK_BINARY || (fi.kind == WK_IQ && fi.sign)) {
    return __uint_as_float(f.pr[0]) * (2.0f * s0 - (sx.x + sx.y));
  } else if constexpr (fi.kind == WK_TERNARY) {
    return __uint_as_float(f.pr[0]) * s0 + __uint_as_float(f.pr[1]) * s1;
  } else {  // IQ linear / table
    if constexpr (fi.half_mid) { s0 -= 0.5f * sx.x; s1 -= 0.5f * sx.y; }
    if constexpr (fi.pgroup == 16) return __uint_as_float(f.pr[0]) * s0 + __uint_as_float(f.pr[1]) * s1;
    else return __uint_as_float(f.pr[0]) * (s0 + s1);
  }
}


// IQ4_NL in the bulk-copy kernel. A byte of the code plane holds two weights, so the table in shared memory is
// [256 bytes][32 lanes] of float2 {grid[low nibble], grid[high nibble]} and a byte costs one permute (byte 1 of the
// offset = the plane byte, byte 0 = 8 * lane), one 8-byte load and one paired FMA; lane l reads slot l of a row, so
// the 32 lanes of a load cover every bank exactly twice. xr[2w + h] = activations of bytes 2h, 2h + 1 of word w,
// each as {low-nibble weight's, high-nibble weight's}.
template <int F>
__device__ __forceinline__ float chunk_value_tbl(const FragT<F>& f, const float4 (&xr)[8], const unsigned char* tbl, unsigned lane8) {
  static_assert(wv_fmt_info(F).table && wv_fmt_info(F).bits_lo == 4, "4-bit table format");
  float2 a0 = make_float2(0.f, 0.f), a1 = a0, b0 = a0, b1 = a0;
#pragma unroll
  for (int w = 0; w < 4; w++) {
    const unsigned bytes = f.lo[w];
    const float2 q0 = *reinterpret_cast<const float2*>(tbl + __byte_perm(bytes, lane8, 0x5504));
    const float2 q1 = *reinterpret_cast<const float2*>(tbl + __byte_perm(bytes, lane8, 0x5514));
    const float2 q2 = *reinterpret_cast<const float2*>(tbl + __byte_perm(bytes, lane8, 0x5524));
    const float2 q3 = *reinterpret_cast<const float2*>(tbl + __byte_perm(bytes, lane8, 0x5534));
    a0 = __ffma2_rn(q0, make_float2(xr[2 * w].x, xr[2 * w].y), a0);
    a1 = __ffma2_rn(q1, make_float2(xr[2 * w].z, xr[2 * w].w), a1);
    b0 = __ffma2_rn(q2, make_float2(xr[2 * w + 1].x, xr[2 * w + 1].y), b0);
    b1 = __ffma2_rn(q3, make_float2(xr[2 * w + 1].z, xr[2 * w + 1].w), b1);
  }
  return __uint_as_float(f.pr[0]) * (((a0.x + a0.y) + (a1.x + a1.y)) + ((b0.x + b0.y) + (b1.x + b1.y)));
}

// ------------------------------------------------------------------ integer-dot chunk math
// Activations arrive as block fixed point (see xquant_kernel): per 32 columns
// X_j = rint(x_j * 2^(22-e)), 2^e > max|x| of the block, split into three byte limbs
// X = L0 + 256 L1 + 65536 L2 packed as int8x4 words in code-group order. Each group of four
// codes meets its four activations in one dp4a per limb (0.75 dp4a per weight, exact integer
// accumulation); the limb sums are recombined in f32 and scaled by sf = 2^(e-22) and the
// block's scale. Per element |x_j - X_j sf| <= 2^-23 of the block maximum (f32's own rounding
// is 2^-24 of the element) and there is no rounding inside the dot. Symmetric formats subtract
// mid in the integer domain (accumulators start at -mid*sum(L)): all-zero weights give exactly 0.
__device__ __forceinline__ int dp4a_uu(unsigned a, unsigned b, int c) {
  int d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_us(unsigned a, unsigned b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

template <int F> struct QCfg {
  static constexpr WvFmtInfo fi = wv_fmt_info(F);
  static constexpr bool HALVES = fi.pgroup == 16;                 // two parameter groups per chunk
  static constexpr bool INT_MID = fi.mid != 0 && !fi.half_mid;    // exact integer offset
  static constexpr int NH = HALVES ? 2 : 1;
  static constexpr int NREC = INT_MID ? 9 : 7;                    // uint4 records per chunk actually read
};

// One chunk's activation record held in registers.
struct XQRegs {
  unsigned xw[24];   // word limb*8 + k
  float4 mt;         // {sf, sf*SX(all), sf*SX(first 16), sf*SX(second 16)}
  int iv[6];         // -mid*sum(limb l, half h) at l*2+h (halves pre-added for 32-wide groups)
};

// Record layout in memory (uint4 units, XS = chunks_per_row | 1), see xquant_kernel:
// [0,6XS) xq, [6XS,7XS) meta, [7XS,9XS) ini.
template <int F, typename P>
__device__ __forceinline__ void load_xq(XQRegs& x, const P* rec, int XS, int c) {
#pragma unroll
  for (int q = 0; q < 6; q++) {
    const uint4 v = rec[q * XS + c];
    x.xw[4 * q] = v.x; x.xw[4 * q + 1] = v.y; x.xw[4 * q + 2] = v.z; x.xw[4 * q + 3] = v.w;
  }
  const uint4 m = rec[6 * XS + c];
  x.mt = make_float4(__uint_as_float(m.x), __uint_as_float(m.y), __uint_as_float(m.z), __uint_as_float(m.w));
#pragma unroll
  for (int i = 0; i < 6; i++) x.iv[i] = 0;
  if constexpr (QCfg<F>::INT_MID) {
    const uint4 a = rec[7 * XS + c], bq = rec[8 * XS + c];
    x.iv[0] = (int)a.x; x.iv[1] = (int)a.y; x.iv[2] = (int)a.z; x.iv[3] = (int)a.w; x.iv[4] = (int)bq.x; x.iv[5] = (int)bq.y;
    if constexpr (!QCfg<F>::HALVES) { x.iv[0] += x.iv[1]; x.iv[2] += x.iv[3]; x.iv[4] += x.iv[5]; }
  }
}

__device__ __forceinline__ int dp4a_su(unsigned a, unsigned b, int c) {
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Block-fixed-point conversion of one 32-column chunk straight into registers (what
// xquant_kernel writes to memory for the register-load kernels). xc points at the chunk's 32
// floats in shared memory. Fully unrolled so that the 24 limb words are built in registers
// with independent dependency chains (the rolled version was latency bound).
template <int F>
__device__ __forceinline__ void quantize_chunk(XQRegs& x, const float* xc) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo;
  float xv[32];
#pragma unroll
  for (int j = 0; j < 32; j++) xv[j] = xc[j];
  float am[4] = {0.f, 0.f, 0.f, 0.f}, pr[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 32; j++) { am[j & 3] = fmaxf(am[j & 3], fabsf(xv[j])); pr[j & 3] = fmaf(xv[j], 0.f, pr[j & 3]); }  // pr: NaN iff any inf / NaN
  const float amax = fmaxf(fmaxf(am[0], am[1]), fmaxf(am[2], am[3]));
  const float probe = (pr[0] + pr[1]) + (pr[2] + pr[3]);
  const unsigned eb = (__float_as_uint(amax) >> 23) & 0xffu;
  float sf = 0.f, inv = 0.f;
  if (probe != 0.f || eb == 255u) sf = __uint_as_float(0x7fc00000u);  // inf / NaN in x: results become NaN
  else if (eb >= 22u) { sf = __uint_as_float((eb - 21u) << 23); inv = __uint_as_float((275u - eb) << 23); }
  int sl[3][2] = {{0, 0}, {0, 0}, {0, 0}};
#pragma unroll
  for (int k = 0; k < 8; k++) {
    int X[4];
    // round to nearest integer through the mantissa of 1.5*2^23 + v (|v| <= 2^22): full-rate
    // FMA + integer subtract instead of the quarter-rate float-to-int conversion
#pragma unroll
    for (int m = 0; m < 4; m++) X[m] = __float_as_int(fmaf(xv[WvLane<BL>::j_of(k, m)], inv, 12582912.0f)) - 0x4B400000;
    const unsigned a01 = __byte_perm(X[0], X[1], 0x6240), a23 = __byte_perm(X[2], X[3], 0x6240);   // {b0,b0',b2,b2'}
    const unsigned w0 = __byte_perm(a01, a23, 0x5410), w2 = __byte_perm(a01, a23, 0x7632);
    const unsigned w1 = __byte_perm(__byte_perm(X[0], X[1], 0x0051), __byte_perm(X[2], X[3], 0x0051), 0x5410);
    x.xw[k] = w0; x.xw[8 + k] = w1; x.xw[16 + k] = w2;
    // 1-bit planes split the halves by byte lane instead of by group; they never need the
    // per-half sums, so everything goes to half 0 for them.
    const int hh = (BL == 1 || k < 4) ? 0 : 1;
    sl[0][hh] = dp4a_uu(w0, 0x01010101u, sl[0][hh]);
    sl[1][hh] = dp4a_uu(w1, 0x01010101u, sl[1][hh]);
    sl[2][hh] = dp4a_su(w2, 0x01010101u, sl[2][hh]);
  }
  const int sx0 = sl[0][0] + (sl[1][0] << 8) + (sl[2][0] << 16), sx1 = sl[0][1] + (sl[1][1] << 8) + (sl[2][1] << 16);
  x.mt = make_float4(sf, sf * (float)(sx0 + sx1), sf * (float)sx0, sf * (float)sx1);
#pragma unroll
  for (int i = 0; i < 6; i++) x.iv[i] = 0;
  if constexpr (QCfg<F>::INT_MID) {
    if constexpr (QCfg<F>::HALVES) {
#pragma unroll
      for (int l = 0; l < 3; l++) { x.iv[l * 2] = -fi.mid * sl[l][0]; x.iv[l * 2 + 1] = -fi.mid * sl[l][1]; }
    } else {
#pragma unroll
      for (int l = 0; l < 3; l++) x.iv[l * 2] = -fi.mid * (sl[l][0] + sl[l][1]);
    }
  }
}

// Contribution of one chunk-row (32 weights of one output row) to that row's sum.
template <int F>
__device__ __forceinline__ float idot_chunk(const FragT<F>& f, const XQRegs& x) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi, SPW = 8 / BL;
  constexpr unsigned MASK = 0x01010101u * ((1u << BL) - 1u);
  constexpr unsigned MASKH = BH ? (0x01010101u * ((1u << BH) - 1u)) << BL : 0u;
  constexpr bool HALVES = QCfg<F>::HALVES;
  constexpr int NH = QCfg<F>::NH;
  // accumulators [limb][half]; the rows a warp processes together supply the independent chains
  int I[3][2];
#pragma unroll
  for (int l = 0; l < 3; l++) { I[l][0] = x.iv[l * 2]; I[l][1] = HALVES ? x.iv[l * 2 + 1] : 0; }
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const int w = k / SPW, sh = k % SPW;
    unsigned bytes = (f.lo[w] >> (BL * sh)) & MASK;
    if constexpr (BH > 0) {
      const int hw = (k * BH) >> 3, hs = (k * BH) & 7;
      unsigned hv = f.hi[hw];
      hv = hs >= BL ? (hv >> (hs - BL)) : (hv << (BL - hs));
      bytes |= hv & MASKH;
    }
    const int h = (HALVES && k >= 4) ? 1 : 0;  // first / second 16 weights of the chunk
    I[0][h] = dp4a_uu(bytes, x.xw[k], I[0][h]);
    I[1][h] = dp4a_uu(bytes, x.xw[8 + k], I[1][h]);
    I[2][h] = dp4a_us(bytes, x.xw[16 + k], I[2][h]);
  }
  // |sum (code - mid) X| <= 15 * 32 * 2^22 < 2^31 for codes of at most 4 bits: recombine the limbs
  // in integer arithmetic and convert once; wider codes recombine in f32.
  constexpr bool SMALL = (BL + BH) <= 4;
  float val[2];
#pragma unroll
  for (int h = 0; h < NH; h++) {
    if constexpr (SMALL) val[h] = (float)(I[0][h] + (I[1][h] << 8) + (I[2][h] << 16));
    else val[h] = fmaf(65536.0f, (float)I[2][h], (float)(I[0][h] + (I[1][h] << 8)));
  }
  const float4 mt = x.mt;
  float v, extra = 0.f;
  if constexpr (fi.kind == WK_KQUANT) {
    // scale bytes were remapped 0 -> 1 at upload (kquant.go:180-182: a zero group scale
    // decodes as d/255), so no test is needed here
    // byte -> float through the conversion unit (one instruction with a byte selector) instead of
    // a byte permute on the integer pipe plus a subtract
    const float t = (float)(unsigned char)(f.pr[2]) * val[0] + (float)(unsigned char)(f.pr[2] >> 8) * val[1];
    v = (__uint_as_float(f.pr[0]) * (1.0f / 255.0f)) * t;
    if constexpr (fi.has_min) {
      const float mm = (float)(signed char)(f.pr[2] >> 16) * mt.z + (float)(signed char)(f.pr[2] >> 24) * mt.w;
      extra = (__uint_as_float(f.pr[1]) * (1.0f / 127.0f)) * mm;
    }
  } else if constexpr (fi.kind == WK_CLASSIC || fi.kind == WK_AFFINE) {
    v = __uint_as_float(f.pr[0]) * val[0];
    if constexpr (fi.has_min) extra = __uint_as_float(f.pr[1]) * mt.y;
  } else if constexpr (fi.kind == WK_TERNARY) {
    v = __uint_as_float(f.pr[0]) * val[0] + __uint_as_float(f.pr[1]) * val[1];
  } else if constexpr (fi.sign) {
    v = __uint_as_float(f.pr[0]) * (2.0f * val[0]);
    extra = -__uint_as_float(f.pr[0]) * mt.y;
  } else {  // IQ linear grids: (code - mid - 0.5)
    constexpr float hm = (float)fi.mid + 0.5f;
    if constexpr (HALVES) {
      v = __uint_as_float(f.pr[0]) * val[0] + __uint_as_float(f.pr[1]) * val[1];
      extra = -hm * (__uint_as_float(f.pr[0]) * mt.z + __uint_as_float(f.pr[1]) * mt.w);
    } else {
      v = __uint_as_float(f.pr[0]) * val[0];
      extra = -hm * __uint_as_float(f.pr[0]) * mt.y;
    }
  }
  return fmaf(mt.x, v, extra);
}

// ------------------------------------------------------------------ two-limb activations (16-bit)
// The default arithmetic of the bulk-copy kernel: per 32-column chunk X_j = rint(x_j * 32512 / amax),
// |X_j| <= 32512, split as X = L0 + 256 L1 with an unsigned low byte and a signed high byte, so a group
// of four codes needs two dp4a instead of three and the limb sums always recombine in 32-bit integers
// (255 * 32 * 32512 < 2^31). Per element |x_j - X_j sf| <= amax / 65024, sf = amax / 32512. A chunk
// whose large values sit next to much smaller ones loses the small ones' low bits; the kernel decides
// per launch, from the whole vector, whether that can matter (see gemv_tma_kernel) and takes the
// three-limb path of quantize_chunk / idot_chunk when it can.
struct XQRegs2 {
  unsigned xw[16];   // word limb*8 + k
  float4 mt;         // {sf, sf*SX(all), sf*SX(first 16), sf*SX(second 16)}
  int iv[4];         // -mid*sum(limb l, half h) at l*2+h (halves pre-added for 32-wide groups)
};

// xv: the chunk's 32 activations (already in registers), amax: their largest magnitude, bad: inf / NaN seen.
template <int F>
__device__ __forceinline__ void quantize_chunk2(XQRegs2& x, const float (&xv)[32], float amax, bool bad) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo;
  float sf = 0.f, inv = 0.f;
  if (bad) sf = __uint_as_float(0x7fc00000u);          // inf / NaN in x: results become NaN
  else if (amax >= 1.0e-30f) { sf = amax * (1.0f / 32512.0f); inv = 32512.0f / amax; }   // |x inv| <= 32512 (1 + 2^-23)
  int sl[2][2] = {{0, 0}, {0, 0}};
#pragma unroll
  for (int k = 0; k < 8; k++) {
    unsigned X[4];
    // the low 23 bits of 1.5*2^23 + rint(v) hold rint(v) in two's complement (|v| < 2^22): bytes 0 and 1
    // are the two limbs as they are, no subtraction needed
#pragma unroll
    for (int m = 0; m < 4; m++) X[m] = __float_as_uint(fmaf(xv[WvLane<BL>::j_of(k, m)], inv, 12582912.0f));
    const unsigned a01 = __byte_perm(X[0], X[1], 0x5140), a23 = __byte_perm(X[2], X[3], 0x5140);   // {b0,b0',b1,b1'}
    const unsigned w0 = __byte_perm(a01, a23, 0x5410), w1 = __byte_perm(a01, a23, 0x7632);
    x.xw[k] = w0; x.xw[8 + k] = w1;
    const int hh = (BL == 1 || k < 4) ? 0 : 1;   // 1-bit planes split the halves by byte lane: everything in half 0
    sl[0][hh] = dp4a_uu(w0, 0x01010101u, sl[0][hh]);
    sl[1][hh] = dp4a_su(w1, 0x01010101u, sl[1][hh]);
  }
  const int sx0 = sl[0][0] + (sl[1][0] << 8), sx1 = sl[0][1] + (sl[1][1] << 8);
  x.mt = make_float4(sf, sf * (float)(sx0 + sx1), sf * (float)sx0, sf * (float)sx1);
#pragma unroll
  for (int i = 0; i < 4; i++) x.iv[i] = 0;
  if constexpr (QCfg<F>::INT_MID) {
    if constexpr (QCfg<F>::HALVES) {
#pragma unroll
      for (int l = 0; l < 2; l++) { x.iv[l * 2] = -fi.mid * sl[l][0]; x.iv[l * 2 + 1] = -fi.mid * sl[l][1]; }
    } else {
#pragma unroll
      for (int l = 0; l < 2; l++) x.iv[l * 2] = -fi.mid * (sl[l][0] + sl[l][1]);
    }
  }
}

// Integer sums of one chunk-row per parameter half; the common tail below turns them into the row's share.
template <int F>
__device__ __forceinline__ void idot_sums2(const FragT<F>& f, const XQRegs2& x, float (&val)[2]) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi, SPW = 8 / BL;
  constexpr unsigned MASK = 0x01010101u * ((1u << BL) - 1u);
  constexpr unsigned MASKH = BH ? (0x01010101u * ((1u << BH) - 1u)) << BL : 0u;
  constexpr bool HALVES = QCfg<F>::HALVES;
  constexpr int NH = QCfg<F>::NH;
  int I[2][2];
#pragma unroll
  for (int l = 0; l < 2; l++) { I[l][0] = x.iv[l * 2]; I[l][1] = HALVES ? x.iv[l * 2 + 1] : 0; }
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const int w = k / SPW, sh = k % SPW;
    unsigned bytes = (f.lo[w] >> (BL * sh)) & MASK;
    if constexpr (BH > 0) {
      const int hw = (k * BH) >> 3, hs = (k * BH) & 7;
      unsigned hv = f.hi[hw];
      hv = hs >= BL ? (hv >> (hs - BL)) : (hv << (BL - hs));
      bytes |= hv & MASKH;
    }
    const int h = (HALVES && k >= 4) ? 1 : 0;
    I[0][h] = dp4a_uu(bytes, x.xw[k], I[0][h]);
    I[1][h] = dp4a_us(bytes, x.xw[8 + k], I[1][h]);
  }
#pragma unroll
  for (int h = 0; h < NH; h++) val[h] = (float)(I[0][h] + (I[1][h] << 8));
}

// Scale / min arithmetic shared by the two- and three-limb paths: val[h] = sum over half h of
// (code - mid) * X, mt = {sf, sf*SX, sf*SX(first 16), sf*SX(second 16)}.
template <int F>
__device__ __forceinline__ float idot_finish(const FragT<F>& f, const float (&val)[2], const float4 mt) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr bool HALVES = QCfg<F>::HALVES;
  float v, extra = 0.f;
  if constexpr (fi.kind == WK_KQUANT) {
    // scale bytes were remapped 0 -> 1 at upload (kquant.go:180-182: a zero group scale decodes as d/255)
    const float t = (float)(unsigned char)(f.pr[2]) * val[0] + (float)(unsigned char)(f.pr[2] >> 8) * val[1];
    v = (__uint_as_float(f.pr[0]) * (1.0f / 255.0f)) * t;
    if constexpr (fi.has_min) {
      const float mm = (float)(signed char)(f.pr[2] >> 16) * mt.z + (float)(signed char)(f.pr[2] >> 24) * mt.w;
      extra = (__uint_as_float(f.pr[1]) * (1.0f / 127.0f)) * mm;
    }
  } else if constexpr (fi.kind == WK_CLASSIC || fi.kind == WK_AFFINE) {
    v = __uint_as_float(f.pr[0]) * val[0];
    if constexpr (fi.has_min) extra = __uint_as_float(f.pr[1]) * mt.y;
  } else if constexpr (fi.kind == WK_TERNARY) {
    v = __uint_as_float(f.pr[0]) * val[0] + __uint_as_float(f.pr[1]) * val[1];
  } else if constexpr (fi.sign) {
    v = __uint_as_float(f.pr[0]) * (2.0f * val[0]);
    extra = -__uint_as_float(f.pr[0]) * mt.y;
  } else {  // IQ linear grids: (code - mid - 0.5)
    constexpr float hm = (float)fi.mid + 0.5f;
    if constexpr (HALVES) {
      v = __uint_as_float(f.pr[0]) * val[0] + __uint_as_float(f.pr[1]) * val[1];
      extra = -hm * (__uint_as_float(f.pr[0]) * mt.z + __uint_as_float(f.pr[1]) * mt.w);
    } else {
      v = __uint_as_float(f.pr[0]) * val[0];
      extra = -hm * __uint_as_float(f.pr[0]) * mt.y;
    }
  }
  return fmaf(mt.x, v, extra);
}

template <int F>
__device__ __forceinline__ float idot_chunk2(const FragT<F>& f, const XQRegs2& x) {
  float val[2] = {0.f, 0.f};
  idot_sums2<F>(f, x, val);
  return idot_finish<F>(f, val, x.mt);
}
// One name for both activation widths (the kernel's main loop is instantiated once per width).
template <int F> __device__ __forceinline__ float idot_any(const FragT<F>& f, const XQRegs& x) { return idot_chunk<F>(f, x); }
template <int F> __device__ __forceinline__ float idot_any(const FragT<F>& f, const XQRegs2& x) { return idot_chunk2<F>(f, x); }

// Launch with programmatic dependent launch allowed: the kernel may start while its
// predecessor drains and must execute griddepcontrol.wait before touching dependent data.
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// Output vectors of a row-sharded GEMV: with n > 0 every output row is stored into each of the n
// vectors (this GPU's own and its peers' mapped ones) instead of into y, so that every rank ends
// up with the whole result without a collective call.
#define WV_MAX_PEERS 8
struct WvPeers {
  float* y[WV_MAX_PEERS];
  int n;
  int self;   // index of this GPU's own vector (host side only)
};
// Set by wv_matvec_dev_gather around its launch (wv_api.cu); the bulk-copy kernels pass it on.
extern thread_local const WvPeers* wv_cur_peers;

// Fused epilogues of the grouped bulk-copy launch, set by the fused entry points around their launch:
// the SwiGLU gate product, a residual add, and per-matrix output vectors on every rank.
struct WvFuse {
  int mode;                 // 0: y_i = W_i x;  1: h = silu(W_0 x) * (W_1 x), stored as output 1
  const float* residual;    // one matrix: y = W x + residual
  int npeers;               // > 0: rows go to py[matrix][rank] (own and peers' vectors, already offset to this rank's rows)
  float* py[4][WV_MAX_PEERS];
  const float* norm_gamma;  // non-null: x is RMS-normalised on its way in, x_j <- x_j / sqrt(mean(x^2) + eps) * gamma_j
  double norm_eps;
};
extern thread_local const WvFuse* wv_cur_fuse;

// wv_gemv.cu
uint4* wv_scratch_take(size_t bytes);
int wv_launch_xquant(int bits_lo, const float* dx, int cols, int batch, int imid, uint4* out, cudaStream_t st);
int wv_sm_count();
// wv_gemv_tma.cu: returns WV_OK, an error, or 1 when the shape does not fit the TMA kernel
int wv_launch_gemv_tma(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st);
int wv_launch_gemv_tma_group(const WvDevBlob* b, int nb, const float* dx, float* const* dy, int batch, int row_begin, int row_end, cudaStream_t st);
// wv_gemv_tc.cu: same contract (all packed integer-code formats, tensor-pipe dot products)
int wv_launch_gemv_tc(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st);
// wv_gemv_mma.cu: same contract; pw = chunk pairs per warp per tile (1, 2, 4)
int wv_launch_gemv_mma(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st, int pw);
