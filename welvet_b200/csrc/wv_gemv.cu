// Fused dequantise-and-dot GEMV for sm_100a: y = W x with W resident in the bit-plane
// layout of wv_common.cuh. Replaces the reference's row-parallel SIMD drivers
// (layers/dense/gemv_parallel.go:12-391 over simd.Dot*Row) and its one-thread-per-row WGSL
// shaders (webgpu/dense_shaders_extra.go) for batch-1 decode.
//
// The kernel is HBM-bound by design (2 flop per 0.16..4 bytes): no tensor cores.
//   * persistent grid, one CTA per SM; every CTA stages x once into shared memory in a
//     lane-friendly permutation plus per-16-column sums of x (for the min / mid terms);
//   * a warp (or a team of S warps splitting the columns) owns R output rows at a time and
//     walks the row in 32-weight chunks, one chunk per lane per step: 128-bit coalesced
//     loads of the code planes straight into registers, D steps prefetched ahead;
//   * codes become floats with one byte-permute each (2^23 + code) and an exact subtract,
//     products accumulate in f32 with packed f32x2 FMAs; asymmetric formats use the
//     reference's own factorisation sc*sum(q*x) + mn*sum(x) (simd/dot_k.go:44-53);
//   * warp-shuffle reduction, one store per row.
#include "wv_common.cuh"
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#ifndef WV_GEMV_THREADS
#define WV_GEMV_THREADS 512
#endif

__constant__ float c_grid4nl[16] = WV_IQ4NL_GRID;

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

// ------------------------------------------------------------------ shared-memory x
// x permutation for lo-plane width B: column 32c + j lives at float ((k*XS + c)*4 + m).
template <int B> __device__ __forceinline__ int x_slot(int col, int XS) {
  const int c = col >> 5, j = col & 31;
  return ((WvLane<B>::k_of(j) * XS + c) << 2) + WvLane<B>::m_of(j);
}

template <int F, int R, int S, int D>
__global__ void __launch_bounds__(WV_GEMV_THREADS, 1)
gemv_chunked_kernel(const WvDevBlob b, const float* __restrict__ x, float* __restrict__ y, int row_begin, int row_end) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo;
  constexpr int NW = WV_GEMV_THREADS / 32, T = NW / S;
  constexpr bool NEED_SX = fi.has_min || fi.sign || fi.half_mid;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int cpr = b.cols >> 5;  // chunks per row
  const int XS = cpr | 1;       // odd stride (in float4) keeps the permuting stores conflict free
  float4* xs4 = reinterpret_cast<float4*>(smem_raw);
  float2* sxs = reinterpret_cast<float2*>(xs4 + 8 * XS);
  float* tbl = reinterpret_cast<float*>(sxs + cpr);
  float* team = tbl + (fi.table ? 512 : 0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tm = warp / S, sid = warp % S;
  const int nrows = row_end - row_begin;
  const int G = (nrows + R - 1) / R;
  const int g_lo = (int)(((long long)blockIdx.x * G) / gridDim.x), g_hi = (int)(((long long)(blockIdx.x + 1) * G) / gridDim.x);
  const int iters = (cpr + 32 * S - 1) / (32 * S);
  const float* xb = x + (size_t)blockIdx.y * b.cols;
  float* yb = y + (size_t)blockIdx.y * b.rows;

  // prefetch cursor and first D steps: weights do not depend on the previous kernel
  FragT<F> buf[D][R];
  int pg = g_lo + tm, pit = 0;
  auto issue = [&](FragT<F> (&dst)[R]) {
    if (pg < g_hi) {
      const int c = (pit * S + sid) * 32 + lane;
      if (c < cpr) {
#pragma unroll
        for (int r = 0; r < R; r++) {
          int row = pg * R + r; row = row < nrows ? row : nrows - 1;
          load_frag<F>(dst[r], b, (long long)(row_begin + row) * cpr + c);
        }
      }
      if (++pit == iters) { pit = 0; pg += T; }
    }
  };
#pragma unroll
  for (int d = 0; d < D; d++) issue(buf[d]);

  // stage x (permuted) and the per-16 sums of x
  for (int col = tid; col < b.cols; col += WV_GEMV_THREADS) reinterpret_cast<float*>(xs4)[x_slot<BL>(col, XS)] = xb[col];
  if constexpr (fi.table) for (int i = tid; i < 512; i += WV_GEMV_THREADS) tbl[i] = c_grid4nl[i >> 5];
  __syncthreads();
  if constexpr (NEED_SX) {
    for (int c = tid; c < cpr; c += WV_GEMV_THREADS) {
      float a = 0.f, bsum = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j++) a += reinterpret_cast<float*>(xs4)[x_slot<BL>(c * 32 + j, XS)];
#pragma unroll
      for (int j = 16; j < 32; j++) bsum += reinterpret_cast<float*>(xs4)[x_slot<BL>(c * 32 + j, XS)];
      sxs[c] = make_float2(a, bsum);
    }
    __syncthreads();
  }

  float acc[R];
#pragma unroll
  for (int r = 0; r < R; r++) acc[r] = 0.f;
  int cg = g_lo + tm, cit = 0, parity = 0;
  const int nsteps = cg < g_hi ? ((g_hi - cg + T - 1) / T) * iters : 0;
  for (int s = 0; s < nsteps; s += D) {
#pragma unroll
    for (int d = 0; d < D; d++) {
      if (s + d < nsteps) {
        FragT<F> cur[R];
#pragma unroll
        for (int r = 0; r < R; r++) cur[r] = buf[d][r];
        issue(buf[d]);
        const int c = (cit * S + sid) * 32 + lane;
        if (c < cpr) {
          float4 xr[8];
#pragma unroll
          for (int k = 0; k < 8; k++) xr[k] = xs4[k * XS + c];
          float2 sx = make_float2(0.f, 0.f);
          if constexpr (NEED_SX) sx = sxs[c];
#pragma unroll
          for (int r = 0; r < R; r++) acc[r] += chunk_value<F>(cur[r], xr, sx, tbl + lane);
        }
        if (++cit == iters) {
#pragma unroll
          for (int r = 0; r < R; r++) {
#pragma unroll
            for (int o = 16; o; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
          }
          if constexpr (S > 1) {
            float* slot = team + ((parity * T + tm) * S) * R;
            if (sid > 0 && lane == 0) {
#pragma unroll
              for (int r = 0; r < R; r++) slot[sid * R + r] = acc[r];
            }
            asm volatile("bar.sync %0, %1;" ::"r"(tm + 1), "r"(32 * S) : "memory");
            if (sid == 0) {
#pragma unroll
              for (int q = 1; q < S; q++) {
#pragma unroll
                for (int r = 0; r < R; r++) acc[r] += slot[q * R + r];
              }
            }
            parity ^= 1;
          }
          if (sid == 0 && lane == 0) {
#pragma unroll
            for (int r = 0; r < R; r++) {
              const int row = cg * R + r;
              if (row < nrows) yb[row_begin + row] = acc[r];
            }
          }
#pragma unroll
          for (int r = 0; r < R; r++) acc[r] = 0.f;
          cit = 0; cg += T;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ FormatNone f32 / f16 / bf16
// Plain streaming GEMV: warp per R rows, lanes read consecutive 16-byte pieces.
template <int DT, int R>
__global__ void __launch_bounds__(WV_GEMV_THREADS, 1)
gemv_dense_kernel(const WvDevBlob b, const float* __restrict__ x, float* __restrict__ y, int row_begin, int row_end) {
  constexpr int EPV = DT == WV_DT_F32 ? 4 : 8;  // elements per 16-byte vector
  constexpr int NW = WV_GEMV_THREADS / 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* xb = x + (size_t)blockIdx.y * b.cols;
  float* yb = y + (size_t)blockIdx.y * b.rows;
  for (int c = tid; c < b.cols; c += WV_GEMV_THREADS) xs[c] = xb[c];
  __syncthreads();
  const int nrows = row_end - row_begin, G = (nrows + R - 1) / R;
  const int g_lo = (int)(((long long)blockIdx.x * G) / gridDim.x), g_hi = (int)(((long long)(blockIdx.x + 1) * G) / gridDim.x);
  const int vpr = b.cols / EPV;
  const uint4* wbase = reinterpret_cast<const uint4*>(b.lo);
  for (int g = g_lo + warp; g < g_hi; g += NW) {
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = 0.f;
    for (int v0 = 0; v0 < vpr; v0 += 64) {
      uint4 wv[2][R];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int v = v0 + u * 32 + lane;
#pragma unroll
        for (int r = 0; r < R; r++) {
          int row = g * R + r; row = row < nrows ? row : nrows - 1;
          wv[u][r] = v < vpr ? __ldg(wbase + (size_t)(row_begin + row) * vpr + v) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int v = v0 + u * 32 + lane;
        if (v < vpr) {
          const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)v * EPV);
          const float4 xa = xp[0];
          float4 xc = make_float4(0, 0, 0, 0);
          if constexpr (EPV == 8) xc = xp[1];
#pragma unroll
          for (int r = 0; r < R; r++) {
            const uint4 q = wv[u][r];
            if constexpr (DT == WV_DT_F32) {
              acc[r] = fmaf(__uint_as_float(q.x), xa.x, acc[r]); acc[r] = fmaf(__uint_as_float(q.y), xa.y, acc[r]);
              acc[r] = fmaf(__uint_as_float(q.z), xa.z, acc[r]); acc[r] = fmaf(__uint_as_float(q.w), xa.w, acc[r]);
            } else {
              const unsigned ws[4] = {q.x, q.y, q.z, q.w};
              const float xe[8] = {xa.x, xa.y, xa.z, xa.w, xc.x, xc.y, xc.z, xc.w};
#pragma unroll
              for (int i = 0; i < 4; i++) {
                float f0, f1;
                if constexpr (DT == WV_DT_BF16) { f0 = __uint_as_float(ws[i] << 16); f1 = __uint_as_float(ws[i] & 0xffff0000u); }
                else {
                  f0 = __half2float(__ushort_as_half((unsigned short)(ws[i] & 0xffffu)));
                  f1 = __half2float(__ushort_as_half((unsigned short)(ws[i] >> 16)));
                }
                acc[r] = fmaf(f0, xe[2 * i], acc[r]); acc[r] = fmaf(f1, xe[2 * i + 1], acc[r]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
#pragma unroll
      for (int o = 16; o; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
      const int row = g * R + r;
      if (lane == 0 && row < nrows) yb[row_begin + row] = acc[r];
    }
  }
}

// ------------------------------------------------------------------ dispatch
int wv_launch_gemv_ragged(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st);

static int g_sm_count = 0;
static int sm_count() {
  if (!g_sm_count) {
    int dev = 0; cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

// Tuning knobs (rows per warp, column split, prefetch depth) can be overridden for
// experiments through wv_set_tuning(); 0 keeps the built-in choice.
static int g_tune_r = 0, g_tune_s = 0, g_tune_d = 0, g_tune_grid = 0;
extern "C" void wv_set_tuning(int r, int s, int d, int grid) { g_tune_r = r; g_tune_s = s; g_tune_d = d; g_tune_grid = grid; }

template <int F, int R, int S, int D>
static int launch_chunked(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb, int re, cudaStream_t st) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  const int cpr = b.cols >> 5, XS = cpr | 1;
  constexpr int NW = WV_GEMV_THREADS / 32, T = NW / S;
  size_t smem = (size_t)8 * XS * 16 + (size_t)cpr * 8 + (fi.table ? 2048 : 0) + (size_t)2 * T * S * R * 4 + 16;
  if (smem > 227 * 1024) return WV_ESHAPE;
  static bool attr_set = false;
  auto kern = gemv_chunked_kernel<F, R, S, D>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) return WV_ECUDA;
    attr_set = true;
  }
  int grid = g_tune_grid > 0 ? g_tune_grid : sm_count();
  const int G = (re - rb + R - 1) / R;
  if (grid > G) grid = G;
  if (grid < 1) grid = 1;
  kern<<<dim3(grid, batch), WV_GEMV_THREADS, smem, st>>>(b, dx, dy, rb, re);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}

template <int F>
static int launch_format(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb, int re, cudaStream_t st) {
  // Default shape heuristic: few long rows -> split columns over 2 warps; many short rows -> 4 rows per warp.
  int R = g_tune_r, S = g_tune_s, D = g_tune_d;
  const int nrows = re - rb;
  const long long warp_slots = (long long)sm_count() * (WV_GEMV_THREADS / 32);
  if (!R) R = (nrows / 4 >= warp_slots / 2) ? 4 : 2;
  if (!S) S = (nrows / R < warp_slots / 2 && (b.cols >> 5) >= 64) ? 2 : 1;
  if (!D) D = 2;
#define WV_CASE(r, s, d) if (R == r && S == s && D == d) return launch_chunked<F, r, s, d>(b, dx, dy, batch, rb, re, st);
  WV_CASE(2, 1, 2) WV_CASE(2, 2, 2) WV_CASE(4, 1, 2) WV_CASE(4, 2, 2)
  WV_CASE(2, 1, 4) WV_CASE(2, 2, 4) WV_CASE(1, 2, 4) WV_CASE(1, 4, 4)
#undef WV_CASE
  return launch_chunked<F, 2, 1, 2>(b, dx, dy, batch, rb, re, st);
}

template <int DT>
static int launch_dense(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb, int re, cudaStream_t st) {
  size_t smem = (size_t)b.cols * 4 + 16;
  if (smem > 227 * 1024) return WV_ESHAPE;
  static bool attr_set = false;
  auto kern = gemv_dense_kernel<DT, 2>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) return WV_ECUDA;
    attr_set = true;
  }
  int grid = g_tune_grid > 0 ? g_tune_grid : sm_count();
  const int G = (re - rb + 1) / 2;
  if (grid > G) grid = G;
  if (grid < 1) grid = 1;
  kern<<<dim3(grid, batch), WV_GEMV_THREADS, smem, st>>>(b, dx, dy, rb, re);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}

int wv_launch_gemv(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st) {
  if (row_end <= row_begin || batch <= 0) return WV_OK;
  if (!b.fast) return wv_launch_gemv_ragged(b, dx, dy, batch, row_begin, row_end, st);
  switch (b.format) {
  case WV_NONE:
    if (b.dtype == WV_DT_F32) return launch_dense<WV_DT_F32>(b, dx, dy, batch, row_begin, row_end, st);
    if (b.dtype == WV_DT_F16) return launch_dense<WV_DT_F16>(b, dx, dy, batch, row_begin, row_end, st);
    return launch_dense<WV_DT_BF16>(b, dx, dy, batch, row_begin, row_end, st);
#define WV_F(f) case f: return launch_format<f>(b, dx, dy, batch, row_begin, row_end, st);
  WV_F(WV_Q8_0) WV_F(WV_Q4_0) WV_F(WV_Q4_1) WV_F(WV_Q5_0) WV_F(WV_Q5_1)
  WV_F(WV_Q2_K) WV_F(WV_Q3_K) WV_F(WV_Q4_K) WV_F(WV_Q5_K) WV_F(WV_Q6_K)
  WV_F(WV_IQ1_S) WV_F(WV_IQ2_XXS) WV_F(WV_IQ2_XS) WV_F(WV_IQ3_XXS) WV_F(WV_IQ3_S) WV_F(WV_IQ4_NL) WV_F(WV_IQ4_XS)
  WV_F(WV_TERNARY) WV_F(WV_BINARY) WV_F(WV_AFFINE)
#undef WV_F
  }
  return WV_EFORMAT;
}
