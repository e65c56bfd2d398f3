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
#include "wv_gemv_common.cuh"
#include "wv_dev_hooks.h"
#include <stdlib.h>
#include <cstdlib>
#include <mutex>

#ifndef WV_GEMV_THREADS
#define WV_GEMV_THREADS 512
#endif

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

// ------------------------------------------------------------------ activation pre-quantisation
// Activation record, identical in the global scratch written by xquant_kernel and in the
// shared-memory copy every GEMV CTA makes of it (uint4 units, XS = chunks_per_row | 1):
//   [0 , 6XS)   xq    24 int8x4 words per chunk, word t = limb*8 + k at uint4 (t>>2)*XS + c
//   [6XS, 7XS)  meta  float4 {sf, sf*SX(all 32), sf*SX(first 16), sf*SX(second 16)}
//   [7XS, 9XS)  ini   -mid * sum(limb l over half h), int (l*2+h) at int4 ((l*2+h)>>2)*XS + c
//                     (only read by formats with an exact integer offset)
// One thread converts one 32-column chunk; launched once per GEMV call, so the per-CTA
// prologue of the GEMV is a plain 16-byte-vector copy.
template <int BL>
__global__ void __launch_bounds__(128) xquant_kernel(const float* __restrict__ x, int cols, int imid, uint4* __restrict__ out) {
  asm volatile("griddepcontrol.wait;" ::: "memory");            // x may be the previous kernel's output
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int cpr = cols >> 5, XS = cpr | 1;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cpr) return;
  const float* xp = x + (size_t)blockIdx.y * cols + (size_t)c * 32;
  uint4* o = out + (size_t)blockIdx.y * 9 * XS;
  float xv[32];
  if ((reinterpret_cast<uintptr_t>(xp) & 15) == 0) {
#pragma unroll
    for (int q = 0; q < 8; q++) { const float4 v = __ldg(reinterpret_cast<const float4*>(xp) + q); xv[4 * q] = v.x; xv[4 * q + 1] = v.y; xv[4 * q + 2] = v.z; xv[4 * q + 3] = v.w; }
  } else {
#pragma unroll
    for (int j = 0; j < 32; j++) xv[j] = __ldg(xp + j);
  }
  float amax = 0.f;
  bool bad = false;
#pragma unroll
  for (int j = 0; j < 32; j++) { amax = fmaxf(amax, fabsf(xv[j])); bad |= !(fabsf(xv[j]) <= 3.4028234e38f); }
  const unsigned eb = (__float_as_uint(amax) >> 23) & 0xffu;
  float sf = 0.f, inv = 0.f;
  if (bad) sf = __uint_as_float(0x7fc00000u);  // inf / NaN in x: the row results become NaN
  else if (eb >= 22u) { sf = __uint_as_float((eb - 21u) << 23); inv = __uint_as_float((275u - eb) << 23); }
  unsigned wd[24];
#pragma unroll
  for (int t = 0; t < 24; t++) wd[t] = 0u;
  int sx[2] = {0, 0}, sl[3][2] = {{0, 0}, {0, 0}, {0, 0}};
#pragma unroll
  for (int j = 0; j < 32; j++) {
    const int k = WvLane<BL>::k_of(j), m = WvLane<BL>::m_of(j), h = j >> 4;
    const int X = __float2int_rn(xv[j] * inv);
    const int L0 = X & 0xff, L1 = (X >> 8) & 0xff, L2 = X >> 16;
    wd[k] |= (unsigned)L0 << (8 * m);
    wd[8 + k] |= (unsigned)L1 << (8 * m);
    wd[16 + k] |= (unsigned)(L2 & 0xff) << (8 * m);
    sx[h] += X; sl[0][h] += L0; sl[1][h] += L1; sl[2][h] += L2;
  }
#pragma unroll
  for (int q = 0; q < 6; q++) o[q * XS + c] = make_uint4(wd[4 * q], wd[4 * q + 1], wd[4 * q + 2], wd[4 * q + 3]);
  const float4 mt = make_float4(sf, sf * (float)(sx[0] + sx[1]), sf * (float)sx[0], sf * (float)sx[1]);
  o[6 * XS + c] = make_uint4(__float_as_uint(mt.x), __float_as_uint(mt.y), __float_as_uint(mt.z), __float_as_uint(mt.w));
  o[7 * XS + c] = make_uint4((unsigned)(-imid * sl[0][0]), (unsigned)(-imid * sl[0][1]), (unsigned)(-imid * sl[1][0]), (unsigned)(-imid * sl[1][1]));
  o[8 * XS + c] = make_uint4((unsigned)(-imid * sl[2][0]), (unsigned)(-imid * sl[2][1]), 0u, 0u);
}

// ------------------------------------------------------------------ integer-dot kernel (register loads)
// Work split: CTA b owns rows [n*b/grid, n*(b+1)/grid); inside the CTA, team t (S warps that
// split the columns) owns an equal contiguous share of those rows and walks it R rows at a
// time, one 32-weight chunk per lane per step, D steps of weight loads in flight.
// Used for shapes the TMA-fed kernel (wv_gemv_tma.cu) does not take.
template <int F, int R, int S, int D>
__global__ void __launch_bounds__(WV_GEMV_THREADS, 1)
gemv_idot_kernel(const WvDevBlob b, const uint4* __restrict__ xqg, float* __restrict__ y, int row_begin, int row_end) {
  constexpr int NW = WV_GEMV_THREADS / 32, T = NW / S;
  constexpr int NREC = QCfg<F>::NREC;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int cpr = b.cols >> 5;
  const int XS = cpr | 1;
  uint4* xq = reinterpret_cast<uint4*>(smem_raw);
  float* team = reinterpret_cast<float*>(xq + NREC * XS);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tm = warp / S, sid = warp % S;
  const int nrows = row_end - row_begin;
  const int c_lo = (int)(((long long)blockIdx.x * nrows) / gridDim.x), c_hi = (int)(((long long)(blockIdx.x + 1) * nrows) / gridDim.x);
  const int r_lo = c_lo + (int)(((long long)tm * (c_hi - c_lo)) / T), r_hi = c_lo + (int)(((long long)(tm + 1) * (c_hi - c_lo)) / T);
  const int iters = (cpr + 32 * S - 1) / (32 * S);
  const int nsteps = ((r_hi - r_lo + R - 1) / R) * iters;
  float* yb = y + (size_t)blockIdx.y * b.rows + row_begin;
  const long long cbase = (long long)row_begin * cpr;

  // weights do not depend on the preceding kernel: start streaming them before waiting for x
  FragT<F> buf[D][R];
  int prow = r_lo, pit = 0, pleft = nsteps;
  auto issue = [&](FragT<F> (&dst)[R]) {
    if (pleft > 0) {
      const int c = (pit * S + sid) * 32 + lane;
      if (c < cpr) {
#pragma unroll
        for (int r = 0; r < R; r++) {
          const int row = min(prow + r, r_hi - 1);
          load_frag<F>(dst[r], b, cbase + (long long)row * cpr + c);
        }
      }
      --pleft;
      if (++pit == iters) { pit = 0; prow += R; }
    }
  };
#pragma unroll
  for (int d = 0; d < D; d++) issue(buf[d]);

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  {
    const uint4* src = xqg + (size_t)blockIdx.y * 9 * XS;
    for (int i = tid; i < NREC * XS; i += WV_GEMV_THREADS) xq[i] = src[i];
  }
  __syncthreads();

  float acc[R];
#pragma unroll
  for (int r = 0; r < R; r++) acc[r] = 0.f;
  int crow = r_lo, cit = 0, parity = 0;
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
          XQRegs xr;
          load_xq<F>(xr, xq, XS, c);
#pragma unroll
          for (int r = 0; r < R; r++) acc[r] += idot_chunk<F>(cur[r], xr);
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
            for (int r = 0; r < R; r++) if (crow + r < r_hi) yb[crow + r] = acc[r];
          }
#pragma unroll
          for (int r = 0; r < R; r++) acc[r] = 0.f;
          cit = 0; crow += R;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ FormatNone f32 / f16 / bf16
// Plain streaming GEMV (the reference's DotTile / DotF16Packed / DotBF16Packed rows,
// layers/dense/simd.go:201-284): two 512-thread CTAs per SM, a warp owns whole rows, lanes
// read consecutive 16-byte vectors, U vectors per lane per step with the next step's loads
// issued before the current step's arithmetic (2*U*512 bytes per warp in flight).
#define WV_DENSE_THREADS 512
template <int DT, int U>
__global__ void __launch_bounds__(WV_DENSE_THREADS, 2)
gemv_dense_kernel(const WvDevBlob b, const float* __restrict__ x, float* __restrict__ y, int row_begin, int row_end) {
  constexpr int EPV = DT == WV_DT_F32 ? 4 : 8;  // elements per 16-byte vector
  constexpr int NW = WV_DENSE_THREADS / 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* xb = x + (size_t)blockIdx.y * b.cols;
  float* yb = y + (size_t)blockIdx.y * b.rows + row_begin;
  const int nrows = row_end - row_begin;
  const int c_lo = (int)(((long long)blockIdx.x * nrows) / gridDim.x), c_hi = (int)(((long long)(blockIdx.x + 1) * nrows) / gridDim.x);
  const int r_lo = c_lo + (int)(((long long)warp * (c_hi - c_lo)) / NW), r_hi = c_lo + (int)(((long long)(warp + 1) * (c_hi - c_lo)) / NW);
  const int vpr = b.cols / EPV;
  const int steps_per_row = (vpr + 32 * U - 1) / (32 * U);
  const int nsteps = (r_hi - r_lo) * steps_per_row;
  const uint4* wbase = reinterpret_cast<const uint4*>(b.lo) + (size_t)row_begin * vpr;
  auto load_step = [&](uint4 (&w)[U], int step) {
    const int row = r_lo + step / steps_per_row, v0 = (step % steps_per_row) * 32 * U;
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int v = v0 + u * 32 + lane;
      w[u] = (step < nsteps && v < vpr) ? __ldg(wbase + (size_t)row * vpr + v) : make_uint4(0, 0, 0, 0);
    }
  };
  uint4 nxt[U];
  load_step(nxt, 0);   // weights do not depend on the previous kernel
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int c = tid; c < b.cols; c += WV_DENSE_THREADS) xs[c] = xb[c];
  __syncthreads();
  float acc = 0.f;
  for (int step = 0; step < nsteps; step++) {
    uint4 cur[U];
#pragma unroll
    for (int u = 0; u < U; u++) cur[u] = nxt[u];
    load_step(nxt, step + 1);
    const int v0 = (step % steps_per_row) * 32 * U;
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int v = v0 + u * 32 + lane;
      if (v < vpr) {
        const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)v * EPV);
        const float4 xa = xp[0];
        const uint4 q = cur[u];
        if constexpr (DT == WV_DT_F32) {
          acc = fmaf(__uint_as_float(q.x), xa.x, acc); acc = fmaf(__uint_as_float(q.y), xa.y, acc);
          acc = fmaf(__uint_as_float(q.z), xa.z, acc); acc = fmaf(__uint_as_float(q.w), xa.w, acc);
        } else {
          const float4 xc = xp[1];
          const unsigned ws[4] = {q.x, q.y, q.z, q.w};
          const float xe[8] = {xa.x, xa.y, xa.z, xa.w, xc.x, xc.y, xc.z, xc.w};
#pragma unroll
          for (int i = 0; i < 4; i++) {
            float f0, f1;
            if constexpr (DT == WV_DT_BF16) { f0 = __uint_as_float(ws[i] << 16); f1 = __uint_as_float(ws[i] & 0xffff0000u); }
            else {
              const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&ws[i]));
              f0 = hf.x; f1 = hf.y;
            }
            acc = fmaf(f0, xe[2 * i], acc); acc = fmaf(f1, xe[2 * i + 1], acc);
          }
        }
      }
    }
    if ((step + 1) % steps_per_row == 0) {
#pragma unroll
      for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) yb[r_lo + step / steps_per_row] = acc;
      acc = 0.f;
    }
  }
}

// ------------------------------------------------------------------ dispatch
int wv_launch_gemv_ragged(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st);

static int g_sm_count = 0;
int wv_sm_count();
static int sm_count() { return wv_sm_count(); }
int wv_sm_count() {
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
#ifdef WV_DEV_HOOKS
extern "C" void wv_set_tuning(int r, int s, int d, int grid) { g_tune_r = r; g_tune_s = s; g_tune_d = d; g_tune_grid = grid; }
#endif

// Scratch arena for quantised activations: a ring of slots, one per GEMV call. A slot is
// reused only after the ring wraps, i.e. after (arena / slot) further calls.
static uint4* g_xq_arena = nullptr;
static size_t g_xq_bytes = 0, g_xq_head = 0;
static std::mutex g_xq_mu;   // host threads may launch concurrently: the ring head moves under a lock
int wv_gemv_scratch_init(size_t bytes) {
  if (g_xq_arena) return WV_OK;
  if (cudaMalloc(&g_xq_arena, bytes) != cudaSuccess) { cudaGetLastError(); return WV_ENOMEM; }
  g_xq_bytes = bytes; g_xq_head = 0;
  return WV_OK;
}
uint4* wv_scratch_take(size_t bytes) {
  bytes = (bytes + 255) & ~(size_t)255;
  std::lock_guard<std::mutex> lk(g_xq_mu);
  if (!g_xq_arena || bytes > g_xq_bytes) return nullptr;
  if (g_xq_head + bytes > g_xq_bytes) g_xq_head = 0;
  uint4* p = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(g_xq_arena) + g_xq_head);
  g_xq_head += bytes;
  return p;
}

template <int BL>
static int launch_xquant(const float* dx, int cols, int batch, int imid, uint4* out, cudaStream_t st) {
  const int cpr = cols >> 5;
  cudaError_t e = launch_pdl(xquant_kernel<BL>, dim3((cpr + 127) / 128, batch), dim3(128), 0, st, dx, cols, imid, out);
  return e == cudaSuccess ? WV_OK : WV_ECUDA;
}
int wv_launch_xquant(int bits_lo, const float* dx, int cols, int batch, int imid, uint4* out, cudaStream_t st) {
  switch (bits_lo) {
  case 1: return launch_xquant<1>(dx, cols, batch, imid, out, st);
  case 2: return launch_xquant<2>(dx, cols, batch, imid, out, st);
  case 4: return launch_xquant<4>(dx, cols, batch, imid, out, st);
  case 8: return launch_xquant<8>(dx, cols, batch, imid, out, st);
  }
  return WV_EFORMAT;
}

template <int F, int R, int S, int D>
static int launch_chunked(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb, int re, cudaStream_t st) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  const int cpr = b.cols >> 5, XS = cpr | 1;
  constexpr int NW = WV_GEMV_THREADS / 32, T = NW / S;
  int dev = 0; cudaGetDevice(&dev);
  int grid = g_tune_grid > 0 ? g_tune_grid : sm_count();
  const int G = fi.table ? (re - rb + R - 1) / R : (re - rb);
  if (grid > G) grid = G;
  if (grid < 1) grid = 1;
  static unsigned attr_mask = 0;
  if constexpr (fi.table) {
    const size_t smem = (size_t)8 * XS * 16 + (size_t)cpr * 8 + 2048 + (size_t)2 * T * S * R * 4 + 16;
    if (smem > 227 * 1024) { wv_set_error("gemv: cols=%d needs %zu bytes of shared memory (max 232448)", b.cols, smem); return WV_ESHAPE; }
    auto kern = gemv_chunked_kernel<F, R, S, D>;
    if (!(attr_mask & (1u << dev))) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) return WV_ECUDA;
      attr_mask |= 1u << dev;
    }
    kern<<<dim3(grid, batch), WV_GEMV_THREADS, smem, st>>>(b, dx, dy, rb, re);
    return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
  } else {
    constexpr int NREC = QCfg<F>::INT_MID ? 9 : 7;
    const size_t smem = (size_t)NREC * XS * 16 + (size_t)2 * T * S * R * 4 + 16;
    if (smem > 227 * 1024) { wv_set_error("gemv: cols=%d needs %zu bytes of shared memory (max 232448)", b.cols, smem); return WV_ESHAPE; }
    auto kern = gemv_idot_kernel<F, R, S, D>;
    if (!(attr_mask & (1u << dev))) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) return WV_ECUDA;
      attr_mask |= 1u << dev;
    }
    uint4* xq = wv_scratch_take((size_t)batch * 9 * XS * 16);
    if (!xq) { wv_set_error("gemv: activation scratch too small for batch=%d cols=%d", batch, b.cols); return WV_ENOMEM; }
    int rc = launch_xquant<fi.bits_lo>(dx, b.cols, batch, QCfg<F>::INT_MID ? fi.mid : 0, xq, st);
    if (rc) return rc;
    cudaError_t e = launch_pdl(kern, dim3(grid, batch), dim3(WV_GEMV_THREADS), smem, st, b, (const uint4*)xq, dy, rb, re);
    if (e != cudaSuccess) { wv_set_error("gemv launch: %s", cudaGetErrorString(e)); return WV_ECUDA; }
    return WV_OK;
  }
}

template <int F>
static int launch_format(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb, int re, cudaStream_t st) {
  int R = g_tune_r, S = g_tune_s, D = g_tune_d;
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  if (!R) R = (fi.table || fi.bits_lo == 8) ? 2 : 4;   // 8-bit planes: 4 rows of fragments would spill
  if (!S) S = fi.table ? 1 : 2;
  if (!D) D = 2;
#define WV_CASE(r, s, d) if (R == r && S == s && D == d) return launch_chunked<F, r, s, d>(b, dx, dy, batch, rb, re, st);
  WV_CASE(2, 1, 2) WV_CASE(2, 2, 2) WV_CASE(2, 1, 4) WV_CASE(2, 2, 4) WV_CASE(4, 1, 2) WV_CASE(4, 2, 2) WV_CASE(2, 4, 2) WV_CASE(1, 1, 4)
#undef WV_CASE
  return launch_chunked<F, 2, 1, 2>(b, dx, dy, batch, rb, re, st);
}

template <int DT>
static int launch_dense(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb, int re, cudaStream_t st) {
  size_t smem = (size_t)b.cols * 4 + 16;
  if (smem > 110 * 1024) { wv_set_error("gemv: cols=%d needs %zu bytes of shared memory for x (max 112640)", b.cols, smem); return WV_ESHAPE; }
  static unsigned attr_mask = 0;
  auto kern = g_tune_d == 8 ? gemv_dense_kernel<DT, 8> : gemv_dense_kernel<DT, 4>;   // vectors per lane per step (tuning hook)
  int dev = 0; cudaGetDevice(&dev);
  const unsigned bit = (1u << dev) << (g_tune_d == 8 ? 16 : 0);
  if (!(attr_mask & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024) != cudaSuccess) return WV_ECUDA;
    attr_mask |= bit;
  }
  int grid = g_tune_grid > 0 ? g_tune_grid : 2 * sm_count();
  if (grid > re - rb) grid = re - rb;
  if (grid < 1) grid = 1;
  cudaError_t e = launch_pdl(kern, dim3(grid, batch), dim3(WV_DENSE_THREADS), smem, st, b, dx, dy, rb, re);
  if (e != cudaSuccess) { wv_set_error("gemv (dense) launch: %s", cudaGetErrorString(e)); return WV_ECUDA; }
  return WV_OK;
}

// ------------------------------------------------------------------ greedy pick over the logits
// sampling.ArgMax (reference model/sampling/argmax.go:4-18): first index of the strict maximum; a
// NaN never wins and a NaN in position 0 keeps index 0. One CTA: 128256 logits are 0.5 MB, a few
// microseconds from L2 right after the LM-head GEMV wrote them, and nothing is read back but the index.
__global__ void __launch_bounds__(1024, 1) argmax_kernel(const float* __restrict__ v, int n, int* __restrict__ out) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (n <= 0) { if (tid == 0) *out = 0; return; }
  const float first = v[0];
  if (first != first) { if (tid == 0) *out = 0; return; }   // NaN in position 0: nothing compares greater
  float best = first;
  int bi = 0;
  for (int i = tid; i < n; i += 1024) {
    const float x = v[i];
    if (x > best) { best = x; bi = i; }   // indices rise within a thread: ties keep the earliest
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = s_val[lane]; bi = s_idx[lane];
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) *out = bi;
  }
}
int wv_launch_argmax(const float* d_logits, int n, int* d_out, cudaStream_t st) {
  argmax_kernel<<<1, 1024, 0, st>>>(d_logits, n, d_out);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}

thread_local const WvPeers* wv_cur_peers = nullptr;
thread_local const WvFuse* wv_cur_fuse = nullptr;

// Copies n floats of this GPU's slice to the same position of every other rank's vector (the
// kernels without a peer-storing epilogue finish with this).
__global__ void scatter_slice_kernel(const WvPeers peers, int n) {
  const float* src = peers.y[peers.self];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const float v = src[i];
    for (int q = 0; q < peers.n; q++) if (q != peers.self) peers.y[q][i] = v;
  }
}

// ------------------------------------------------------------------ arrival flags of the gather
struct WvFlagPeers { unsigned* f[WV_MAX_PEERS]; int n, self; };

// One thread per rank: this rank's new step number goes to word `self` of every rank's flags.
__global__ void gather_signal_kernel(const WvFlagPeers p) {
  __shared__ unsigned s_epoch;
  if (threadIdx.x == 0) s_epoch = ++p.f[p.self][p.n];          // word n: steps signalled by this rank
  __syncthreads();
  if ((int)threadIdx.x < p.n) {
    __threadfence_system();                                     // the rows stored by the preceding kernels first
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.f[threadIdx.x] + p.self), "r"(s_epoch) : "memory");
  }
}
// One thread per rank polls its word until it reaches this rank's new wait number; bounded.
__global__ void gather_wait_kernel(unsigned* flags, int n, int* err, int max_polls) {
  __shared__ unsigned s_epoch;
  if (threadIdx.x == 0) s_epoch = ++flags[n + 1];               // word n + 1: steps waited for by this rank
  __syncthreads();
  if ((int)threadIdx.x < n) {
    bool ok = false;
    for (int i = 0; i < max_polls && !ok; i++) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
      ok = (int)(v - s_epoch) >= 0;
      if (!ok) __nanosleep(256);
    }
    if (!ok) atomicCAS_system(err, 0, 700 + (int)threadIdx.x);
  }
}
// Signal and wait in one launch (a step whose consumers follow at once needs both, and a launch costs more than
// either does): thread q tells rank q that this rank's rows are stored, then polls rank q's word here. Launched
// with programmatic stream serialisation, so that it is resident and past its set-up when the GEMV before it ends.
__global__ void gather_sync_kernel(const WvFlagPeers p, int* err, int max_polls) {
  __shared__ unsigned s_sig, s_wait;
  asm volatile("griddepcontrol.wait;" ::: "memory");              // the preceding kernel's stores are complete and visible
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  unsigned* own = p.f[p.self];
  if (threadIdx.x == 0) { s_sig = ++own[p.n]; s_wait = ++own[p.n + 1]; }
  __syncthreads();
  if ((int)threadIdx.x < p.n) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.f[threadIdx.x] + p.self), "r"(s_sig) : "memory");
    bool ok = false;
    for (int i = 0; i < max_polls && !ok; i++) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(own + threadIdx.x) : "memory");
      ok = (int)(v - s_wait) >= 0;
      if (!ok) __nanosleep(64);
    }
    if (!ok) atomicCAS_system(err, 0, 700 + (int)threadIdx.x);
  }
}
static int gather_max_polls() {
  // Bound of the wait: polls of about a quarter microsecond each. 250 ms by default (host jitter between ranks:
  // a slow graph launch, a first-call attribute set), WELVET_CUDA_GATHER_WAIT_MS overrides it within [1, 2000].
  static int max_polls = 0;
  if (!max_polls) {
    long ms = 250;
    if (const char* e = getenv("WELVET_CUDA_GATHER_WAIT_MS")) { long v = atol(e); if (v >= 1 && v <= 2000) ms = v; }
    max_polls = (int)(ms * 4000);
  }
  return max_polls;
}
int* wv_tma_err_ptr();
int wv_launch_gather_sync(unsigned* const* flags_all, int world, int rank, cudaStream_t st) {
  WvFlagPeers p{};
  p.n = world; p.self = rank;
  for (int q = 0; q < world; q++) p.f[q] = flags_all[q];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1); cfg.blockDim = dim3(32); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gather_sync_kernel, p, wv_tma_err_ptr(), gather_max_polls()) == cudaSuccess ? WV_OK : WV_ECUDA;
}
int wv_launch_gather_signal(unsigned* const* flags_all, int world, int rank, cudaStream_t st) {
  WvFlagPeers p{};
  p.n = world; p.self = rank;
  for (int q = 0; q < world; q++) p.f[q] = flags_all[q];
  gather_signal_kernel<<<1, 32, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}
int wv_launch_gather_wait(unsigned* flags_own, int world, cudaStream_t st) {
  gather_wait_kernel<<<1, 32, 0, st>>>(flags_own, world, wv_tma_err_ptr(), gather_max_polls());
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}

// Kernels that load planes through registers (and the FormatNone streaming kernel).
static int launch_gemv_regs(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st) {
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

int wv_launch_gemm_tcgen05(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st);   // wv_gemm_tcgen05.cu
// Development switch (libraries built with the hooks only): WV_BATCH_LOOP=1 in the environment keeps batches on the
// one-row-at-a-time kernels, for timing one path against the other.
int wv_tma_tuning_rt();   // wv_gemv_tma.cu
static bool batch_loop_forced() {
#ifdef WV_DEV_HOOKS
  static const bool v = [] { const char* e = getenv("WV_BATCH_LOOP"); return e && *e == '1'; }();
  return v;
#else
  return false;
#endif
}

// Smallest batch of an L2-resident matrix that goes to the tensor-core kernel (development builds: WV_BATCH_MIN overrides).
static int batch_min() {
#ifdef WV_DEV_HOOKS
  static const int v = [] { const char* e = getenv("WV_BATCH_MIN"); const int n = e ? atoi(e) : 0; return n >= 2 ? n : 6; }();
  return v;
#else
  return 6;
#endif
}

int wv_launch_gemv(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st) {
  if (row_end <= row_begin || batch <= 0) return WV_OK;
  const WvPeers* pp = wv_cur_peers;
  if (pp && batch != 1) return WV_ESHAPE;
  // Measured at 4096 x 4096 (L2-resident): the tensor-core kernel costs 17-20 us whatever the batch, a batch-1 launch
  // 5 us per row, so small batches of a matrix that stays in L2 run row by row; a matrix that does not fit L2 would
  // be streamed from HBM once per row, so there the tensor-core kernel takes every batch.
  const WvFmtInfo bfi = wv_fmt_info(b.format);
  const bool big = (double)b.n * (bfi.bits_lo + bfi.bits_hi) / 8.0 > 64e6;
  if ((batch >= batch_min() || (batch >= 2 && big)) && !pp && !wv_cur_fuse && !g_tune_r && !wv_tma_tuning_rt() && !batch_loop_forced()) {   // a kernel forced by a tuning code keeps the batch on it
    // Several activation rows: the tensor-core kernel streams and dequantises the matrix once for up to 256 of
    // them. What it does not take (FormatNone, ragged rows) runs row by row below.
    int rc = wv_launch_gemm_tcgen05(b, dx, dy, batch < 256 ? batch : 256, row_begin, row_end, st);
    if (rc != 1) {
      for (int b0 = 256; b0 < batch && !rc; b0 += 256) {
        const int nb = batch - b0 < 256 ? batch - b0 : 256;
        const float* xs = dx + (size_t)b0 * b.cols;
        float* ys = dy + (size_t)b0 * b.rows;
        rc = nb >= 2 ? wv_launch_gemm_tcgen05(b, xs, ys, nb, row_begin, row_end, st) : wv_launch_gemv(b, xs, ys, 1, row_begin, row_end, st);
      }
      return rc;
    }
  }
  if (b.fast && b.format != WV_NONE && !g_tune_r) {   // an explicit tuning override selects the register-load kernels
    const int rc = wv_launch_gemv_tma(b, dx, dy, batch, row_begin, row_end, st);   // stores to the peers in its epilogue
    if (rc != 1) return rc;
  }
  // no peer-storing epilogue on the remaining paths: compute into the own vector, then copy the slice out
  float* out = pp ? pp->y[pp->self] : dy;
  const int rc = b.fast ? launch_gemv_regs(b, dx, out, batch, row_begin, row_end, st)
                        : wv_launch_gemv_ragged(b, dx, out, batch, row_begin, row_end, st);
  if (rc || !pp) return rc;
  WvPeers shifted = *pp;
  for (int q = 0; q < shifted.n; q++) shifted.y[q] += row_begin;
  const int n = row_end - row_begin, blocks = (n + 255) / 256;
  scatter_slice_kernel<<<blocks > 64 ? 64 : blocks, 256, 0, st>>>(shifted, n);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}


// ------------------------------------------------------------------ entry point that allocates nothing
// Some embedders reach this library at a point where they can no longer allocate device
// memory: a serving process that has already handed every remaining byte of HBM to its own
// pools (KV cache, another framework's caching allocator) gets out-of-memory from any later
// cudaMalloc, and a latency-critical decode loop cannot afford the device-wide synchronisation
// that cudaMalloc / cudaFree imply. wv_matvec_dev takes its activation scratch from an arena
// that wv_init obtained with cudaMalloc; this variant of the same GEMV (activation
// pre-quantisation + register-load integer-dot kernel) keeps that scratch in a fixed array
// inside the library image instead, so the call itself performs no allocation of any kind.
//
// Limits: batch 1, packed integer-code formats (not IQ4_NL, not FormatNone: those kernels use
// no scratch), chunk-aligned shapes, cols <= WV_STATIC_MAX_COLS. Every GPU that loads the
// library carries the array (about 148 KB) until the process exits. All calls share it and it
// keeps the previous call's contents; the pre-quantisation kernel rewrites every record the
// GEMV reads, so nothing has to be cleared, but two calls that overlap on the GPU (different
// streams) race on it — issue them on one stream.
#define WV_STATIC_MAX_COLS 32768
static __device__ __align__(256) uint4 g_static_xq[9 * ((WV_STATIC_MAX_COLS >> 5) | 1)];

// In host code the name g_static_xq is only a stand-in for the symbol, not a device address;
// the address a kernel may use comes from cudaGetSymbolAddress, once per device.
static uint4* g_static_xq_addr[64] = {nullptr};

int wv_api_get_blob(uint64_t key, WvDevBlob* out);  // wv_api.cu
int wv_api_bind_device();                           // wv_api.cu: makes the library's device current, returns its index or an error

template <int F>
static int launch_static(const WvDevBlob& b, const float* dx, float* dy, uint4* xq, int dev, cudaStream_t st) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  if constexpr (fi.table || fi.kind == WK_NONE) {
    wv_set_error("wv_matvec_dev_static: format %d uses no scratch and has no static variant", F);
    return WV_EFORMAT;
  } else {
    constexpr int R = 2, S = 1, D = 2;
    const int cpr = b.cols >> 5, XS = cpr | 1;
    const size_t smem = (size_t)QCfg<F>::NREC * XS * 16 + (size_t)2 * (WV_GEMV_THREADS / 32) * R * 4 + 16;
    auto kern = gemv_idot_kernel<F, R, S, D>;
    static unsigned long long attr_mask = 0;   // the attribute is set once per device, not per call
    if (!(attr_mask & (1ull << dev))) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) return WV_ECUDA;
      attr_mask |= 1ull << dev;
    }
    int rc = launch_xquant<fi.bits_lo>(dx, b.cols, 1, QCfg<F>::INT_MID ? fi.mid : 0, xq, st);
    if (rc) return rc;
    int grid = wv_sm_count();
    if (grid > b.rows) grid = b.rows;
    cudaError_t e = launch_pdl(kern, dim3(grid, 1), dim3(WV_GEMV_THREADS), smem, st, b, (const uint4*)xq, dy, 0, b.rows);
    if (e != cudaSuccess) { wv_set_error("wv_matvec_dev_static: launch: %s", cudaGetErrorString(e)); return WV_ECUDA; }
    return WV_OK;
  }
}

// y[out] = W x[in] for a resident blob, device pointers, asynchronous on `stream`; performs no
// cudaMalloc / cudaFree and calls no allocating routine. The first call on a device resolves
// the address of the static scratch (cudaGetSymbolAddress with that device current); make that
// first call before starting any stream capture.
extern "C" int wv_matvec_dev_static(uint64_t key, const float* dx, float* dy, int in, int out, void* stream) {
  const int dev = wv_api_bind_device();   // cudaSetDevice(bound device): a fresh host thread starts on device 0
  if (dev < 0) return dev;
  if (!dx || !dy) { wv_set_error("wv_matvec_dev_static: null pointer"); return WV_EARG; }
  WvDevBlob b;
  int rc = wv_api_get_blob(key, &b);
  if (rc) return rc;
  if (in != b.cols || out != b.rows) { wv_set_error("wv_matvec_dev_static: size mismatch rows=%d cols=%d in=%d out=%d", b.rows, b.cols, in, out); return WV_ESHAPE; }
  if (!b.fast) { wv_set_error("wv_matvec_dev_static: cols=%d is not chunk aligned", b.cols); return WV_ESHAPE; }
  if (b.cols > WV_STATIC_MAX_COLS) {
    wv_set_error("wv_matvec_dev_static: cols=%d exceeds the static scratch maximum of %d", b.cols, WV_STATIC_MAX_COLS);
    return WV_ESHAPE;
  }
  if (dev >= 64) { wv_set_error("wv_matvec_dev_static: bad device"); return WV_ECUDA; }
  if (!g_static_xq_addr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_xq);
    if (e != cudaSuccess || !p) { wv_set_error("wv_matvec_dev_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e)); return WV_ECUDA; }
    g_static_xq_addr[dev] = static_cast<uint4*>(p);
  }
  uint4* xq = g_static_xq_addr[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (b.format) {
#define WV_F(f) case f: return launch_static<f>(b, dx, dy, xq, dev, st);
  WV_F(WV_Q8_0) WV_F(WV_Q4_0) WV_F(WV_Q4_1) WV_F(WV_Q5_0) WV_F(WV_Q5_1)
  WV_F(WV_Q2_K) WV_F(WV_Q3_K) WV_F(WV_Q4_K) WV_F(WV_Q5_K) WV_F(WV_Q6_K)
  WV_F(WV_IQ1_S) WV_F(WV_IQ2_XXS) WV_F(WV_IQ2_XS) WV_F(WV_IQ3_XXS) WV_F(WV_IQ3_S) WV_F(WV_IQ4_NL) WV_F(WV_IQ4_XS)
  WV_F(WV_TERNARY) WV_F(WV_BINARY) WV_F(WV_AFFINE) WV_F(WV_NONE)
#undef WV_F
  }
  wv_set_error("wv_matvec_dev_static: unknown format %d", b.format);
  return WV_EFORMAT;
}
