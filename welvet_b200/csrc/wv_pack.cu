// quant.Pack on the device: f32 weights -> the reference's packed wire arrays, byte for byte.
// Restates quant/q4_0.go:10-45, q4_1.go:8-49, q5_0.go:8-45, q5_1.go:8-46, q8_0.go:8-44,
// kquant.go:62-176, iq.go:70-167, ternary.go:11-51, binary.go:11-47, affine_pack.go:15-86 and
// core/floatconv.go:6-18,39-41. One thread owns one block / group / super-block and walks it in
// the reference's order, so sequential float32 sums (absMean) round identically. Compiled with
// --fmad=false; divisions and f64 steps use the IEEE-rounded intrinsics. Packing is an
// upload-time step, not the hot path: clarity over speed.
#include "wv_common.cuh"

__constant__ float c_pack_iq4nl[16] = WV_IQ4NL_GRID;

__device__ __forceinline__ int go_round(double v) { return (int)round(v); }  // math.Round: half away from zero
__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ void put_f32(uint8_t* p, float v) {
  unsigned u = __float_as_uint(v);
  p[0] = (uint8_t)u; p[1] = (uint8_t)(u >> 8); p[2] = (uint8_t)(u >> 16); p[3] = (uint8_t)(u >> 24);
}
__device__ __forceinline__ void put_u32(uint8_t* p, unsigned u) {
  p[0] = (uint8_t)u; p[1] = (uint8_t)(u >> 8); p[2] = (uint8_t)(u >> 16); p[3] = (uint8_t)(u >> 24);
}
__device__ __forceinline__ float max_abs(const float* w, long long s, long long e) {
  float m = 0.f;
  for (long long i = s; i < e; i++) { float a = fabsf(w[i]); if (a > m) m = a; }
  return m;
}
__device__ __forceinline__ void min_max(const float* w, long long s, long long e, float& mn, float& mx) {
  mn = mx = w[s];
  for (long long i = s + 1; i < e; i++) { float v = w[i]; if (v < mn) mn = v; if (v > mx) mx = v; }
}
__device__ __forceinline__ float abs_mean(const float* w, long long s, long long e) {
  float sum = 0.f;
  for (long long i = s; i < e; i++) sum = __fadd_rn(sum, fabsf(w[i]));
  return __fdiv_rn(sum, (float)(e - s));
}
// OR `bits` low bits of v into a zeroed byte buffer at bit position pos (LSB-first).
__device__ __forceinline__ void put_bits(uint8_t* buf, long long pos, unsigned v, int bits) {
  unsigned sh = (unsigned)(pos & 7);
  unsigned long long t = (unsigned long long)v << sh;
  long long by = pos >> 3;
  for (int k = 0; k * 8 < (int)(bits + sh); k++) buf[by + k] |= (uint8_t)(t >> (8 * k));
}

__global__ void pack_classic_kernel(int format, const float* __restrict__ w, long long n, uint8_t* __restrict__ raw) {
  const WvFmtInfo fi = wv_fmt_info(format);
  long long bi = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long nb = (n + 31) / 32;
  if (bi >= nb) return;
  long long s = bi * 32, e = s + 32 > n ? n : s + 32;
  uint8_t* o = raw + bi * fi.wire_block;
  float scale, mn = 0.f;
  if (fi.has_min) {
    float mx; min_max(w, s, e, mn, mx);
    scale = __fdiv_rn(__fsub_rn(mx, mn), format == WV_Q4_1 ? 15.f : 31.f);
  } else {
    scale = __fdiv_rn(max_abs(w, s, e), format == WV_Q4_0 ? 7.f : (format == WV_Q5_0 ? 15.f : 127.f));
  }
  if (scale == 0.f) scale = 1.f;
  put_f32(o, scale);
  if (fi.has_min) put_f32(o + 4, mn);
  uint8_t* q = o + (fi.has_min ? 8 : 4);
  const int nq = (fi.bits_lo + fi.bits_hi) * 4;
  for (int k = 0; k < nq; k++) q[k] = 0;
  for (int j = 0; j < 32; j++) {
    long long i = s + j;
    const bool live = i < n;
    switch (format) {
    case WV_Q4_0: {
      int v = 0;
      if (live) v = clampi(go_round((double)__fdiv_rn(w[i], scale)), -8, 7);
      q[j >> 1] |= (uint8_t)((v & 0xF) << (4 * (j & 1)));
      break;
    }
    case WV_Q4_1: {
      int v = 0;
      if (live) v = clampi(go_round((double)__fdiv_rn(__fsub_rn(w[i], mn), scale)), 0, 15);
      q[j >> 1] |= (uint8_t)(v << (4 * (j & 1)));
      break;
    }
    case WV_Q5_0: {
      int v = 16;
      if (live) v = clampi(go_round(__ddiv_rn((double)w[i], (double)scale)) + 16, 0, 31);
      put_bits(q, 5LL * j, (unsigned)v, 5);
      break;
    }
    case WV_Q5_1: {
      int v = 0;
      if (live) v = clampi(go_round((double)__fdiv_rn(__fsub_rn(w[i], mn), scale)), 0, 31);
      put_bits(q, 5LL * j, (unsigned)v, 5);
      break;
    }
    default: {  // Q8_0
      int v = 0;
      if (live) v = clampi(go_round(__ddiv_rn((double)w[i], (double)scale)), -127, 127);
      q[j] = (uint8_t)(signed char)v;
    }
    }
  }
}

__global__ void pack_k_kernel(int format, const float* __restrict__ w, long long n, uint8_t* __restrict__ raw) {
  const WvFmtInfo fi = wv_fmt_info(format);
  const int bits = fi.bits_lo + fi.bits_hi, qmax = (1 << bits) - 1, mid = fi.mid;
  long long si = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long nsb = (n + 255) / 256;
  if (si >= nsb) return;
  uint8_t* o = raw + si * fi.wire_block;
  for (int k = 0; k < fi.wire_block; k++) o[k] = 0;
  uint8_t* qs = o + (fi.has_min ? 40 : 24);
  float gscale[16], gmin[16];
  long long base = si * 256;
  for (int g = 0; g < 16; g++) {
    long long gs = base + g * 16, ge = gs + 16;
    gscale[g] = 0.f; gmin[g] = 0.f;
    if (gs >= n) { gscale[g] = 1.f; continue; }
    if (ge > n) ge = n;
    if (fi.has_min) {
      float mn, mx; min_max(w, gs, ge, mn, mx);
      float sc = __fdiv_rn(__fsub_rn(mx, mn), (float)qmax);
      if (sc == 0.f) sc = 1.f;
      gmin[g] = mn; gscale[g] = sc;
      for (int j = 0; j < 16; j++) {
        long long i = gs + j;
        int q = 0;
        if (i < n) q = clampi(go_round((double)__fdiv_rn(__fsub_rn(w[i], mn), sc)), 0, qmax);
        put_bits(qs, (long long)(g * 16 + j) * bits, (unsigned)q, bits);
      }
    } else {
      float sc = __fdiv_rn(max_abs(w, gs, ge), (float)mid);
      if (sc == 0.f) sc = 1.f;
      gscale[g] = sc;
      for (int j = 0; j < 16; j++) {
        long long i = gs + j;
        int q = mid;
        if (i < n) q = clampi(go_round(__ddiv_rn((double)w[i], (double)sc)) + mid, 0, qmax);
        put_bits(qs, (long long)(g * 16 + j) * bits, (unsigned)q, bits);
      }
    }
  }
  float d = 0.f, dmin = 0.f;
  for (int g = 0; g < 16; g++) {
    if (gscale[g] > d) d = gscale[g];
    if (fi.has_min) { float a = fabsf(gmin[g]); if (a > dmin) dmin = a; }
  }
  if (d == 0.f) d = 1.f;
  if (fi.has_min && dmin == 0.f) dmin = 1.f;
  put_f32(o, d); put_f32(o + 4, dmin);
  for (int g = 0; g < 16; g++)
    o[8 + g] = (uint8_t)clampi(go_round(__dmul_rn(__ddiv_rn((double)gscale[g], (double)d), 255.0)), 0, 255);
  if (fi.has_min)
    for (int g = 0; g < 16; g++) {
      int u = 0;
      if (dmin > 0.f) u = clampi(go_round(__dmul_rn(__ddiv_rn((double)gmin[g], (double)dmin), 127.0)), -127, 127);
      o[24 + g] = (uint8_t)(signed char)u;
    }
}

__global__ void pack_iq_kernel(int format, const float* __restrict__ w, long long n, uint8_t* __restrict__ raw, float* __restrict__ scales) {
  const WvFmtInfo fi = wv_fmt_info(format);
  const int bits = fi.bits_lo + fi.bits_hi, group = fi.pgroup, qmax = (1 << bits) - 1;
  const float midf = (float)fi.mid + 0.5f;
  long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long nscale = (n + group - 1) / group;
  if (s >= nscale) return;
  long long st = s * group, en = st + group > n ? n : st + group;
  float amax = max_abs(w, st, en), scale;
  if (fi.table || bits == 1) scale = amax;
  else { float denom = __fsub_rn((float)qmax, midf); if (denom < 1.f) denom = 1.f; scale = __fdiv_rn(amax, denom); }
  if (scale == 0.f) scale = 1.f;
  scales[s] = scale;
  for (int j = 0; j < group; j++) {
    long long i = st + j;
    int q = 0;
    if (i < n) {
      if (fi.table) {
        float target = __fdiv_rn(w[i], scale), best_err = 1e30f;
        for (int c = 0; c < 16; c++) { float e = fabsf(__fsub_rn(c_pack_iq4nl[c], target)); if (e < best_err) { best_err = e; q = c; } }
      } else if (bits == 1) q = w[i] >= 0.f ? 1 : 0;
      else q = clampi(go_round(__dadd_rn(__ddiv_rn((double)w[i], (double)scale), (double)midf)), 0, qmax);
    }
    put_bits(raw, i * bits, (unsigned)q, bits);
  }
}

__global__ void pack_bitnet_kernel(int format, int group, const float* __restrict__ w, long long n, uint8_t* __restrict__ raw, float* __restrict__ scales) {
  // ternary (16 / word), binary g32 (32 / word), binary g128 (row aligned: 4 words share a scale)
  long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int width = format == WV_TERNARY ? 16 : (group == 128 ? 128 : 32);
  long long ng = (n + width - 1) / width;
  if (g >= ng) return;
  long long s = g * width, e = s + width > n ? n : s + width;
  float scale = abs_mean(w, s, e);
  if (group == 128) {  // BlobFromMLX1Bit on {scale = 2 s_g, bias = -s_g}: quant/binary_g128.go:46-58
    float v = scale;   // -bias
    if (v == 0.f) v = __fmul_rn(__fmul_rn(2.f, scale), 0.5f);
    if (v == 0.f) v = 1.f;
    scale = v;
  } else if (scale == 0.f) scale = 1.f;
  scales[g] = scale;
  if (format == WV_TERNARY) {
    unsigned word = 0;
    for (int j = 0; j < 16; j++) {
      long long i = s + j;
      unsigned code = 1;
      if (i < n) code = (unsigned)(clampi(go_round((double)__fdiv_rn(w[i], scale)), -1, 1) + 1);
      word |= (code & 3u) << (2 * j);
    }
    put_u32(raw + g * 4, word);
  } else {
    for (int wd = 0; wd < width / 32; wd++) {
      unsigned word = 0;
      for (int j = 0; j < 32; j++) { long long i = s + wd * 32 + j; if (i < n && w[i] >= 0.f) word |= 1u << j; }
      put_u32(raw + (g * (width / 32) + wd) * 4, word);
    }
  }
}

__global__ void pack_affine_kernel(int group, const float* __restrict__ w, long long n, uint8_t* __restrict__ raw,
                                   float* __restrict__ scales, float* __restrict__ biases) {
  long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n / group) return;
  long long s = g * group;
  float mn, mx; min_max(w, s, s + group, mn, mx);
  float sc = __fdiv_rn(__fsub_rn(mx, mn), 15.f);
  if (sc == 0.f || isnan(sc) || isinf(sc)) { sc = 1.f; mn = 0.f; }
  scales[g] = sc; biases[g] = mn;
  const float inv = __fdiv_rn(1.f, sc);
  for (int wi = 0; wi < group / 8; wi++) {
    unsigned word = 0;
    for (int j = 0; j < 8; j++) {
      int code = clampi(go_round((double)__fmul_rn(__fsub_rn(w[s + wi * 8 + j], mn), inv)), 0, 15);
      word |= (unsigned)code << (4 * j);
    }
    put_u32(raw + (s / 8 + wi) * 4, word);
  }
}

__global__ void pack_none_kernel(int dtype, const float* __restrict__ w, long long n, uint8_t* __restrict__ raw) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    unsigned b = __float_as_uint(w[i]);
    if (dtype == WV_DT_F32) { reinterpret_cast<unsigned*>(raw)[i] = b; continue; }
    unsigned short h;
    if (dtype == WV_DT_BF16) h = (unsigned short)(b >> 16);
    else {  // Float32ToFloat16: truncate, flush small to zero, overflow to inf
      unsigned short sign = (unsigned short)((b >> 16) & 0x8000u);
      int expo = (int)((b >> 23) & 0xff) - 127 + 15;
      unsigned mant = b & 0x7fffffu;
      if (expo <= 0) h = sign;
      else if (expo >= 31) h = sign | 0x7c00;
      else h = sign | (unsigned short)(expo << 10) | (unsigned short)(mant >> 13);
    }
    reinterpret_cast<unsigned short*>(raw)[i] = h;
  }
}

int wv_launch_pack(int format, int dtype, int group, const float* d_w, int rows, int cols, uint8_t* d_raw,
                   float* d_scales, float* d_mins, cudaStream_t st) {
  const WvFmtInfo fi = wv_fmt_info(format);
  const long long n = (long long)rows * cols;
  const int nt = 128;
  auto blocks = [&](long long items) { return (unsigned)((items + nt - 1) / nt); };
  switch (fi.kind) {
  case WK_NONE: pack_none_kernel<<<148 * 8, 256, 0, st>>>(dtype, d_w, n, d_raw); break;
  case WK_CLASSIC: pack_classic_kernel<<<blocks((n + 31) / 32), nt, 0, st>>>(format, d_w, n, d_raw); break;
  case WK_KQUANT: pack_k_kernel<<<blocks((n + 255) / 256), nt, 0, st>>>(format, d_w, n, d_raw); break;
  case WK_IQ: pack_iq_kernel<<<blocks((n + fi.pgroup - 1) / fi.pgroup), nt, 0, st>>>(format, d_w, n, d_raw, d_scales); break;
  case WK_TERNARY: pack_bitnet_kernel<<<blocks((n + 15) / 16), nt, 0, st>>>(format, 16, d_w, n, d_raw, d_scales); break;
  case WK_BINARY: pack_bitnet_kernel<<<blocks((n + group - 1) / group), nt, 0, st>>>(format, group, d_w, n, d_raw, d_scales); break;
  case WK_AFFINE: pack_affine_kernel<<<blocks(n / group), nt, 0, st>>>(group, d_w, n, d_raw, d_scales, d_mins); break;
  default: return WV_EFORMAT;
  }
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}
