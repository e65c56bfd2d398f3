/*
 * welvet_oracle.c — CPU restatement of openfluke/welvet's Dense MatVec path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA product
 * path; nothing in the product may call it. It restates, function by
 * function, the reference's Go code (paths are relative to the reference
 * module root):
 *
 *   quant/helpers.go       bit I/O, roundToInt (math.Round), absMean, ranges
 *   quant/q4_0.go q4_1.go q5_0.go q5_1.go q8_0.go      classic 32-blocks
 *   quant/kquant.go        Q2_K..Q6_K super-blocks
 *   quant/iq.go            IQ1_S..IQ4_XS
 *   quant/ternary.go binary.go binary_g128.go          BitNet style packs
 *   quant/affine_pack.go affine_g64.go                 MLX affine 4-bit
 *   quant/none.go, core/floatconv.go, weights/native.go  FormatNone f32/f16/bf16
 *   weights/packed_wire.go wire encode/decode
 *   simd/dot_q4_amd64.s dot_qx_amd64.s avx2_amd64.s dot_k.go dot_qx.go
 *   layers/dense/gemv_parallel.go                      SIMD path (f64 accumulate)
 *
 * Float semantics pinned: amd64 Go rounds every float32 operation separately
 * (no fused multiply-add unless GOAMD64=v3), so this file must be compiled
 * with -ffp-contract=off and without -ffast-math. math.Round is C round().
 *
 * PARITY STATUS: the reference tree holds no golden vectors, known-answer
 * tests or fixtures for this path and its toolchain (Go) is not available
 * where this was written, so this restatement is "parity unpinned" against
 * the reference binary. It is pinned instead against a second, independently
 * structured numpy restatement (oracle_np.py) and hand-derived single-block
 * vectors (tests/golden).
 */
#define _GNU_SOURCE
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#if defined(__x86_64__)
#include <immintrin.h>
#endif

/* quant.Format values, quant/format.go:9-39 */
enum {
  F_NONE = 0, F_Q8_0, F_Q4_0, F_Q4_1, F_Q5_0, F_Q5_1,
  F_Q2_K, F_Q3_K, F_Q4_K, F_Q5_K, F_Q6_K,
  F_IQ1_S, F_IQ2_XXS, F_IQ2_XS, F_IQ3_XXS, F_IQ3_S, F_IQ4_NL, F_IQ4_XS,
  F_TERNARY, F_BINARY, F_AFFINE, F_COUNT
};
/* core.DType values used by FormatNone, core/dtype.go:14-17 */
enum { DT_F32 = 1, DT_F16 = 2, DT_BF16 = 3 };

typedef struct {
  int32_t format;
  int32_t dtype;         /* FormatNone only */
  int32_t rows, cols;
  int32_t block_weights; /* quant.Blob.BlockWeights */
  int32_t _pad;
  uint8_t *raw;  uint64_t nraw;
  float *scales; uint64_t ns;
  float *mins;   uint64_t nm;
} wvo_blob;

/* ---------- helpers (quant/helpers.go) ---------- */
static inline void put_f32(uint8_t *b, float v) { memcpy(b, &v, 4); }
static inline float get_f32(const uint8_t *b) { float v; memcpy(&v, b, 4); return v; }
static inline void put_u32(uint8_t *b, uint32_t v) { memcpy(b, &v, 4); }
static inline uint32_t get_u32(const uint8_t *b) { uint32_t v; memcpy(&v, b, 4); return v; }
static inline int clamp_int(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
static inline float abs32(float v) { return v < 0 ? -v : v; }
static inline int round_to_int(double v) { return (int)round(v); }

static float abs_mean(const float *w, int64_t s, int64_t e) {
  if (e <= s) return 0;
  float sum = 0;
  for (int64_t i = s; i < e; i++) sum += abs32(w[i]);
  return sum / (float)(e - s);
}
static float max_abs_range(const float *w, int64_t s, int64_t e) {
  float m = 0;
  for (int64_t i = s; i < e; i++) { float a = abs32(w[i]); if (a > m) m = a; }
  return m;
}
static void min_max_range(const float *w, int64_t s, int64_t e, float *mn, float *mx) {
  if (s >= e) { *mn = 0; *mx = 0; return; }
  float a = w[s], b = w[s];
  for (int64_t i = s + 1; i < e; i++) { if (w[i] < a) a = w[i]; if (w[i] > b) b = w[i]; }
  *mn = a; *mx = b;
}

/* bitWriter / bitReader: LSB-first inside a byte, bytes ascending. */
typedef struct { uint8_t *buf; uint64_t len; uint64_t pos; } bitw;
static inline void bw_write(bitw *b, uint32_t val, int nbits) {
  for (int i = 0; i < nbits; i++) {
    if ((val >> i) & 1) b->buf[b->pos >> 3] |= (uint8_t)(1u << (b->pos & 7));
    b->pos++;
  }
}
typedef struct { const uint8_t *buf; uint64_t len; uint64_t pos; } bitr;
static inline uint32_t br_read(bitr *b, int nbits) {
  uint32_t v = 0;
  for (int i = 0; i < nbits; i++) {
    if ((b->pos >> 3) < b->len && ((b->buf[b->pos >> 3] >> (b->pos & 7)) & 1)) v |= 1u << i;
    b->pos++;
  }
  return v;
}

/* ---------- k-quant / IQ specs (quant/kquant.go:36-60, quant/iq.go:49-68) ---------- */
typedef struct { int bits, has_dmin, qmax, mid; } kspec;
static int kspec_for(int f, kspec *s) {
  switch (f) {
  case F_Q2_K: *s = (kspec){2, 1, 3, 0}; return 1;
  case F_Q3_K: *s = (kspec){3, 1, 7, 0}; return 1;
  case F_Q4_K: *s = (kspec){4, 1, 15, 0}; return 1;
  case F_Q5_K: *s = (kspec){5, 1, 31, 0}; return 1;
  case F_Q6_K: *s = (kspec){6, 0, 63, 32}; return 1;
  }
  return 0;
}
static int k_super_bytes(kspec s) { return 8 + 16 + (s.has_dmin ? 16 : 0) + (256 * s.bits + 7) / 8; }

typedef struct { int bits, group, nonlinear; float mid; } iqspec;
static int iqspec_for(int f, iqspec *s) {
  switch (f) {
  case F_IQ1_S:   *s = (iqspec){1, 32, 0, 0.5f}; return 1;
  case F_IQ2_XXS: *s = (iqspec){2, 32, 0, 1.5f}; return 1;
  case F_IQ2_XS:  *s = (iqspec){2, 16, 0, 1.5f}; return 1;
  case F_IQ3_XXS: *s = (iqspec){3, 32, 0, 3.5f}; return 1;
  case F_IQ3_S:   *s = (iqspec){3, 16, 0, 3.5f}; return 1;
  case F_IQ4_NL:  *s = (iqspec){4, 32, 1, 0.0f}; return 1;
  case F_IQ4_XS:  *s = (iqspec){4, 16, 0, 7.5f}; return 1;
  }
  return 0;
}
/* quant/iq.go:23-40 */
static const float iq4nl_grid[16] = {
  -1.0f, -0.6961928f, -0.52507305f, -0.3949175f, -0.28444138f, -0.18477343f, -0.091050036f, 0.0f,
  0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f, 0.562617f, 0.72295684f, 1.0f};

/* ---------- float16 / bfloat16 codecs (core/floatconv.go) ---------- */
static uint16_t f32_to_f16_trunc(float f) { /* Float32ToFloat16: truncation, flush-to-zero */
  uint32_t b; memcpy(&b, &f, 4);
  uint16_t sign = (uint16_t)((b >> 16) & 0x8000);
  int expo = (int)((b >> 23) & 0xff) - 127 + 15;
  uint32_t mant = b & 0x7fffff;
  if (expo <= 0) return sign;
  if (expo >= 31) return sign | 0x7c00;
  return sign | (uint16_t)(expo << 10) | (uint16_t)(mant >> 13);
}
static float f16_to_f32(uint16_t h) { /* Float16ToFloat32 */
  uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t expo = (h >> 10) & 0x1f, mant = h & 0x3ff, u;
  if (expo == 0) {
    if (mant == 0) { u = sign; }
    else { float d = (float)mant / 1024 / 16384; uint32_t db; memcpy(&db, &d, 4); u = sign | db; }
  } else if (expo == 31) { u = sign | 0x7f800000u | (mant << 13); }
  else { u = sign | ((expo - 15 + 127) << 23) | (mant << 13); }
  float r; memcpy(&r, &u, 4); return r;
}
static uint16_t f32_to_bf16_trunc(float f) { uint32_t b; memcpy(&b, &f, 4); return (uint16_t)(b >> 16); }
static float bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float r; memcpy(&r, &u, 4); return r; }

/* ---------- sizes ---------- */
/* Bytes/elements a packer produces for rows x cols. block_weights only matters for
 * BinaryPacked (32 vs 128) and AffinePacked (group). Returns 0 on success. */
int wvo_sizes(int format, int dtype, int block_weights, int rows, int cols,
              uint64_t *nraw, uint64_t *ns, uint64_t *nm) {
  if (rows <= 0 || cols <= 0) return -1;
  uint64_t n = (uint64_t)rows * (uint64_t)cols;
  *nraw = 0; *ns = 0; *nm = 0;
  kspec ks; iqspec is;
  switch (format) {
  case F_NONE:
    *nraw = n * (dtype == DT_F32 ? 4 : 2);
    if (dtype != DT_F32 && dtype != DT_F16 && dtype != DT_BF16) return -2;
    return 0;
  case F_Q4_0: *nraw = (n + 31) / 32 * 20; return 0;
  case F_Q4_1: *nraw = (n + 31) / 32 * 24; return 0;
  case F_Q5_0: *nraw = (n + 31) / 32 * 24; return 0;
  case F_Q5_1: *nraw = (n + 31) / 32 * 28; return 0;
  case F_Q8_0: *nraw = (n + 31) / 32 * 36; return 0;
  case F_TERNARY: *ns = (n + 15) / 16; *nraw = *ns * 4; return 0;
  case F_BINARY:
    if (block_weights == 128) {
      if (cols % 128) return -3;
      *nraw = (uint64_t)rows * (cols / 32) * 4; *ns = (uint64_t)rows * (cols / 128); return 0;
    }
    *ns = (n + 31) / 32; *nraw = *ns * 4; return 0;
  case F_AFFINE: {
    int g = block_weights > 0 ? block_weights : 64;
    if (cols % 8 || cols % g || g % 8) return -3;
    *nraw = (uint64_t)rows * (cols / 8) * 4; *ns = *nm = (uint64_t)rows * (cols / g); return 0;
  }
  }
  if (kspec_for(format, &ks)) { *nraw = (n + 255) / 256 * (uint64_t)k_super_bytes(ks); return 0; }
  if (iqspec_for(format, &is)) {
    uint64_t padn = (n + is.group - 1) / is.group * is.group;
    *ns = padn / is.group; *nraw = (padn * is.bits + 7) / 8; return 0;
  }
  return -2;
}

/* ---------- Pack ---------- */
static void pack_q4_0(const float *w, int64_t n, uint8_t *raw) { /* quant/q4_0.go:10-45,142-154 */
  int64_t nb = (n + 31) / 32;
  for (int64_t bi = 0; bi < nb; bi++) {
    int64_t s = bi * 32, e = s + 32 > n ? n : s + 32;
    float scale = max_abs_range(w, s, e) / 7;
    if (scale == 0) scale = 1;
    uint8_t *o = raw + bi * 20;
    put_f32(o, scale);
    for (int j = 0; j < 16; j++) {
      int8_t q[2];
      for (int k = 0; k < 2; k++) {
        int64_t i = s + j * 2 + k;
        int v = 0;
        if (i < n) {
          v = (int)round((double)(w[i] / scale));
          if (v > 7) v = 7;
          if (v < -8) v = -8;
        }
        q[k] = (int8_t)v;
      }
      o[4 + j] = (uint8_t)((q[0] & 0xF) | ((q[1] & 0xF) << 4));
    }
  }
}
static void pack_q4_1(const float *w, int64_t n, uint8_t *raw) { /* quant/q4_1.go:8-49 */
  int64_t nb = (n + 31) / 32;
  for (int64_t bi = 0; bi < nb; bi++) {
    int64_t s = bi * 32, e = s + 32 > n ? n : s + 32;
    float mn, mx; min_max_range(w, s, e, &mn, &mx);
    float scale = (mx - mn) / 15;
    if (scale == 0) scale = 1;
    uint8_t *o = raw + bi * 24;
    put_f32(o, scale); put_f32(o + 4, mn);
    for (int j = 0; j < 16; j++) {
      uint8_t nib[2];
      for (int k = 0; k < 2; k++) {
        int64_t i = s + j * 2 + k;
        int q = 0;
        if (i < n) q = clamp_int(round_to_int((double)((w[i] - mn) / scale)), 0, 15);
        nib[k] = (uint8_t)q;
      }
      o[8 + j] = (uint8_t)(nib[0] | (nib[1] << 4));
    }
  }
}
static void pack_q5_0(const float *w, int64_t n, uint8_t *raw) { /* quant/q5_0.go:8-45 */
  int64_t nb = (n + 31) / 32;
  for (int64_t bi = 0; bi < nb; bi++) {
    int64_t s = bi * 32, e = s + 32 > n ? n : s + 32;
    float scale = max_abs_range(w, s, e) / 15;
    if (scale == 0) scale = 1;
    uint8_t *o = raw + bi * 24;
    put_f32(o, scale);
    bitw bw = {o + 4, 20, 0};
    for (int j = 0; j < 32; j++) {
      int64_t i = s + j;
      int q = 16;
      if (i < n) q = clamp_int(round_to_int((double)w[i] / (double)scale) + 16, 0, 31);
      bw_write(&bw, (uint32_t)q, 5);
    }
  }
}
static void pack_q5_1(const float *w, int64_t n, uint8_t *raw) { /* quant/q5_1.go:8-46 */
  int64_t nb = (n + 31) / 32;
  for (int64_t bi = 0; bi < nb; bi++) {
    int64_t s = bi * 32, e = s + 32 > n ? n : s + 32;
    float mn, mx; min_max_range(w, s, e, &mn, &mx);
    float scale = (mx - mn) / 31;
    if (scale == 0) scale = 1;
    uint8_t *o = raw + bi * 28;
    put_f32(o, scale); put_f32(o + 4, mn);
    bitw bw = {o + 8, 20, 0};
    for (int j = 0; j < 32; j++) {
      int64_t i = s + j;
      int q = 0;
      if (i < n) q = clamp_int(round_to_int((double)((w[i] - mn) / scale)), 0, 31);
      bw_write(&bw, (uint32_t)q, 5);
    }
  }
}
static void pack_q8_0(const float *w, int64_t n, uint8_t *raw) { /* quant/q8_0.go:8-44 */
  int64_t nb = (n + 31) / 32;
  for (int64_t bi = 0; bi < nb; bi++) {
    int64_t s = bi * 32, e = s + 32 > n ? n : s + 32;
    float scale = max_abs_range(w, s, e) / 127;
    if (scale == 0) scale = 1;
    uint8_t *o = raw + bi * 36;
    put_f32(o, scale);
    for (int j = 0; j < 32; j++) {
      int64_t i = s + j;
      int q = 0;
      if (i < n) q = clamp_int(round_to_int((double)w[i] / (double)scale), -127, 127);
      o[4 + j] = (uint8_t)(int8_t)q;
    }
  }
}
static void pack_k(kspec sp, const float *w, int64_t n, uint8_t *raw) { /* quant/kquant.go:62-176 */
  int sbb = k_super_bytes(sp);
  int64_t nsb = (n + 255) / 256;
  for (int64_t si = 0; si < nsb; si++) {
    int64_t base = si * 256;
    uint8_t *o = raw + si * sbb;
    float gscale[16], gmin[16];
    uint32_t qs[256];
    memset(gscale, 0, sizeof gscale); memset(gmin, 0, sizeof gmin); memset(qs, 0, sizeof qs);
    for (int g = 0; g < 16; g++) {
      int64_t gs = base + g * 16, ge = gs + 16;
      if (gs >= n) { gscale[g] = 1; continue; }
      if (ge > n) ge = n;
      if (sp.has_dmin) {
        float mn, mx; min_max_range(w, gs, ge, &mn, &mx);
        float sc = (mx - mn) / (float)sp.qmax;
        if (sc == 0) sc = 1;
        gmin[g] = mn; gscale[g] = sc;
        for (int j = 0; j < 16; j++) {
          int64_t i = gs + j;
          int q = 0;
          if (i < n) q = clamp_int(round_to_int((double)((w[i] - mn) / sc)), 0, sp.qmax);
          qs[g * 16 + j] = (uint32_t)q;
        }
      } else {
        float amax = max_abs_range(w, gs, ge);
        float sc = amax / (float)sp.mid;
        if (sc == 0) sc = 1;
        gscale[g] = sc;
        for (int j = 0; j < 16; j++) {
          int64_t i = gs + j;
          int q = sp.mid;
          if (i < n) q = clamp_int(round_to_int((double)w[i] / (double)sc) + sp.mid, 0, sp.qmax);
          qs[g * 16 + j] = (uint32_t)q;
        }
      }
    }
    float d = 0, dmin = 0;
    for (int g = 0; g < 16; g++) {
      if (gscale[g] > d) d = gscale[g];
      if (sp.has_dmin) { float a = abs32(gmin[g]); if (a > dmin) dmin = a; }
    }
    if (d == 0) d = 1;
    if (sp.has_dmin && dmin == 0) dmin = 1;
    put_f32(o, d); put_f32(o + 4, dmin);
    for (int g = 0; g < 16; g++)
      o[8 + g] = (uint8_t)clamp_int(round_to_int((double)gscale[g] / (double)d * 255), 0, 255);
    int qoff = 24;
    if (sp.has_dmin) {
      for (int g = 0; g < 16; g++) {
        uint8_t u = 0;
        if (dmin > 0) u = (uint8_t)clamp_int(round_to_int((double)gmin[g] / (double)dmin * 127), -127, 127);
        o[qoff + g] = u;
      }
      qoff += 16;
    }
    bitw bw = {o + qoff, (uint64_t)(sbb - qoff), 0};
    for (int i = 0; i < 256; i++) bw_write(&bw, qs[i], sp.bits);
  }
}
static void pack_iq(iqspec sp, const float *w, int64_t n, uint8_t *raw, uint64_t nraw, float *scales) {
  /* quant/iq.go:70-167 */
  int64_t padn = (n + sp.group - 1) / sp.group * sp.group;
  int64_t nscale = padn / sp.group;
  int qmax = (1 << sp.bits) - 1;
  bitw bw = {raw, nraw, 0};
  for (int64_t s = 0; s < nscale; s++) {
    int64_t st = s * sp.group, en = st + sp.group;
    if (en > n) en = n;
    if (st >= n) {
      scales[s] = 1;
      for (int j = 0; j < sp.group; j++) bw_write(&bw, 0, sp.bits);
      continue;
    }
    if (sp.nonlinear) {
      float scale = max_abs_range(w, st, en);
      if (scale == 0) scale = 1;
      scales[s] = scale;
      for (int j = 0; j < sp.group; j++) {
        int64_t i = st + j;
        int best = 0; float best_err = 1e30f;
        if (i < n) {
          float target = w[i] / scale;
          for (int c = 0; c < 16; c++) {
            float e = abs32(iq4nl_grid[c] - target);
            if (e < best_err) { best_err = e; best = c; }
          }
        }
        bw_write(&bw, (uint32_t)best, 4);
      }
      continue;
    }
    float amax = max_abs_range(w, st, en), scale;
    if (sp.bits == 1) scale = amax;
    else {
      float denom = (float)qmax - sp.mid;
      if (denom < 1) denom = 1;
      scale = amax / denom;
    }
    if (scale == 0) scale = 1;
    scales[s] = scale;
    for (int j = 0; j < sp.group; j++) {
      int64_t i = st + j;
      int q = 0;
      if (i < n) {
        if (sp.bits == 1) { if (w[i] >= 0) q = 1; }
        else q = clamp_int(round_to_int((double)w[i] / (double)scale + (double)sp.mid), 0, qmax);
      }
      bw_write(&bw, (uint32_t)q, sp.bits);
    }
  }
}
static void pack_ternary(const float *w, int64_t n, uint8_t *raw, float *scales) { /* quant/ternary.go:11-51 */
  int64_t ng = (n + 15) / 16;
  for (int64_t g = 0; g < ng; g++) {
    int64_t s = g * 16, e = s + 16 > n ? n : s + 16;
    float scale = abs_mean(w, s, e);
    if (scale == 0) scale = 1;
    scales[g] = scale;
    uint32_t word = 0;
    for (int j = 0; j < 16; j++) {
      int64_t i = s + j;
      uint32_t code = 1;
      if (i < n) {
        int q = clamp_int(round_to_int((double)(w[i] / scale)), -1, 1);
        code = (uint32_t)(q + 1);
      }
      word |= (code & 3) << (j * 2);
    }
    put_u32(raw + g * 4, word);
  }
}
static void pack_binary32(const float *w, int64_t n, uint8_t *raw, float *scales) { /* quant/binary.go:11-47 */
  int64_t ng = (n + 31) / 32;
  for (int64_t g = 0; g < ng; g++) {
    int64_t s = g * 32, e = s + 32 > n ? n : s + 32;
    float scale = abs_mean(w, s, e);
    if (scale == 0) scale = 1;
    scales[g] = scale;
    uint32_t word = 0;
    for (int j = 0; j < 32; j++) {
      int64_t i = s + j;
      if (i < n && w[i] >= 0) word |= 1u << j;
    }
    put_u32(raw + g * 4, word);
  }
}
/* Harness definition (the reference has no f32 packer for the g128 layout; its g128
 * blobs come from MLX tensors through BlobFromMLX1Bit, quant/binary_g128.go:23-69):
 * bit = (w >= 0); s_g = absMean over the row-aligned 128 group; the MLX tensors that
 * would encode that are scale = 2*s_g, bias = -s_g, which BlobFromMLX1Bit maps back
 * to Scales = -bias (0 -> scale*0.5, 0 -> 1). */
static void pack_binary128(const float *w, int rows, int cols, uint8_t *raw, float *scales) {
  int gpr = cols / 128, wpr = cols / 32;
  for (int r = 0; r < rows; r++) {
    for (int g = 0; g < gpr; g++) {
      int64_t s = (int64_t)r * cols + g * 128;
      float sg = abs_mean(w, s, s + 128);
      float mlx_scale = 2 * sg, mlx_bias = -sg;
      float v = -mlx_bias;
      if (v == 0) v = mlx_scale * 0.5f;
      if (v == 0) v = 1;
      scales[(int64_t)r * gpr + g] = v;
    }
    for (int wi = 0; wi < wpr; wi++) {
      uint32_t word = 0;
      int64_t s = (int64_t)r * cols + wi * 32;
      for (int j = 0; j < 32; j++) if (w[s + j] >= 0) word |= 1u << j;
      put_u32(raw + ((int64_t)r * wpr + wi) * 4, word);
    }
  }
}
static void pack_affine4(const float *w, int rows, int cols, int group, uint8_t *raw, float *scales, float *biases) {
  /* quant/affine_pack.go:15-86 */
  int wpr = cols / 8, gpr = cols / group, wig = group / 8;
  const float levels = 15.0f;
  for (int r = 0; r < rows; r++) {
    int64_t ro = (int64_t)r * cols;
    for (int g = 0; g < gpr; g++) {
      int cb = g * group;
      float mn = w[ro + cb], mx = mn;
      for (int j = 1; j < group; j++) {
        float v = w[ro + cb + j];
        if (v < mn) mn = v;
        if (v > mx) mx = v;
      }
      float s = (mx - mn) / levels;
      if (s == 0 || isnan(s) || isinf(s)) { s = 1; mn = 0; }
      int64_t si = (int64_t)r * gpr + g;
      scales[si] = s; biases[si] = mn;
      float inv_s = 1 / s;
      for (int wi = 0; wi < wig; wi++) {
        uint32_t word = 0;
        int base = cb + wi * 8;
        for (int j = 0; j < 8; j++) {
          float v = w[ro + base + j];
          int code = (int)round((double)((v - mn) * inv_s));
          if (code < 0) code = 0;
          if (code > 15) code = 15;
          word |= (uint32_t)code << (j * 4);
        }
        put_u32(raw + ((int64_t)r * wpr + g * wig + wi) * 4, word);
      }
    }
  }
}

/* Pack into caller-allocated buffers sized by wvo_sizes. out->format/dtype/rows/cols/
 * block_weights must be set; raw must be zero-filled by the caller (bit writers OR in). */
int wvo_pack(const float *w, wvo_blob *out) {
  if (!w || !out || out->rows <= 0 || out->cols <= 0) return -1;
  int64_t n = (int64_t)out->rows * out->cols;
  kspec ks; iqspec is;
  switch (out->format) {
  case F_NONE:
    if (out->dtype == DT_F32) { memcpy(out->raw, w, (size_t)n * 4); }
    else if (out->dtype == DT_F16) { for (int64_t i = 0; i < n; i++) { uint16_t h = f32_to_f16_trunc(w[i]); memcpy(out->raw + i * 2, &h, 2); } }
    else if (out->dtype == DT_BF16) { for (int64_t i = 0; i < n; i++) { uint16_t h = f32_to_bf16_trunc(w[i]); memcpy(out->raw + i * 2, &h, 2); } }
    else return -2;
    out->block_weights = 1; return 0;
  case F_Q4_0: pack_q4_0(w, n, out->raw); out->block_weights = 32; return 0;
  case F_Q4_1: pack_q4_1(w, n, out->raw); out->block_weights = 32; return 0;
  case F_Q5_0: pack_q5_0(w, n, out->raw); out->block_weights = 32; return 0;
  case F_Q5_1: pack_q5_1(w, n, out->raw); out->block_weights = 32; return 0;
  case F_Q8_0: pack_q8_0(w, n, out->raw); out->block_weights = 32; return 0;
  case F_TERNARY: pack_ternary(w, n, out->raw, out->scales); out->block_weights = 16; return 0;
  case F_BINARY:
    if (out->block_weights == 128) { if (out->cols % 128) return -3; pack_binary128(w, out->rows, out->cols, out->raw, out->scales); return 0; }
    pack_binary32(w, n, out->raw, out->scales); out->block_weights = 32; return 0;
  case F_AFFINE: {
    int g = out->block_weights > 0 ? out->block_weights : 64;
    if (out->cols % 8 || out->cols % g || g % 8) return -3;
    pack_affine4(w, out->rows, out->cols, g, out->raw, out->scales, out->mins);
    out->block_weights = g; return 0;
  }
  }
  if (kspec_for(out->format, &ks)) { pack_k(ks, w, n, out->raw); out->block_weights = 256; return 0; }
  if (iqspec_for(out->format, &is)) { pack_iq(is, w, n, out->raw, out->nraw, out->scales); out->block_weights = 32; return 0; }
  return -2;
}

/* ---------- Unpack: the definition of the dequantised weights ---------- */
static inline float decode_k_weight(float d, float dmin, uint8_t scale_u, uint8_t min_u, uint32_t q, kspec sp) {
  /* quant/kquant.go:178-188 */
  float sc = d * (float)scale_u / 255;
  if (sc == 0) sc = d / 255;
  if (sp.has_dmin) {
    float mn = dmin * (float)(int8_t)min_u / 127;
    return mn + (float)q * sc;
  }
  return sc * (float)((int)q - sp.mid);
}
static inline float iq_dequant(iqspec sp, float scale, uint32_t q) { /* quant/iq.go:169-180 */
  if (sp.nonlinear) return scale * iq4nl_grid[q & 15];
  if (sp.bits == 1) return (q & 1) ? scale : -scale;
  return scale * ((float)q - sp.mid);
}
static int binary_is_g128(const wvo_blob *b) { return b->format == F_BINARY && b->block_weights == 128; }

int wvo_unpack(const wvo_blob *b, float *out) {
  if (!b || !out) return -1;
  int64_t n = (int64_t)b->rows * b->cols;
  const uint8_t *raw = b->raw;
  kspec ks; iqspec is;
  switch (b->format) {
  case F_NONE:
    if ((b->dtype == DT_F32 && b->nraw < (uint64_t)n * 4) || (b->dtype != DT_F32 && b->nraw < (uint64_t)n * 2)) return -3;
    if (b->dtype == DT_F32) memcpy(out, raw, (size_t)n * 4);
    else if (b->dtype == DT_F16) for (int64_t i = 0; i < n; i++) { uint16_t h; memcpy(&h, raw + i * 2, 2); out[i] = f16_to_f32(h); }
    else if (b->dtype == DT_BF16) for (int64_t i = 0; i < n; i++) { uint16_t h; memcpy(&h, raw + i * 2, 2); out[i] = bf16_to_f32(h); }
    else return -2;
    return 0;
  case F_Q4_0: { /* quant/q4_0.go:47-79 */
    int64_t nb = (int64_t)(b->nraw / 20);
    for (int64_t bi = 0; bi < nb; bi++) {
      const uint8_t *o = raw + bi * 20; float scale = get_f32(o); int64_t st = bi * 32;
      for (int j = 0; j < 16; j++) {
        uint8_t wb = o[4 + j];
        int8_t q1 = (int8_t)(wb & 0xF); if (q1 > 7) q1 -= 16;
        int8_t q2 = (int8_t)(wb >> 4); if (q2 > 7) q2 -= 16;
        int64_t i1 = st + j * 2, i2 = i1 + 1;
        if (i1 < n) out[i1] = (float)q1 * scale;
        if (i2 < n) out[i2] = (float)q2 * scale;
      }
    }
    return 0;
  }
  case F_Q4_1: { /* quant/q4_1.go:51-76 */
    int64_t nb = (int64_t)(b->nraw / 24);
    for (int64_t bi = 0; bi < nb; bi++) {
      const uint8_t *o = raw + bi * 24; float scale = get_f32(o), mn = get_f32(o + 4); int64_t st = bi * 32;
      for (int j = 0; j < 16; j++) for (int k = 0; k < 2; k++) {
        int64_t i = st + j * 2 + k; if (i >= n) break;
        int q = (o[8 + j] >> (4 * k)) & 0xF;
        out[i] = mn + (float)q * scale;
      }
    }
    return 0;
  }
  case F_Q5_0: { /* quant/q5_0.go:47-68 */
    int64_t nb = (int64_t)(b->nraw / 24);
    for (int64_t bi = 0; bi < nb; bi++) {
      const uint8_t *o = raw + bi * 24; float scale = get_f32(o); bitr br = {o + 4, 20, 0}; int64_t st = bi * 32;
      for (int j = 0; j < 32; j++) { int q = (int)br_read(&br, 5) - 16; if (st + j < n) out[st + j] = (float)q * scale; }
    }
    return 0;
  }
  case F_Q5_1: { /* quant/q5_1.go:48-70 */
    int64_t nb = (int64_t)(b->nraw / 28);
    for (int64_t bi = 0; bi < nb; bi++) {
      const uint8_t *o = raw + bi * 28; float scale = get_f32(o), mn = get_f32(o + 4); bitr br = {o + 8, 20, 0}; int64_t st = bi * 32;
      for (int j = 0; j < 32; j++) { int q = (int)br_read(&br, 5); if (st + j < n) out[st + j] = mn + (float)q * scale; }
    }
    return 0;
  }
  case F_Q8_0: { /* quant/q8_0.go:46-66 */
    int64_t nb = (int64_t)(b->nraw / 36);
    for (int64_t bi = 0; bi < nb; bi++) {
      const uint8_t *o = raw + bi * 36; float scale = get_f32(o); int64_t st = bi * 32;
      for (int j = 0; j < 32; j++) { if (st + j >= n) break; out[st + j] = (float)(int8_t)o[4 + j] * scale; }
    }
    return 0;
  }
  case F_TERNARY: { /* quant/ternary.go:53-91 */
    int64_t ng = (int64_t)(b->nraw / 4);
    for (int64_t g = 0; g < ng; g++) {
      uint32_t word = get_u32(raw + g * 4);
      float scale = (uint64_t)g < b->ns ? b->scales[g] : 1.0f;
      for (int j = 0; j < 16; j++) {
        int64_t i = g * 16 + j; if (i >= n) break;
        uint32_t c = (word >> (j * 2)) & 3;
        out[i] = c == 0 ? -scale : (c == 2 ? scale : 0.0f);
      }
    }
    return 0;
  }
  case F_BINARY: { /* quant/binary.go:49-84, binary_g128.go:96-128 */
    if (binary_is_g128(b)) {
      int gpr = b->cols / 128, wpr = b->cols / 32;
      for (int r = 0; r < b->rows; r++) for (int g = 0; g < gpr; g++) {
        int64_t si = (int64_t)r * gpr + g;
        float scale = (uint64_t)si < b->ns ? b->scales[si] : 1.0f;
        for (int wi = 0; wi < 4; wi++) {
          uint64_t wo = ((uint64_t)r * wpr + g * 4 + wi) * 4;
          if (wo + 4 > b->nraw) return 0;
          uint32_t word = get_u32(raw + wo);
          int64_t base = (int64_t)r * b->cols + g * 128 + wi * 32;
          for (int j = 0; j < 32; j++) { if (base + j >= n) return 0; out[base + j] = ((word >> j) & 1) ? scale : -scale; }
        }
      }
      return 0;
    }
    int64_t ng = (int64_t)(b->nraw / 4);
    for (int64_t g = 0; g < ng; g++) {
      uint32_t word = get_u32(raw + g * 4);
      float scale = (uint64_t)g < b->ns ? b->scales[g] : 1.0f;
      for (int j = 0; j < 32; j++) { int64_t i = g * 32 + j; if (i >= n) break; out[i] = ((word >> j) & 1) ? scale : -scale; }
    }
    return 0;
  }
  case F_AFFINE: { /* quant/affine_g64.go:121-175 */
    int group = b->block_weights > 0 ? b->block_weights : 64;
    int wpr = b->cols / 8, gpr = b->cols / group, wig = group / 8;
    for (int r = 0; r < b->rows; r++) for (int g = 0; g < gpr; g++) {
      int64_t si = (int64_t)r * gpr + g;
      float s = (uint64_t)si < b->ns ? b->scales[si] : 1.0f;
      float beta = (uint64_t)si < b->nm ? b->mins[si] : 0.0f;
      for (int wi = 0; wi < wig; wi++) {
        uint32_t word = get_u32(raw + ((int64_t)r * wpr + g * wig + wi) * 4);
        int64_t base = (int64_t)r * b->cols + g * group + wi * 8;
        for (int j = 0; j < 8; j++) { uint32_t code = (word >> (j * 4)) & 15; out[base + j] = s * (float)code + beta; }
      }
    }
    return 0;
  }
  }
  if (kspec_for(b->format, &ks)) { /* quant/kquant.go:190-237 */
    int sbb = k_super_bytes(ks);
    int64_t nsb = (int64_t)(b->nraw / sbb);
    for (int64_t si = 0; si < nsb; si++) {
      const uint8_t *o = raw + si * sbb;
      float d = get_f32(o), dmin = get_f32(o + 4);
      const uint8_t *scales = o + 8, *mins = ks.has_dmin ? o + 24 : NULL;
      int qoff = ks.has_dmin ? 40 : 24;
      bitr br = {o + qoff, (uint64_t)(sbb - qoff), 0};
      for (int g = 0; g < 16; g++) {
        uint8_t mu = mins ? mins[g] : 0;
        for (int j = 0; j < 16; j++) {
          int64_t idx = si * 256 + g * 16 + j;
          uint32_t q = br_read(&br, ks.bits);
          if (idx >= n) continue;
          out[idx] = decode_k_weight(d, dmin, scales[g], mu, q, ks);
        }
      }
    }
    return 0;
  }
  if (iqspec_for(b->format, &is)) { /* quant/iq.go:182-219 */
    bitr br = {raw, b->nraw, 0};
    for (uint64_t s = 0; s < b->ns; s++) {
      float scale = b->scales[s];
      for (int j = 0; j < is.group; j++) {
        uint32_t q = br_read(&br, is.bits);
        int64_t i = (int64_t)s * is.group + j;
        if (i >= n) continue;
        out[i] = iq_dequant(is, scale, q);
      }
    }
    return 0;
  }
  return -2;
}

/* ---------- scalar MatVec (quant.MatVec, quant/matvec.go:5-35): f32, flat order ---------- */
static float sum32(const float *x) { /* quant/binary_g128.go:203-212 */
  float s0 = 0, s1 = 0, s2 = 0, s3 = 0;
  for (int i = 0; i < 32; i += 4) { s0 += x[i]; s1 += x[i + 1]; s2 += x[i + 2]; s3 += x[i + 3]; }
  return s0 + s1 + s2 + s3;
}
static float binary_word_sum1(const float *x, uint32_t word) { /* quant/binary_g128_amd64.s:7-54 */
  float a[4] = {0, 0, 0, 0};
  for (int k = 0; k < 8; k++)
    for (int l = 0; l < 4; l++) a[l] += ((word >> (k * 4 + l)) & 1) ? x[k * 4 + l] : 0.0f;
  return (a[0] + a[1]) + (a[2] + a[3]);
}
static void matvec_binary_g128_rows(const wvo_blob *b, const float *x, float *y, const float *sum_all, int lo, int hi) {
  /* quant/binary_g128.go:214-239 */
  int gpr = b->cols / 128, wpr = b->cols / 32;
  for (int r = lo; r < hi; r++) {
    float acc = 0;
    for (int g = 0; g < gpr; g++) {
      float scale = b->scales[(int64_t)r * gpr + g];
      for (int wi = 0; wi < 4; wi++) {
        uint32_t word = get_u32(b->raw + ((int64_t)r * wpr + g * 4 + wi) * 4);
        float s1 = binary_word_sum1(x + g * 128 + wi * 32, word);
        acc += scale * (2 * s1 - sum_all[g * 4 + wi]);
      }
    }
    y[r] = acc;
  }
}
static void matvec_affine_rows(const wvo_blob *b, const float *x, float *y, const float *sum_x, int lo, int hi) {
  /* quant/affine_g64.go:229-268 */
  int group = b->block_weights > 0 ? b->block_weights : 64;
  int wpr = b->cols / 8, gpr = b->cols / group, wig = group / 8;
  for (int r = lo; r < hi; r++) {
    float acc = 0;
    for (int g = 0; g < gpr; g++) {
      float s = b->scales[(int64_t)r * gpr + g], beta = b->mins[(int64_t)r * gpr + g];
      float code_dot = 0;
      for (int wi = 0; wi < wig; wi++) {
        uint32_t word = get_u32(b->raw + ((int64_t)r * wpr + g * wig + wi) * 4);
        const float *xb = x + g * group + wi * 8;
        for (int j = 0; j < 8; j++) code_dot += (float)((word >> (j * 4)) & 15) * xb[j];
      }
      acc += s * code_dot + beta * sum_x[g];
    }
    y[r] = acc;
  }
}

/* y = W x following quant.MatVec for packed formats; for FormatNone it follows the route
 * Dense actually takes, weights.matVecNativeF64 (weights/native.go:1120-1137): decode each
 * weight to f64, accumulate in f64, cast the row sum to f32. */
int wvo_matvec(const wvo_blob *b, const float *x, float *y) {
  if (!b || !x || !y) return -1;
  int rows = b->rows, cols = b->cols;
  int64_t n = (int64_t)rows * cols;
  if (b->format == F_NONE) {
    for (int r = 0; r < rows; r++) {
      double sum = 0;
      for (int c = 0; c < cols; c++) {
        int64_t i = (int64_t)r * cols + c;
        float w;
        if (b->dtype == DT_F32) w = get_f32(b->raw + i * 4);
        else { uint16_t h; memcpy(&h, b->raw + i * 2, 2); w = b->dtype == DT_F16 ? f16_to_f32(h) : bf16_to_f32(h); }
        sum += (double)w * (double)x[c];
      }
      y[r] = (float)sum;
    }
    return 0;
  }
  if (binary_is_g128(b)) {
    int wpr = cols / 32;
    float *sum_all = malloc(sizeof(float) * wpr);
    for (int w = 0; w < wpr; w++) sum_all[w] = sum32(x + w * 32);
    matvec_binary_g128_rows(b, x, y, sum_all, 0, rows);
    free(sum_all);
    return 0;
  }
  if (b->format == F_AFFINE) {
    int group = b->block_weights > 0 ? b->block_weights : 64, gpr = cols / group;
    float *sum_x = malloc(sizeof(float) * gpr);
    for (int g = 0; g < gpr; g++) { float s = 0; for (int j = 0; j < group; j++) s += x[g * group + j]; sum_x[g] = s; }
    matvec_affine_rows(b, x, y, sum_x, 0, rows);
    free(sum_x);
    return 0;
  }
  /* All other formats: y[i/cols] += w_i * x[i%cols] with w_i exactly as Unpack yields it
   * (e.g. q4_0.go:106 float32(q)*scale*x, kquant.go:243-245), in flat index order. */
  float *w = malloc(sizeof(float) * (size_t)n);
  if (!w) return -4;
  int rc = wvo_unpack(b, w);
  if (rc) { free(w); return rc; }
  for (int r = 0; r < rows; r++) {
    float acc = 0;
    const float *wr = w + (int64_t)r * cols;
    for (int c = 0; c < cols; c++) acc += wr[c] * x[c];
    y[r] = acc;
  }
  free(w);
  return 0;
}

/* Σ_j |w_rj x_j| per row in f64: the denominator of the output tolerance. */
int wvo_sum_abs_wx(const wvo_blob *b, const float *x, double *out) {
  int64_t n = (int64_t)b->rows * b->cols;
  float *w = malloc(sizeof(float) * (size_t)n);
  if (!w) return -4;
  int rc = wvo_unpack(b, w);
  if (rc) { free(w); return rc; }
  for (int r = 0; r < b->rows; r++) {
    double s = 0;
    for (int c = 0; c < b->cols; c++) s += fabs((double)w[(int64_t)r * b->cols + c] * (double)x[c]);
    out[r] = s;
  }
  free(w);
  return 0;
}

/* ---------- SIMD path (dense.MatVecPackedBlob / ForwardSIMD): once-built caches + f64 dots ---------- */
typedef struct {
  int format, dtype, rows, cols, group;
  int has_dmin, mid, iq_kind, iq_group; float iq_mid;
  float *scales, *mins;  /* per block / group, absolute */
  int8_t *qs;            /* Int8QS: one byte per weight */
  uint32_t *q4;          /* Q4Packed words */
  float *f32;            /* F32Cache (ternary / binary g32) or FormatNone f32 */
  const wvo_blob *blob;  /* borrowed: binary g128, f16/bf16 native */
} simd_cache;

void wvo_simd_free(void *p) {
  simd_cache *c = p;
  if (!c) return;
  free(c->scales); free(c->mins); free(c->qs); free(c->q4); free(c->f32); free(c);
}

/* Builds what quant.EnsureQ4SIMDCache / EnsureQ8SIMDCache / EnsureFusedSIMDCache /
 * EnsureKSIMDCache / EnsureIQSIMDCache / EnsureAffineSIMDCache / EnsureFloatCache build
 * (quant/q4_simd.go, qx_simd.go, k_iq_simd.go). Not timed, as in the reference. */
void *wvo_simd_prepare(const wvo_blob *b) {
  simd_cache *c = calloc(1, sizeof *c);
  c->format = b->format; c->dtype = b->dtype; c->rows = b->rows; c->cols = b->cols; c->blob = b;
  c->group = b->block_weights;
  int64_t n = (int64_t)b->rows * b->cols;
  int64_t nb = (n + 31) / 32;
  kspec ks; iqspec is;
  switch (b->format) {
  case F_NONE:
    if (b->dtype == DT_F32) { c->f32 = malloc((size_t)n * 4); memcpy(c->f32, b->raw, (size_t)n * 4); }
    return c;
  case F_Q4_0: case F_Q4_1: {
    int bb = b->format == F_Q4_0 ? 20 : 24, qo = b->format == F_Q4_0 ? 4 : 8;
    c->scales = malloc(nb * 4); c->q4 = malloc(nb * 16);
    if (b->format == F_Q4_1) c->mins = malloc(nb * 4);
    for (int64_t bi = 0; bi < nb; bi++) {
      const uint8_t *o = b->raw + bi * bb;
      c->scales[bi] = get_f32(o);
      if (c->mins) c->mins[bi] = get_f32(o + 4);
      for (int k = 0; k < 4; k++) c->q4[bi * 4 + k] = get_u32(o + qo + k * 4);
    }
    return c;
  }
  case F_Q8_0: {
    c->scales = malloc(nb * 4); c->qs = malloc(nb * 32);
    for (int64_t bi = 0; bi < nb; bi++) {
      const uint8_t *o = b->raw + bi * 36;
      c->scales[bi] = get_f32(o);
      for (int j = 0; j < 32; j++) c->qs[bi * 32 + j] = (int8_t)o[4 + j];
    }
    return c;
  }
  case F_Q5_0: case F_Q5_1: {
    int is1 = b->format == F_Q5_1, bb = is1 ? 28 : 24;
    c->scales = malloc(nb * 4); c->qs = malloc(nb * 32);
    if (is1) c->mins = malloc(nb * 4);
    for (int64_t bi = 0; bi < nb; bi++) {
      const uint8_t *o = b->raw + bi * bb;
      c->scales[bi] = get_f32(o);
      if (is1) c->mins[bi] = get_f32(o + 4);
      bitr br = {o + (is1 ? 8 : 4), 20, 0};
      for (int j = 0; j < 32; j++) { int q = (int)br_read(&br, 5); c->qs[bi * 32 + j] = (int8_t)(is1 ? q : q - 16); }
    }
    return c;
  }
  case F_TERNARY: case F_BINARY:
    if (binary_is_g128(b)) return c;
    c->f32 = malloc((size_t)n * 4);
    wvo_unpack(b, c->f32);
    return c;
  case F_AFFINE: {
    int group = b->block_weights > 0 ? b->block_weights : 64;
    c->group = group;
    c->qs = malloc((size_t)n);
    int wpr = b->cols / 8;
    for (int r = 0; r < b->rows; r++) for (int w = 0; w < wpr; w++) {
      uint32_t word = get_u32(b->raw + ((int64_t)r * wpr + w) * 4);
      for (int j = 0; j < 8; j++) c->qs[(int64_t)r * b->cols + w * 8 + j] = (int8_t)((word >> (j * 4)) & 15);
    }
    c->scales = malloc(b->ns * 4); memcpy(c->scales, b->scales, b->ns * 4);
    c->mins = malloc(b->nm * 4); memcpy(c->mins, b->mins, b->nm * 4);
    return c;
  }
  }
  if (kspec_for(b->format, &ks)) {
    int sbb = k_super_bytes(ks);
    int64_t nsb = (int64_t)(b->nraw / sbb);
    c->qs = malloc(nsb * 256); c->scales = malloc(nsb * 16 * 4); c->mins = calloc(nsb * 16, 4);
    c->has_dmin = ks.has_dmin; c->mid = ks.mid;
    for (int64_t si = 0; si < nsb; si++) {
      const uint8_t *o = b->raw + si * sbb;
      float d = get_f32(o), dmin = get_f32(o + 4);
      int qoff = ks.has_dmin ? 40 : 24;
      bitr br = {o + qoff, (uint64_t)(sbb - qoff), 0};
      for (int g = 0; g < 16; g++) {
        float sc = d * (float)o[8 + g] / 255;
        if (sc == 0) sc = d / 255;
        c->scales[si * 16 + g] = sc;
        if (ks.has_dmin) c->mins[si * 16 + g] = dmin * (float)(int8_t)o[24 + g] / 127;
        for (int j = 0; j < 16; j++) c->qs[si * 256 + g * 16 + j] = (int8_t)br_read(&br, ks.bits);
      }
    }
    return c;
  }
  if (iqspec_for(b->format, &is)) {
    int64_t padn = (n + is.group - 1) / is.group * is.group;
    c->qs = malloc(padn);
    bitr br = {b->raw, b->nraw, 0};
    for (int64_t i = 0; i < padn; i++) c->qs[i] = (int8_t)br_read(&br, is.bits);
    c->scales = malloc(b->ns * 4); memcpy(c->scales, b->scales, b->ns * 4);
    c->iq_group = is.group; c->iq_mid = is.mid;
    c->iq_kind = is.bits == 1 ? 1 : (is.nonlinear ? 2 : 0);
    return c;
  }
  free(c);
  return NULL;
}

/* 32-weight block dots restating the Plan 9 kernels. Eight f64 partial sums a[0..7]
 * (four 2-lane registers), weight j of each 8-chunk goes to a[j]; reduction tree
 * ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)); then times scale (simd/dot_q4_amd64.s:24-102,
 * dot_qx_amd64.s:11-61). f32*int products are exact in f64, so fused and unfused agree. */
#if defined(__x86_64__)
__attribute__((target("avx2,fma")))
static inline double block_dot32_i8_avx2(const float *in, const int8_t *qs, float scale) {
  __m128d a0 = _mm_setzero_pd(), a1 = a0, a2 = a0, a3 = a0;
  for (int c = 0; c < 4; c++) {
    int32_t w0, w1; memcpy(&w0, qs + c * 8, 4); memcpy(&w1, qs + c * 8 + 4, 4);
    __m128 q0 = _mm_cvtepi32_ps(_mm_cvtepi8_epi32(_mm_cvtsi32_si128(w0)));
    __m128 q1 = _mm_cvtepi32_ps(_mm_cvtepi8_epi32(_mm_cvtsi32_si128(w1)));
    __m128 x0 = _mm_loadu_ps(in + c * 8), x1 = _mm_loadu_ps(in + c * 8 + 4);
    a0 = _mm_fmadd_pd(_mm_cvtps_pd(q0), _mm_cvtps_pd(x0), a0);
    a1 = _mm_fmadd_pd(_mm_cvtps_pd(_mm_movehl_ps(q0, q0)), _mm_cvtps_pd(_mm_movehl_ps(x0, x0)), a1);
    a2 = _mm_fmadd_pd(_mm_cvtps_pd(q1), _mm_cvtps_pd(x1), a2);
    a3 = _mm_fmadd_pd(_mm_cvtps_pd(_mm_movehl_ps(q1, q1)), _mm_cvtps_pd(_mm_movehl_ps(x1, x1)), a3);
  }
  a0 = _mm_add_pd(a0, a2); a1 = _mm_add_pd(a1, a3); a0 = _mm_add_pd(a0, a1);
  double lo = _mm_cvtsd_f64(a0), hi = _mm_cvtsd_f64(_mm_unpackhi_pd(a0, a0));
  return (lo + hi) * (double)scale;
}
__attribute__((target("avx2,fma")))
static inline double dot_f32_acc_f64_avx2(const float *x, const float *w, int n, double prev) {
  /* simd/avx2_amd64.s:14-79 */
  __m128d a0 = _mm_setzero_pd(), a1 = a0, a2 = a0, a3 = a0;
  int i = 0;
  for (; i + 8 <= n; i += 8) {
    __m128 x0 = _mm_loadu_ps(x + i), x1 = _mm_loadu_ps(x + i + 4), w0 = _mm_loadu_ps(w + i), w1 = _mm_loadu_ps(w + i + 4);
    a0 = _mm_fmadd_pd(_mm_cvtps_pd(w0), _mm_cvtps_pd(x0), a0);
    a1 = _mm_fmadd_pd(_mm_cvtps_pd(_mm_movehl_ps(w0, w0)), _mm_cvtps_pd(_mm_movehl_ps(x0, x0)), a1);
    a2 = _mm_fmadd_pd(_mm_cvtps_pd(w1), _mm_cvtps_pd(x1), a2);
    a3 = _mm_fmadd_pd(_mm_cvtps_pd(_mm_movehl_ps(w1, w1)), _mm_cvtps_pd(_mm_movehl_ps(x1, x1)), a3);
  }
  a0 = _mm_add_pd(a0, a2); a1 = _mm_add_pd(a1, a3); a0 = _mm_add_pd(a0, a1);
  double s = _mm_cvtsd_f64(a0) + _mm_cvtsd_f64(_mm_unpackhi_pd(a0, a0));
  s += prev;
  for (; i < n; i++) s += (double)x[i] * (double)w[i];
  return s;
}
static int have_avx2(void) { static int v = -1; if (v < 0) v = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma"); return v; }
#else
static int have_avx2(void) { return 0; }
#endif

static int g_force_scalar = 0;
void wvo_force_scalar(int on) { g_force_scalar = on; }

static inline double block_dot32_i8_scalar(const float *in, const int8_t *qs, float scale) {
  double a[8] = {0};
  for (int c = 0; c < 4; c++) for (int j = 0; j < 8; j++) a[j] += (double)(float)qs[c * 8 + j] * (double)in[c * 8 + j];
  double lo = (a[0] + a[4]) + (a[2] + a[6]), hi = (a[1] + a[5]) + (a[3] + a[7]);
  return (lo + hi) * (double)scale;
}
static inline double block_dot32_i8(const float *in, const int8_t *qs, float scale) {
#if defined(__x86_64__)
  if (have_avx2() && !g_force_scalar) return block_dot32_i8_avx2(in, qs, scale);
#endif
  return block_dot32_i8_scalar(in, qs, scale);
}
static inline double dot_f32_acc_f64(const float *x, const float *w, int n, double prev) {
#if defined(__x86_64__)
  if (have_avx2() && !g_force_scalar) return dot_f32_acc_f64_avx2(x, w, n, prev);
#endif
  double a[8] = {0};
  int i = 0;
  for (; i + 8 <= n; i += 8) for (int j = 0; j < 8; j++) a[j] += (double)x[i + j] * (double)w[i + j];
  double s = ((a[0] + a[4]) + (a[2] + a[6])) + ((a[1] + a[5]) + (a[3] + a[7]));
  s += prev;
  for (; i < n; i++) s += (double)x[i] * (double)w[i];
  return s;
}
static inline void q4_unpack_block(const uint32_t *p4, int8_t *q, int sign_extend) {
  /* nibble k of word w is weight 8w+k (simd/dot_q4.go:44-58) */
  for (int w = 0; w < 4; w++) for (int k = 0; k < 8; k++) {
    int v = (p4[w] >> (k * 4)) & 0xF;
    if (sign_extend && v > 7) v -= 16;
    q[w * 8 + k] = (int8_t)v;
  }
}
static inline double block_sum_x_q41(const float *in) { /* X12 accumulator of q41BlockDot32Avx2 */
  double l0 = 0, l1 = 0;
  for (int c = 0; c < 4; c++) for (int p = 0; p < 4; p++) { l0 += (double)in[c * 8 + p * 2]; l1 += (double)in[c * 8 + p * 2 + 1]; }
  return l0 + l1;
}

/* One output row through the fused SIMD-path dot for the cache's format. */
static float simd_row(const simd_cache *c, const float *x, int r, const float *aux) {
  int cols = c->cols;
  int64_t base = (int64_t)r * cols;
  double sum = 0;
  switch (c->format) {
  case F_NONE:
    if (c->dtype == DT_F32) return (float)dot_f32_acc_f64(x, c->f32 + base, cols, 0);
    { /* simd/dot_lowp.go:50-74, dot_lowp_amd64.go:13-35: tiles of 8 through DotTile */
      float buf[8];
      for (int i = 0; i < cols;) {
        int m = cols - i < 8 ? cols - i : 8;
        for (int k = 0; k < m; k++) {
          uint16_t h; memcpy(&h, c->blob->raw + (base + i + k) * 2, 2);
          buf[k] = c->dtype == DT_F16 ? f16_to_f32(h) : bf16_to_f32(h);
        }
        sum = dot_f32_acc_f64(x + i, buf, m, sum);
        i += m;
      }
      return (float)sum;
    }
  case F_TERNARY:
    return (float)dot_f32_acc_f64(x, c->f32 + base, cols, 0);
  case F_BINARY:
    return (float)dot_f32_acc_f64(x, c->f32 + base, cols, 0); /* g128 never reaches here */
  case F_Q4_0: case F_Q4_1: { /* simd/dot_q4_amd64.go:8-38, dot_qx_amd64.go:43-73 */
    int i = 0;
    if (base % 32 == 0) for (; i + 32 <= cols; i += 32) {
      int64_t blk = (base + i) / 32;
      int8_t q[32];
      q4_unpack_block(c->q4 + (base + i) / 8, q, c->format == F_Q4_0);
      double d = block_dot32_i8(x + i, q, c->scales[blk]);
      if (c->format == F_Q4_1) d += block_sum_x_q41(x + i) * (double)c->mins[blk];
      sum += d;
    }
    /* Scalar tails (dot_q4.go:66-76, dot_qx.go:113-119). When a row does not start on a
     * 32-boundary the reference Q4_0 SIMD driver goes through dotQ4_0RowFusedTile, which
     * indexes words by globalIdx/8 without the nibble offset; SIMD-path parity is therefore
     * only asserted for cols % 32 == 0 and ragged shapes are checked against wvo_matvec. */
    for (; i < cols; i++) {
      int64_t gi = base + i;
      int v = (c->q4[gi / 8] >> ((gi % 8) * 4)) & 0xF;
      if (c->format == F_Q4_0) { if (v > 7) v -= 16; sum += (double)x[i] * (double)v * (double)c->scales[gi / 32]; }
      else sum += (double)x[i] * ((double)c->mins[gi / 32] + (double)v * (double)c->scales[gi / 32]);
    }
    return (float)sum;
  }
  case F_Q8_0: case F_Q5_0: { /* simd/dot_qx_amd64.go:13-27, dot_qx.go:39-59 */
    int i = 0;
    if (base % 32 == 0) for (; i + 32 <= cols; i += 32) sum += block_dot32_i8(x + i, c->qs + base + i, c->scales[(base + i) / 32]);
    for (; i < cols; i++) sum += (double)x[i] * (double)c->qs[base + i] * (double)c->scales[(base + i) / 32];
    return (float)sum;
  }
  case F_Q5_1: { /* simd/dot_qx.go:134-166 */
    int i = 0;
    if (base % 32 == 0) for (; i + 32 <= cols; i += 32) {
      int64_t blk = (base + i) / 32;
      double sc = c->scales[blk], mn = c->mins[blk], accq = 0, sumx = 0;
      for (int j = 0; j < 32; j++) { double xi = x[i + j]; accq += xi * (double)(uint8_t)c->qs[base + i + j]; sumx += xi; }
      sum += accq * sc + mn * sumx;
    }
    for (; i < cols; i++) { int64_t blk = (base + i) / 32; sum += (double)x[i] * ((double)c->mins[blk] + (double)(uint8_t)c->qs[base + i] * (double)c->scales[blk]); }
    return (float)sum;
  }
  case F_AFFINE: { /* simd/dot_k.go:140-165; aux = AffineSumX */
    int group = c->group, groups = cols / group;
    int64_t sb = (int64_t)r * groups;
    for (int g = 0; g < groups; g++) {
      double sc = c->scales[sb + g], beta = c->mins[sb + g], accq = 0;
      for (int j = 0; j < group; j++) accq += (double)x[g * group + j] * (double)(uint8_t)c->qs[base + g * group + j];
      sum += accq * sc + beta * (double)aux[g];
    }
    return (float)sum;
  }
  }
  kspec ks; iqspec is;
  if (kspec_for(c->format, &ks)) { /* simd/dot_k.go:25-74 */
    int i = 0;
    if (base % 16 == 0) for (; i + 16 <= cols; i += 16) {
      int64_t g = (base + i) / 16;
      double sc = c->scales[g];
      if (c->has_dmin) {
        double mn = c->mins[g], accq = 0, sumx = 0;
        for (int j = 0; j < 16; j++) { double xi = x[i + j]; accq += xi * (double)(uint8_t)c->qs[base + i + j]; sumx += xi; }
        sum += accq * sc + mn * sumx;
      } else {
        double acc = 0;
        for (int j = 0; j < 16; j++) acc += (double)x[i + j] * (double)((int)(uint8_t)c->qs[base + i + j] - c->mid);
        sum += acc * sc;
      }
    }
    for (; i < cols; i++) {
      int64_t g = (base + i) / 16; int q = (uint8_t)c->qs[base + i];
      if (c->has_dmin) sum += (double)x[i] * ((double)c->mins[g] + (double)q * (double)c->scales[g]);
      else sum += (double)x[i] * (double)c->scales[g] * (double)(q - c->mid);
    }
    return (float)sum;
  }
  if (iqspec_for(c->format, &is)) { /* simd/dot_k.go:78-136 */
    int sg = c->iq_group, i = 0;
    if (base % sg == 0) for (; i + sg <= cols; i += sg) {
      double sc = c->scales[(base + i) / sg], acc = 0;
      for (int j = 0; j < sg; j++) {
        uint8_t q = (uint8_t)c->qs[base + i + j];
        double code = c->iq_kind == 1 ? ((q & 1) ? 1.0 : -1.0) : (c->iq_kind == 2 ? (double)iq4nl_grid[q & 15] : (double)q - (double)c->iq_mid);
        acc += (double)x[i + j] * code;
      }
      sum += acc * sc;
    }
    for (; i < cols; i++) {
      double sc = c->scales[(base + i) / sg]; uint8_t q = (uint8_t)c->qs[base + i];
      double code = c->iq_kind == 1 ? ((q & 1) ? 1.0 : -1.0) : (c->iq_kind == 2 ? (double)iq4nl_grid[q & 15] : (double)q - (double)c->iq_mid);
      sum += (double)x[i] * code * sc;
    }
    return (float)sum;
  }
  return 0;
}

typedef struct { const simd_cache *c; const float *x; float *y; const float *aux; int lo, hi; } simd_job;
static void simd_rows(const simd_job *j) {
  const simd_cache *c = j->c;
  int cols = c->cols, r = j->lo;
  if (c->format == F_BINARY && !c->f32) { /* g128: native packed rows, quant/binary_g128.go:214-239 */
    matvec_binary_g128_rows(c->blob, j->x, j->y, j->aux, j->lo, j->hi);
    return;
  }
  /* Rows4 drivers keep the activation block hot across four rows
   * (simd/dot_q4_amd64.go:25-38, dot_qx_amd64.go:29-41,59-73). Per-row arithmetic is unchanged. */
  if (cols % 32 == 0 && (c->format == F_Q8_0 || c->format == F_Q5_0)) {
    for (; r + 3 < j->hi; r += 4) {
      double acc[4] = {0, 0, 0, 0};
      for (int i = 0; i < cols; i += 32)
        for (int k = 0; k < 4; k++) { int64_t bw = (int64_t)(r + k) * cols + i; acc[k] += block_dot32_i8(j->x + i, c->qs + bw, c->scales[bw / 32]); }
      for (int k = 0; k < 4; k++) j->y[r + k] = (float)acc[k];
    }
  } else if (cols % 32 == 0 && (c->format == F_Q4_0 || c->format == F_Q4_1)) {
    for (; r + 3 < j->hi; r += 4) {
      double acc[4] = {0, 0, 0, 0};
      for (int i = 0; i < cols; i += 32) {
        double sx = c->format == F_Q4_1 ? block_sum_x_q41(j->x + i) : 0;
        for (int k = 0; k < 4; k++) {
          int64_t bw = (int64_t)(r + k) * cols + i;
          int8_t q[32];
          q4_unpack_block(c->q4 + bw / 8, q, c->format == F_Q4_0);
          double d = block_dot32_i8(j->x + i, q, c->scales[bw / 32]);
          if (c->format == F_Q4_1) d += sx * (double)c->mins[bw / 32];
          acc[k] += d;
        }
      }
      for (int k = 0; k < 4; k++) j->y[r + k] = (float)acc[k];
    }
  }
  for (; r < j->hi; r++) j->y[r] = simd_row(c, j->x, r, j->aux);
}
static void *simd_thread(void *p) { simd_rows(p); return NULL; }

/* Formats whose reference SIMD driver shards rows over goroutines (gemv*ParallelF32,
 * quant/binary_g128.go:172-201). FormatNone f32/f16/bf16 loop serially over rows
 * (layers/dense/simd.go:201-215,253-284). */
static int format_is_row_parallel(const simd_cache *c) { return c->format != F_NONE; }

/* y = W x on the SIMD path. threads<=0 means all online cores (GOMAXPROCS default).
 * Returns the worker count actually used (1 when serial), <0 on error. */
int wvo_simd_matvec(void *cache, const float *x, float *y, int threads) {
  simd_cache *c = cache;
  if (!c || !x || !y) return -1;
  int rows = c->rows, cols = c->cols;
  float *aux = NULL;
  if (c->format == F_AFFINE) { /* simd.AffineSumX, f32 */
    int g = c->group, groups = cols / g;
    aux = malloc(sizeof(float) * groups);
    for (int k = 0; k < groups; k++) { float s = 0; for (int j = 0; j < g; j++) s += x[k * g + j]; aux[k] = s; }
  } else if (c->format == F_BINARY && !c->f32) {
    aux = malloc(sizeof(float) * (cols / 32));
    for (int w = 0; w < cols / 32; w++) aux[w] = sum32(x + w * 32);
  }
  if (threads <= 0) { threads = (int)sysconf(_SC_NPROCESSORS_ONLN); if (threads < 1) threads = 1; }
  int workers = threads;
  if (rows < 64 || threads < 2 || !format_is_row_parallel(c)) workers = 1;
  if (workers > rows) workers = rows;
  if (workers == 1) {
    simd_job j = {c, x, y, aux, 0, rows};
    simd_rows(&j);
  } else { /* layers/dense/gemv_parallel.go:12-42 */
    int chunk = (rows + workers - 1) / workers;
    pthread_t *th = malloc(sizeof(pthread_t) * workers);
    simd_job *jobs = malloc(sizeof(simd_job) * workers);
    int started = 0;
    for (int w = 0; w < workers; w++) {
      int lo = w * chunk, hi = lo + chunk > rows ? rows : lo + chunk;
      if (lo >= hi) break;
      jobs[w] = (simd_job){c, x, y, aux, lo, hi};
      pthread_create(&th[w], NULL, simd_thread, &jobs[w]);
      started++;
    }
    for (int w = 0; w < started; w++) pthread_join(th[w], NULL);
    free(th); free(jobs);
    workers = started;
  }
  free(aux);
  return workers;
}

int wvo_matvec_simd(const wvo_blob *b, const float *x, float *y, int threads) {
  void *c = wvo_simd_prepare(b);
  if (!c) return -2;
  int rc = wvo_simd_matvec(c, x, y, threads);
  wvo_simd_free(c);
  return rc < 0 ? rc : 0;
}

/* ---------- packed wire (weights/packed_wire.go:30-110) ---------- */
uint64_t wvo_wire_size(const wvo_blob *b) {
  if (b->format == F_NONE) return b->nraw;
  return 12 + b->ns * 4 + b->nm * 4 + b->nraw;
}
int wvo_wire_encode(const wvo_blob *b, uint8_t *out) {
  if (b->format == F_NONE) { memcpy(out, b->raw, b->nraw); return 0; }
  uint32_t ns = (uint32_t)b->ns, nm = (uint32_t)b->nm, nr = (uint32_t)b->nraw;
  put_u32(out, ns); put_u32(out + 4, nm); put_u32(out + 8, nr);
  memcpy(out + 12, b->scales, (size_t)ns * 4);
  memcpy(out + 12 + (size_t)ns * 4, b->mins, (size_t)nm * 4);
  memcpy(out + 12 + (size_t)ns * 4 + (size_t)nm * 4, b->raw, nr);
  return 0;
}
/* Fills counts and offsets of the three arrays inside the wire buffer and re-infers
 * BlockWeights the way DecodePackedWire + InferBinaryBlockWeights do. */
int wvo_wire_decode(int format, int rows, int cols, const uint8_t *wire, uint64_t n,
                    uint64_t *ns, uint64_t *nm, uint64_t *nr, uint64_t *off_scales,
                    uint64_t *off_mins, uint64_t *off_raw, int *block_weights) {
  *block_weights = 0;
  if (format == F_NONE) {
    uint64_t need = (uint64_t)rows * cols * 4;
    if (n < need) return -3;
    *ns = *nm = 0; *nr = need; *off_scales = *off_mins = *off_raw = 0; *block_weights = 1;
    return 0;
  }
  if (n < 12) return -3;
  *ns = get_u32(wire); *nm = get_u32(wire + 4); *nr = get_u32(wire + 8);
  if (n < 12 + *ns * 4 + *nm * 4 + *nr) return -3;
  *off_scales = 12; *off_mins = 12 + *ns * 4; *off_raw = *off_mins + *nm * 4;
  if (format == F_BINARY) {
    *block_weights = 32;
    if (cols > 0 && cols % 128 == 0 && *ns == (uint64_t)rows * (cols / 128)) *block_weights = 128;
  }
  return 0;
}

/* ---------- greedy sampling (model/sampling/argmax.go:4-18) ----------
 * First index of the strict maximum: `v > maxVal` never holds for NaN, so NaN never wins, and a
 * NaN in position 0 keeps index 0. Empty input returns 0. */
int wvo_argmax(const float *logits, int64_t n) {
  if (n <= 0) return 0;
  int64_t max_idx = 0;
  float max_val = logits[0];
  for (int64_t i = 0; i < n; i++) {
    float v = logits[i];
    if (v > max_val) { max_val = v; max_idx = i; }
  }
  return (int)max_idx;
}

/* ---------- pointwise activation (core/activate.go:6-38, values core/layer.go:91-98) ----------
 * core.Activate in float64. An unknown value comes back unchanged, as in the reference's
 * default arm; *known (may be NULL) reports whether the value is one of the eight. */
double wvo_activate(double x, int act, int *known) {
  if (known) *known = 1;
  switch (act) {
  case -1: return x;                                   /* ActivationLinear */
  case 0: return x < 0 ? 0.0 : x;                      /* ActivationReLU */
  case 6: return x < 0 ? 0.0 : x * x;                  /* ActivationReLU2 */
  case 5: return x < 0 ? 0.01 * x : x;                 /* ActivationLeakyReLU */
  case 1: return x / (1 + exp(-x));                    /* ActivationSilu */
  case 2: return 0.5 * x * (1 + tanh(sqrt(2 / M_PI) * (x + 0.044715 * x * x * x)));  /* ActivationGELU */
  case 3: return tanh(x);                              /* ActivationTanh */
  case 4: return 1 / (1 + exp(-x));                    /* ActivationSigmoid */
  }
  if (known) *known = 0;
  return x;
}

/* ---------- decode steps between the projections (host float64 arithmetic of the reference) ---------- */

/* rmsnorm.forwardHost, scalar arm, T = float32 (layers/rmsnorm/cpu.go:76-85): per token row
 * inv = 1 / sqrt(sum(x^2) / dim + eps); xhat = x * inv; y = xhat * gamma, each cast to float32. */
void wvo_rmsnorm(const float *x, const float *gamma, float *xhat, float *y, int ntok, int dim, double eps) {
  for (int t = 0; t < ntok; t++) {
    const float *row = x + (size_t)t * dim;
    double sum_sq = 0;
    for (int i = 0; i < dim; i++) { double v = (double)row[i]; sum_sq += v * v; }
    double inv = 1.0 / sqrt(sum_sq / (double)dim + eps);
    for (int i = 0; i < dim; i++) {
      double xh = (double)row[i] * inv;
      if (xhat) xhat[(size_t)t * dim + i] = (float)xh;
      y[(size_t)t * dim + i] = (float)(xh * (double)gamma[i]);
    }
  }
}

/* applyRoPE (layers/mha/rope.go:6-21): rotates pairs (d, d + headDim/2) in place. */
void wvo_rope(double *vec, int pos, int num_heads, int head_dim, double theta) {
  int half = head_dim / 2;
  if (half <= 0 || theta <= 0) return;
  for (int h = 0; h < num_heads; h++) {
    int base = h * head_dim;
    for (int d = 0; d < half; d++) {
      double angle = (double)pos / pow(theta, (double)(2 * d) / (double)head_dim);
      double c = cos(angle), s = sin(angle);
      double v0 = vec[base + d], v1 = vec[base + d + half];
      vec[base + d] = v0 * c - v1 * s;
      vec[base + d + half] = v0 * s + v1 * c;
    }
  }
}

/* attnForward (layers/mha/attn.go:15-120) for seqLen 1, standard softmax, every cache position
 * 0 .. kvLen-1 allowed (the causal mask for the query at position kvLen-1), no ALiBi, no dropout.
 * Q [numHeads*headDim]; cacheK / cacheV [msl][numKVHeads*headDim], position p in row p % msl. */
void wvo_attn_decode(const double *q, const double *cache_k, const double *cache_v, double *out, int num_heads,
                     int num_kv_heads, int head_dim, int kv_len, int msl, double scale) {
  int heads_per_kv = num_heads / num_kv_heads, kv_dim = num_kv_heads * head_dim;
  double *scores = (double *)malloc(sizeof(double) * (size_t)(kv_len > 0 ? kv_len : 1));
  for (int h = 0; h < num_heads; h++) {
    int kv_head = h / heads_per_kv, q_off = h * head_dim;
    double max_score = -1e9;
    for (int kp = 0; kp < kv_len; kp++) {
      size_t kb = (size_t)(kp % msl) * kv_dim + (size_t)kv_head * head_dim;
      double dot = 0;
      for (int d = 0; d < head_dim; d++) dot += q[q_off + d] * cache_k[kb + d];
      double score = dot * scale;
      scores[kp] = score;
      if (score > max_score) max_score = score;
    }
    if (kv_len == 0) { for (int d = 0; d < head_dim; d++) out[q_off + d] = 0; continue; }
    double exp_sum = 0;
    for (int i = 0; i < kv_len; i++) { scores[i] = exp(scores[i] - max_score); exp_sum += scores[i]; }
    double inv = 1.0 / exp_sum;
    for (int i = 0; i < kv_len; i++) scores[i] *= inv;
    for (int d = 0; d < head_dim; d++) {
      double sum = 0;
      for (int kp = 0; kp < kv_len; kp++) sum += scores[kp] * cache_v[(size_t)(kp % msl) * kv_dim + (size_t)kv_head * head_dim + d];
      out[q_off + d] = sum;
    }
  }
  free(scores);
}

/* simd.SiluMulF32 (simd/silu.go:14-27): out[i] = float32(g / (1 + exp(-g)) * up[i]), g = float64(gate[i]). */
void wvo_silu_mul(const float *gate, const float *up, float *out, int n) {
  for (int i = 0; i < n; i++) {
    double g = (double)gate[i];
    out[i] = (float)(g / (1 + exp(-g)) * (double)up[i]);
  }
}

/* ---------- quant.DecodeRow (quant/decode_row.go:7-187, binary_g128.go:130-157, affine_g64.go:121-175) ----------
 * One output row of a packed blob. Q8_0, Q4_0, ternary and binary walk the flat index themselves; the row-aligned
 * layouts walk their words; everything else copies the row out of a full Unpack. FormatNone is refused (-2), a row
 * out of range or a short dst is a shape error (-1). */
int wvo_decode_row(const wvo_blob *b, int row, float *dst, int64_t ndst) {
  if (!b) return -2;
  if (row < 0 || row >= b->rows || ndst < b->cols) return -1;
  const int cols = b->cols;
  const int64_t base = (int64_t)row * cols, n = (int64_t)b->rows * cols;
  switch (b->format) {
  case F_NONE: return -2;
  case F_Q8_0:
    for (int c = 0; c < cols; c++) {
      int64_t i = base + c, bi = i / 32, j = i % 32, off = bi * 36;
      if ((uint64_t)(off + 4 + j) >= b->nraw || i >= n) { dst[c] = 0; continue; }
      dst[c] = (float)(int8_t)b->raw[off + 4 + j] * get_f32(b->raw + off);
    }
    return 0;
  case F_Q4_0:
    for (int c = 0; c < cols; c++) {
      int64_t i = base + c;
      if (i >= n) { dst[c] = 0; continue; }
      int64_t bi = i / 32, j = i % 32, off = bi * 20;
      if ((uint64_t)(off + 4 + j / 2) >= b->nraw) { dst[c] = 0; continue; }
      uint8_t w = b->raw[off + 4 + j / 2];
      int8_t q = (int8_t)((j % 2 == 0) ? (w & 0xF) : (w >> 4));
      if (q > 7) q -= 16;
      dst[c] = (float)q * get_f32(b->raw + off);
    }
    return 0;
  case F_TERNARY:
    for (int c = 0; c < cols; c++) {
      int64_t i = base + c;
      if (i >= n) { dst[c] = 0; continue; }
      int64_t g = i / 16, j = i % 16;
      if ((uint64_t)(g * 4 + 4) > b->nraw) { dst[c] = 0; continue; }
      uint32_t code = (get_u32(b->raw + g * 4) >> (j * 2)) & 3;
      float scale = (uint64_t)g < b->ns ? b->scales[g] : 1.0f;
      dst[c] = code == 0 ? -scale : (code == 2 ? scale : 0.0f);
    }
    return 0;
  case F_BINARY:
    if (binary_is_g128(b)) {
      int gpr = cols / 128, wpr = cols / 32;
      for (int g = 0; g < gpr; g++) {
        int64_t si = (int64_t)row * gpr + g;
        float scale = (uint64_t)si < b->ns ? b->scales[si] : 1.0f;
        for (int wi = 0; wi < 4; wi++) {
          uint32_t word = get_u32(b->raw + ((int64_t)row * wpr + g * 4 + wi) * 4);
          for (int j = 0; j < 32; j++) dst[g * 128 + wi * 32 + j] = ((word >> j) & 1) ? scale : -scale;
        }
      }
      return 0;
    }
    for (int c = 0; c < cols; c++) {
      int64_t i = base + c;
      if (i >= n) { dst[c] = 0; continue; }
      int64_t g = i / 32, j = i % 32;
      if ((uint64_t)(g * 4 + 4) > b->nraw) { dst[c] = 0; continue; }
      float scale = (uint64_t)g < b->ns ? b->scales[g] : 1.0f;
      dst[c] = ((get_u32(b->raw + g * 4) >> j) & 1) ? scale : -scale;
    }
    return 0;
  case F_AFFINE: {
    int group = b->block_weights > 0 ? b->block_weights : 64;
    int wpr = cols / 8, gpr = cols / group, wig = group / 8;
    for (int g = 0; g < gpr; g++) {
      int64_t si = (int64_t)row * gpr + g;
      float s = (uint64_t)si < b->ns ? b->scales[si] : 1.0f;
      float beta = (uint64_t)si < b->nm ? b->mins[si] : 0.0f;
      for (int wi = 0; wi < wig; wi++) {
        uint32_t word = get_u32(b->raw + ((int64_t)row * wpr + g * wig + wi) * 4);
        for (int j = 0; j < 8; j++) dst[g * group + wi * 8 + j] = s * (float)((word >> (j * 4)) & 15) + beta;
      }
    }
    return 0;
  }
  default: {
    float *all = (float *)malloc((size_t)n * sizeof(float));
    if (!all) return -4;
    int rc = wvo_unpack(b, all);
    if (!rc) memcpy(dst, all + base, (size_t)cols * sizeof(float));
    free(all);
    return rc;
  }
  }
}

/* ---------- top-K sampling (model/sampling/topk.go:11-50) ----------
 * Greedy when top_k == 1, temperature <= 0 or deterministic. Otherwise candidates are logit / temperature (float32),
 * sorted by value descending, cut to top_k when 0 < top_k < n; p_i = exp(float64(val_i - max)) with the subtraction
 * in float32; r = u * sum, and the first i with r <= running sum wins, else the last candidate. `u` stands for the
 * reference's rand.Float64(). sort.Slice is not stable, so the order of equal values is open in the reference; this
 * restatement orders them by rising index. */
typedef struct { int32_t idx; float val; } topk_pair;
static int topk_cmp(const void *a, const void *b) {
  const topk_pair *p = (const topk_pair *)a, *q = (const topk_pair *)b;
  if (p->val > q->val) return -1;
  if (p->val < q->val) return 1;
  return p->idx < q->idx ? -1 : (p->idx > q->idx ? 1 : 0);
}
int wvo_topk_sample(const float *logits, int64_t n, int top_k, float temperature, int deterministic, double u) {
  if (n <= 0) return 0;
  if (top_k == 1 || temperature <= 0 || deterministic) return wvo_argmax(logits, n);
  topk_pair *cands = (topk_pair *)malloc((size_t)n * sizeof(topk_pair));
  if (!cands) return -1;
  for (int64_t i = 0; i < n; i++) { cands[i].idx = (int32_t)i; cands[i].val = logits[i] / temperature; }
  qsort(cands, (size_t)n, sizeof(topk_pair), topk_cmp);
  int64_t k = (top_k > 0 && top_k < n) ? top_k : n;
  float maxv = cands[0].val;
  double *probs = (double *)malloc((size_t)k * sizeof(double));
  if (!probs) { free(cands); return -1; }
  double sum = 0;
  for (int64_t i = 0; i < k; i++) { float d = cands[i].val - maxv; probs[i] = exp((double)d); sum += probs[i]; }
  double r = u * sum, acc = 0.0;
  int pick = cands[k - 1].idx;
  for (int64_t i = 0; i < k; i++) { acc += probs[i]; if (r <= acc) { pick = cands[i].idx; break; } }
  free(probs); free(cands);
  return pick;
}
