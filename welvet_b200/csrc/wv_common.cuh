// Shared definitions for the Welvet CUDA backend: format table, device-resident blob
// layout, and the index helpers every kernel (re-layout, unpack, pack, GEMV) agrees on.
//
// Device layout. A packed blob arrives in the reference's wire layout (quant/pack.go,
// weights/packed_wire.go) and is re-laid-out once at upload into bit planes that can be
// streamed with aligned vector loads. Bytes per weight never grow:
//
//   lo plane   BITS_LO bits per code, codes in flat-index order, LSB-first inside u32 words
//              (for 2/4-bit k-quants, IQ, ternary, binary and affine this is the wire stream
//              itself; Q4_0 stores code^8 and Q8_0 stores code^0x80 so that every format
//              decodes as (unsigned code - mid)).
//   hi plane   BITS_HI extra high bits per code for 3/5/6-bit formats, stored per 32-weight
//              chunk in "byte-spread" order: the bits for the four codes that share a byte
//              lane position sit 8 bits apart, so one shift + one logic op merges them
//              into the four byte lanes extracted from the lo plane.
//   params     classic blocks: f32 scale (and min) per 32 weights, split out of Raw;
//              k-quants: float2 {d, dmin} per 256 weights plus one u32 (u16 for Q6_K) per
//              32 weights holding {scale[g], scale[g+1], min[g], min[g+1]} bytes;
//              IQ / ternary / binary / affine: the wire's own Scales / Mins arrays.
//
// Within a 32-weight chunk, code j is addressed by (w, s, m): w = word of the lo plane,
// s = shift index, m = byte lane, with j = w*CPW + m*SPW + s, CPW = 32/BITS_LO codes per
// word, SPW = 8/BITS_LO shifts per word. k = w*SPW + s (0..7) names one group of four
// codes that are extracted together as the four bytes of ((lo[w] >> (BITS_LO*s)) & mask).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "welvet_cuda.h"  // status codes of the C ABI

// quant.Format values (reference quant/format.go:9-39)
enum WvFormat : int {
  WV_NONE = 0, WV_Q8_0 = 1, WV_Q4_0 = 2, WV_Q4_1 = 3, WV_Q5_0 = 4, WV_Q5_1 = 5,
  WV_Q2_K = 6, WV_Q3_K = 7, WV_Q4_K = 8, WV_Q5_K = 9, WV_Q6_K = 10,
  WV_IQ1_S = 11, WV_IQ2_XXS = 12, WV_IQ2_XS = 13, WV_IQ3_XXS = 14, WV_IQ3_S = 15,
  WV_IQ4_NL = 16, WV_IQ4_XS = 17, WV_TERNARY = 18, WV_BINARY = 19, WV_AFFINE = 20,
  WV_FORMAT_COUNT = 21
};
// core.DType values accepted for FormatNone (reference core/dtype.go:15-17)
enum WvDType : int { WV_DT_F32 = 1, WV_DT_F16 = 2, WV_DT_BF16 = 3 };

enum WvKind : int { WK_NONE = 0, WK_CLASSIC, WK_KQUANT, WK_IQ, WK_TERNARY, WK_BINARY, WK_AFFINE };

struct WvFmtInfo {
  int kind;
  int bits_lo, bits_hi;
  int pgroup;      // weights per parameter group (0: run-time, from BlockWeights)
  int has_min;     // asymmetric: w = min + code*scale
  int mid;         // integer subtracted from the stored code
  int half_mid;    // IQ linear grids: a further 0.5 is subtracted
  int sign;        // 1-bit formats: w = scale*(2*code-1)
  int table;       // IQ4_NL: w = scale*grid[code]
  int wire_block;  // bytes of one wire block / super-block in Raw (0: plain stream)
  int wire_bw;     // weights per wire block
};

__host__ __device__ constexpr WvFmtInfo wv_fmt_info(int f) {
  switch (f) {
  //                 kind        lo hi  pg min mid half sign tbl  wb   wbw
  case WV_Q8_0:    return {WK_CLASSIC, 8, 0, 32, 0, 128, 0, 0, 0, 36, 32};
  case WV_Q4_0:    return {WK_CLASSIC, 4, 0, 32, 0, 8, 0, 0, 0, 20, 32};
  case WV_Q4_1:    return {WK_CLASSIC, 4, 0, 32, 1, 0, 0, 0, 0, 24, 32};
  case WV_Q5_0:    return {WK_CLASSIC, 4, 1, 32, 0, 16, 0, 0, 0, 24, 32};
  case WV_Q5_1:    return {WK_CLASSIC, 4, 1, 32, 1, 0, 0, 0, 0, 28, 32};
  case WV_Q2_K:    return {WK_KQUANT, 2, 0, 16, 1, 0, 0, 0, 0, 104, 256};
  case WV_Q3_K:    return {WK_KQUANT, 2, 1, 16, 1, 0, 0, 0, 0, 136, 256};
  case WV_Q4_K:    return {WK_KQUANT, 4, 0, 16, 1, 0, 0, 0, 0, 168, 256};
  case WV_Q5_K:    return {WK_KQUANT, 4, 1, 16, 1, 0, 0, 0, 0, 200, 256};
  case WV_Q6_K:    return {WK_KQUANT, 4, 2, 16, 0, 32, 0, 0, 0, 216, 256};
  case WV_IQ1_S:   return {WK_IQ, 1, 0, 32, 0, 0, 0, 1, 0, 0, 32};
  case WV_IQ2_XXS: return {WK_IQ, 2, 0, 32, 0, 1, 1, 0, 0, 0, 32};
  case WV_IQ2_XS:  return {WK_IQ, 2, 0, 16, 0, 1, 1, 0, 0, 0, 16};
  case WV_IQ3_XXS: return {WK_IQ, 2, 1, 32, 0, 3, 1, 0, 0, 0, 32};
  case WV_IQ3_S:   return {WK_IQ, 2, 1, 16, 0, 3, 1, 0, 0, 0, 16};
  case WV_IQ4_NL:  return {WK_IQ, 4, 0, 32, 0, 0, 0, 0, 1, 0, 32};
  case WV_IQ4_XS:  return {WK_IQ, 4, 0, 16, 0, 7, 1, 0, 0, 0, 16};
  case WV_TERNARY: return {WK_TERNARY, 2, 0, 16, 0, 1, 0, 0, 0, 0, 16};
  case WV_BINARY:  return {WK_BINARY, 1, 0, 0, 0, 0, 0, 1, 0, 0, 32};
  case WV_AFFINE:  return {WK_AFFINE, 4, 0, 0, 1, 0, 0, 0, 0, 0, 8};
  default:         return {WK_NONE, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1};
  }
}

// IQ4_NL grid (reference quant/iq.go:23-40)
#define WV_IQ4NL_GRID { -1.0f, -0.6961928f, -0.52507305f, -0.3949175f, -0.28444138f, -0.18477343f, \
  -0.091050036f, 0.0f, 0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f, 0.562617f, \
  0.72295684f, 1.0f }

// Device-resident blob (one cache entry, or one row shard of it).
struct WvDevBlob {
  int format, dtype, rows, cols;
  int group;            // BlockWeights as given / inferred (binary 32|128, affine group)
  int fast;             // 1 when the chunked kernels apply (row starts are chunk aligned)
  long long n;          // rows*cols
  long long nchunks;    // padded 32-weight chunks
  const uint32_t* lo;   // lo plane (or raw elements for FormatNone)
  const uint32_t* hi;   // hi plane or null
  const float* p0;      // scales   (k-quants: float2 {d,dmin} per super-block)
  const float* p1;      // mins
  const uint32_t* km;   // k-quants: per-chunk scale/min bytes
};

// ---- chunk-internal addressing -------------------------------------------------------
template <int B> struct WvLane {
  static constexpr int CPW = 32 / B;   // codes per lo word
  static constexpr int SPW = 8 / B;    // shifts per lo word
  static constexpr unsigned MASK = 0x01010101u * ((1u << B) - 1u);
  // j (0..31) -> k (0..7) and m (0..3)
  __host__ __device__ static constexpr int k_of(int j) { return (j / CPW) * SPW + (j % CPW) % SPW; }
  __host__ __device__ static constexpr int m_of(int j) { return (j % CPW) / SPW; }
  __host__ __device__ static constexpr int j_of(int k, int m) { return (k / SPW) * CPW + m * SPW + (k % SPW); }
};
__host__ __device__ inline int wv_k_of(int B, int j) { int cpw = 32 / B, spw = 8 / B; return (j / cpw) * spw + (j % cpw) % spw; }
__host__ __device__ inline int wv_m_of(int B, int j) { int cpw = 32 / B, spw = 8 / B; return (j % cpw) / spw; }

// hi plane: H bits of code (k, m) live in word (k*H)/8 of the chunk at bit 8*m + (k*H)%8.
__host__ __device__ inline int wv_hi_word(int H, int k) { return (k * H) >> 3; }
__host__ __device__ inline int wv_hi_bit(int H, int k, int m) { return 8 * m + ((k * H) & 7); }

// Code of flat weight index i from the device planes (slow path: unpack, ragged GEMV).
__device__ __forceinline__ unsigned wv_dev_code(const WvDevBlob& b, int BL, int BH, long long i) {
  long long bit = i * BL;
  unsigned c = (b.lo[bit >> 5] >> (bit & 31)) & ((1u << BL) - 1u);
  if (BH) {
    long long ch = i >> 5; int j = (int)(i & 31);
    int k = wv_k_of(BL, j), m = wv_m_of(BL, j);
    unsigned hw = b.hi[ch * BH + wv_hi_word(BH, k)];
    c |= ((hw >> wv_hi_bit(BH, k, m)) & ((1u << BH) - 1u)) << BL;
  }
  return c;
}

// Thread-local last-error text (wv_api.cu).
void wv_set_error(const char* fmt, ...);

// Launchers implemented across the .cu files.
int wv_launch_relayout(const WvDevBlob& dst, const uint8_t* d_raw, size_t nraw, cudaStream_t st);
int wv_launch_unpack(const WvDevBlob& b, float* d_out, cudaStream_t st);
int wv_launch_unpack_rows(const WvDevBlob& b, int row, int nrows, float* d_out, cudaStream_t st);
int wv_launch_gemv(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end,
                   cudaStream_t st);
int wv_launch_pack(int format, int dtype, int group, const float* d_w, int rows, int cols, uint8_t* d_raw,
                   float* d_scales, float* d_mins, cudaStream_t st);
