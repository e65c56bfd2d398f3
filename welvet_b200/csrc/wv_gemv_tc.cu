// Batch-1 GEMV for every packed integer-code format with the dot products on the tensor pipe.
//
// Why: the integer pipe of an SM issues dp4a / logic / shift instructions at half rate, and a dp4a
// GEMV needs about 0.9 of them per weight (extraction + two dp4a per four codes), which bounds it at
// ~8 us for a 58.7 M-weight matrix whatever its byte count. Here mma.sync m16n8k32 (u8 x s8 -> s32)
// does the multiply-adds of 16 rows x 32 columns at once and the integer pipe is left with the code
// extraction alone.
//
//   * A operand = 16 rows x one 32-column chunk of unsigned codes, unpacked from the bit planes by
//     the lane that holds the fragment (one 32-bit word of the lo plane per row per lane);
//   * B operand = the chunk's activations as 16-bit block fixed point X = rint(x * 32512 / amax),
//     split into two signed byte digits X = d0 + 256 d1; a chunk takes two operand columns
//     (formats with one parameter group per chunk) or four (two groups per chunk: the columns of a
//     group are zero outside its 16 weights), so four / two chunks are chained into one accumulator
//     and every lane of a quad ends with the two digit sums of "its" chunk (or half chunk) for rows
//     g and g + 8;
//   * the integer sums go through the same scale / min arithmetic as the dp4a kernels (idot_finish);
//   * tiles (16-row blocks x 64-chunk column segments, two blocks per stage) are fetched by tensor-map
//     copies (cp.async.bulk.tensor, 128-byte swizzle for the planes with >= 128 bytes per segment row,
//     plain 2-D boxes for the few smaller parameter planes) into a shared-memory ring with bounded waits;
//   * x is quantised once per launch by a small kernel in front (tc_xquant_kernel, chained by programmatic
//     dependent launch: it runs while the GEMV's CTAs are being placed) and every CTA brings the ready record
//     (digits in operand order, scale factors, sums) into shared memory with one bulk copy;
//   * a vector whose chunks mix large and much smaller values (see the criterion in the kernel) gets a
//     second pass over the matrix with the 16-bit residual of the first quantisation: 32 bits in all.
#include "wv_gemv_common.cuh"
#include "wv_tma_common.cuh"
#include "wv_dev_hooks.h"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>

#define TC_WARPS 16
#define TC_THREADS ((TC_WARPS + 1) * 32)
#define TC_MAX_STAGES 8
#define TC_SEG 64            // chunks per column segment
#define TC_RB 2              // 16-row blocks per stage, at most


struct TcGeom {
  int cpr;               // chunks per row
  int nseg;              // column segments per row
  int nrows;             // rows of this launch
  int blk_base, blk_rem; // CTA b owns blk_base (+1 if b < blk_rem) blocks of 16 rows
  int nstage;
  int rb;                // 16-row blocks per stage (1 or 2)
  int gsh;               // log2(chunks per parameter group) for binary / affine
  int force_wide;        // development switch: always run the residual pass
  unsigned blk_bytes;    // shared-memory bytes of one 16-row block of one segment (all planes, regions 1024-aligned)
  unsigned tx_bytes;     // bytes the copy engine delivers for one block (full boxes; what lies outside the tensor is zero-filled)
  unsigned off[5];       // plane offsets inside a block (lo, hi, p0, p1, km)
  unsigned segb[5];      // bytes per segment row of each plane (0 = absent)
  unsigned tiled[5];     // 1: {128 B, rows, pieces} map with 128-byte swizzle; 0: plain 2-D box of segb bytes
  unsigned dig_off, meta_off, red_off, bar_off;
  int prequant;          // 1: the activation record comes from tc_xquant_kernel; 0: the CTA builds it from x
  unsigned rec_stride;   // bytes between the activation records of consecutive batch rows
  unsigned rec_pass;     // bytes from a row's first-pass record to its residual record
};

__device__ __forceinline__ void mma_u8s8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void tc_tma_3d(unsigned dst, const CUtensorMap* tm, int c0, int c1, int c2, unsigned bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(tm)), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_tma_2d(unsigned dst, const CUtensorMap* tm, int c0, int c1, unsigned bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(tm)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
// Byte o of row r of a plane inside a block: swizzled [piece][16 rows][128 B] or plain [16 rows][segb].
__device__ __forceinline__ unsigned tc_addr(unsigned tiled, unsigned segb, unsigned o, unsigned r) {
  if (tiled) return (o >> 7) * 2048u + r * 128u + ((((o >> 4) & 7u) ^ (r & 7u)) << 4) + (o & 15u);
  return r * segb + o;
}

template <int F> struct TcCfg {
  static constexpr WvFmtInfo fi = wv_fmt_info(F);
  static constexpr bool HALVES = QCfg<F>::HALVES;        // two parameter groups per chunk
  static constexpr bool INT_MID = QCfg<F>::INT_MID;
  static constexpr int UNIT = HALVES ? 2 : 4;            // chunks chained into one accumulator
  static constexpr int UPW = (TC_SEG / UNIT) / TC_WARPS; // units per warp per segment
  static constexpr bool OK = !fi.table && fi.kind != WK_NONE;
};

// Group index kk (0..7) of the codes a lane holds for operand half hi (k = 16 hi + 4 t + m <-> code (kk, m)).
template <int BL> __device__ __forceinline__ int tc_kk(int t, int hi) { return BL == 8 ? t + 4 * hi : 2 * t + hi; }

// ------------------------------------------------------------------ activation record
// tc_xquant_kernel turns x into the record the GEMV's CTAs copy into shared memory, once per launch instead of
// once per CTA (148 times): per chunk 64 bytes of operand digits and 32 bytes of scale factors and sums, then a
// 16-byte tail {passes, -, -, -} and the CTAs' partial statistics. Four threads per chunk: thread q takes the
// eight activations of operand positions k = 4q .. 4q+3 and 16+4q .. 16+4q+3 and writes their digits where lane
// t = q of the GEMV reads them. First pass: X = rint(x * 32512 / amax) per chunk. When the statistics of the whole
// vector ask for it (see the criterion below) the last CTA to finish also writes a second record with the
// residual x - X sf against a 65024 times finer step.
#define TCX_THREADS 256
#define TCX_MAX_CTAS 8

template <int BL>
__device__ __forceinline__ void tcx_load(const float* xc, int q, bool al32, float (&xv)[8]) {
  // xv[hi * 4 + m] = activation of operand position k = 16 hi + 4 q + m. The loads are shaped so that a warp
  // instruction touches as few 128-byte lines as possible.
  if (al32 && BL == 4) {
    float e[8];
    asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(e[0]), "=f"(e[1]), "=f"(e[2]), "=f"(e[3]), "=f"(e[4]), "=f"(e[5]), "=f"(e[6]), "=f"(e[7]) : "l"(xc + 8 * q));
#pragma unroll
    for (int m = 0; m < 4; m++) { xv[m] = e[2 * m]; xv[4 + m] = e[2 * m + 1]; }   // position (hi, m) is column 8q + 2m + hi
  } else if (al32 && BL == 8) {
    const float4 e0 = __ldg(reinterpret_cast<const float4*>(xc) + q), e1 = __ldg(reinterpret_cast<const float4*>(xc) + 4 + q);
    xv[0] = e0.x; xv[1] = e0.y; xv[2] = e0.z; xv[3] = e0.w; xv[4] = e1.x; xv[5] = e1.y; xv[6] = e1.z; xv[7] = e1.w;
  } else {
#pragma unroll
    for (int m = 0; m < 4; m++) {
      xv[m] = __ldg(xc + WvLane<BL>::j_of(tc_kk<BL>(q, 0), m));
      xv[4 + m] = __ldg(xc + WvLane<BL>::j_of(tc_kk<BL>(q, 1), m));
    }
  }
}

// One task (four threads of a quad work on one chunk; all 32 lanes of the warp must call this together).
// Returns the chunk's {amax, sum |x|} in thread q == 0 (NaN sum for a chunk with inf / NaN), zero elsewhere.
__device__ __forceinline__ float2 tcx_task(int pass, bool on, int c, int q, const float (&xv)[8], unsigned char* rec, int cpr, int mid, int halves) {
  float amax = 0.f, asum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) { amax = fmaxf(amax, fabsf(xv[i])); asum += fabsf(xv[i]); }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1)); asum += __shfl_xor_sync(0xffffffffu, asum, 1);
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2)); asum += __shfl_xor_sync(0xffffffffu, asum, 2);
  const bool bad = !(asum <= 3.0e38f);   // inf or NaN in the chunk
  float sf = 0.f, inv = 0.f;
  if (bad) sf = __uint_as_float(0x7fc00000u);
  else if (amax >= 1.0e-30f) { sf = amax * (1.0f / 32512.0f); inv = 32512.0f / amax; }   // |x inv| <= 32512 (1 + 2^-23)
  // The low 16 bits of the float 1.5 * 2^23 + rint(v) are rint(v) in two's complement. Digits: d0 = low byte as it
  // is (read as signed), d1 = (X + 128) >> 8, i.e. byte 1 after adding 128.
  unsigned B[8];
#pragma unroll
  for (int i = 0; i < 8; i++) B[i] = __float_as_uint(fmaf(xv[i], inv, 12582912.0f));
  if (pass == 1) {
    // residual of the first quantisation against a 65024 times finer step: |r| <= sf / 2 -> |X2| <= 32512
    const float inv2 = 65024.0f * inv;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float r = fmaf(-(float)((int)B[i] - 0x4B400000), sf, xv[i]);
      B[i] = __float_as_uint(fmaf(r, inv2, 12582912.0f));
    }
    sf *= (1.0f / 65024.0f);
  }
  unsigned w0[2], w1[2];
  int sx = 0;
#pragma unroll
  for (int hi = 0; hi < 2; hi++) {
    const unsigned* e = B + hi * 4;
    sx += (int)(e[0] + e[1] + e[2] + e[3]);
    w0[hi] = __byte_perm(__byte_perm(e[0], e[1], 0x0040), __byte_perm(e[2], e[3], 0x0040), 0x5410);
    w1[hi] = __byte_perm(__byte_perm(e[0] + 128u, e[1] + 128u, 0x0051), __byte_perm(e[2] + 128u, e[3] + 128u, 0x0051), 0x5410);
  }
  sx = (int)((unsigned)sx - 8u * 0x4B400000u);   // wraps back to the sum of the eight integers
  // sums of X over the chunk and over its halves (threads 0,1 hold the first 16 weights of 2- and 4-bit planes)
  const int s01 = sx + __shfl_xor_sync(0xffffffffu, sx, 1);
  const int sall = s01 + __shfl_xor_sync(0xffffffffu, s01, 2);
  if (on) {
    unsigned char* d = rec + (size_t)c * 64;
    *reinterpret_cast<uint2*>(d + q * 8) = make_uint2(w0[0], w0[1]);
    *reinterpret_cast<uint2*>(d + 32 + q * 8) = make_uint2(w1[0], w1[1]);
    if (q == 0) {        // s01 is the first half's sum here, sall - s01 the second half's
      const int s23 = sall - s01;
      float4* meta = reinterpret_cast<float4*>(rec + (size_t)cpr * 64) + (size_t)c * 2;
      meta[0] = make_float4(sf, sf * (float)sall, sf * (float)s01, sf * (float)s23);
      *reinterpret_cast<int4*>(meta + 1) = make_int4(halves ? -mid * s01 : -mid * sall, -mid * s23, 0, 0);
    }
  }
  float2 st = make_float2(0.f, 0.f);
  if (on && q == 0) st = bad ? make_float2(0.f, __uint_as_float(0x7fc00000u)) : make_float2(amax, asum);
  return st;
}

template <int BL>
__global__ void __launch_bounds__(TCX_THREADS) tc_xquant_kernel(const float* __restrict__ x, int cols, int mid, int halves, unsigned char* __restrict__ recs,
                                                                unsigned rec_stride, unsigned rec_pass, unsigned* __restrict__ counters, int force_wide) {
  __shared__ float s_part[TCX_THREADS / 32][2];
  __shared__ int s_last;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMV behind may be placed right away
  asm volatile("griddepcontrol.wait;" ::: "memory");                // x may be the previous kernel's output
  const int cpr = cols >> 5, ntask = cpr * 4;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* xrow = x + (size_t)blockIdx.y * cols;
  unsigned char* rec = recs + (size_t)blockIdx.y * rec_stride;
  const bool al32 = (reinterpret_cast<uintptr_t>(xrow) & 31) == 0;
  float st_a = 0.f, st_s = 0.f;
  for (int base = blockIdx.x * TCX_THREADS; base < ntask; base += gridDim.x * TCX_THREADS) {   // warp-uniform trip count
    const int task = base + tid;
    const bool on = task < ntask;
    const int c = on ? task >> 2 : 0, q = task & 3;
    float xv[8];
    tcx_load<BL>(xrow + (size_t)c * 32, q, al32, xv);
    if (!on) {
#pragma unroll
      for (int i = 0; i < 8; i++) xv[i] = 0.f;
    }
    const float2 st = tcx_task(0, on, c, q, xv, rec, cpr, mid, halves);
    st_a += st.x; st_s += st.y;
  }
  // Pass decision, from the whole vector: A = sum over chunks of the chunk's largest magnitude, S = sum |x_j|.
  // With 16-bit records an element is off by at most amax_chunk / 65024, so a row's error is at most
  // sum_chunks amax_c / 65024 * sum_{j in c} |w_j|, about w_mean * 4.9e-4 * A for weights that are not concentrated
  // on a chunk's small elements, against a budget of 1e-3 * w_mean * S. A <= S / 4 keeps an eightfold margin
  // (N(0,1) data: A / S = 0.09); vectors with isolated outliers, inf or NaN fail the test and get the residual
  // pass. Weights that sit exactly on the small elements of outlier chunks can exceed either bound: no criterion
  // on x alone excludes that.
#pragma unroll
  for (int o = 16; o; o >>= 1) { st_a += __shfl_xor_sync(0xffffffffu, st_a, o); st_s += __shfl_xor_sync(0xffffffffu, st_s, o); }
  if (lane == 0) { s_part[warp][0] = st_a; s_part[warp][1] = st_s; }
  __syncthreads();
  int* tail = reinterpret_cast<int*>(rec + (size_t)cpr * 96);
  float* parts = reinterpret_cast<float*>(tail + 4);
  if (tid == 0) {
    float a = 0.f, sm = 0.f;
    for (int w = 0; w < TCX_THREADS / 32; w++) { a += s_part[w][0]; sm += s_part[w][1]; }
    parts[2 * blockIdx.x] = a; parts[2 * blockIdx.x + 1] = sm;
    __threadfence();
    const unsigned prev = atomicAdd(&counters[blockIdx.y], 1u);
    s_last = prev == gridDim.x - 1;
    if (s_last) counters[blockIdx.y] = 0u;   // ready for the next launch that gets this counter
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float ta = 0.f, ts = 0.f;
  for (int i = 0; i < (int)gridDim.x; i++) { ta += __ldcg(parts + 2 * i); ts += __ldcg(parts + 2 * i + 1); }   // fixed order
  const int npass = (!(ta <= 0.25f * ts) || force_wide) ? 2 : 1;
  if (tid == 0) { tail[0] = npass; tail[1] = 0; tail[2] = 0; tail[3] = 0; }
  if (npass == 1) return;
  // rare: the residual record, by this one CTA
  unsigned char* rec2 = rec + rec_pass;
  for (int base = 0; base < ntask; base += TCX_THREADS) {
    const int task = base + tid;
    const bool on = task < ntask;
    const int c = on ? task >> 2 : 0, q = task & 3;
    float xv[8];
    tcx_load<BL>(xrow + (size_t)c * 32, q, al32, xv);
    if (!on) {
#pragma unroll
      for (int i = 0; i < 8; i++) xv[i] = 0.f;
    }
    tcx_task(1, on, c, q, xv, rec2, cpr, mid, halves);
  }
  if (tid == 0) { int* tail2 = reinterpret_cast<int*>(rec2 + (size_t)cpr * 96); tail2[0] = 2; tail2[1] = 0; tail2[2] = 0; tail2[3] = 0; }
}

// The two A registers (operand halves k < 16 and k >= 16) of one row of one chunk. lo_a / hi_a: offsets from the
// aligned base of the word(s) this lane reads (tc_lane_lo / tc_lane_hi plus stage, block and row offsets).
template <int F>
__device__ __forceinline__ void tc_load_a(const unsigned char* smem, unsigned lo_a, unsigned hi_a, int t, unsigned& q0, unsigned& q1) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi;
  auto ld32 = [&](unsigned o) { return *reinterpret_cast<const unsigned*>(smem + o); };
  if constexpr (BL == 8) {
    // words t and t + 4: the second sits in the neighbouring 16-byte unit (address bit 4 flipped under the swizzle)
    q0 = ld32(lo_a); q1 = ld32(lo_a ^ 16u);
  } else if constexpr (BL == 4) {
    const unsigned w = ld32(lo_a);
    q0 = w & 0x0F0F0F0Fu; q1 = (w >> 4) & 0x0F0F0F0Fu;
  } else if constexpr (BL == 2) {
    const unsigned w = ld32(lo_a) >> (4 * (t & 1));
    q0 = w & 0x03030303u; q1 = (w >> 2) & 0x03030303u;
  } else {
    const unsigned w = ld32(lo_a) >> (2 * t);
    q0 = w & 0x01010101u; q1 = (w >> 1) & 0x01010101u;
  }
  if constexpr (BH == 1) {
    constexpr unsigned MH = 0x01010101u << BL;
    const unsigned h = ld32(hi_a) >> (2 * t);
    q0 |= (h << BL) & MH; q1 |= ((h >> 1) << BL) & MH;
  } else if constexpr (BH == 2) {
    constexpr unsigned MH = 0x03030303u << BL;
    const unsigned h = ld32(hi_a) >> (4 * (t & 1));
    q0 |= (h << BL) & MH; q1 |= ((h >> 2) << BL) & MH;
  }
}
// Four 8 x 16-byte matrices in one instruction: lane l supplies the address of row l & 7 of matrix l >> 3 and receives
// from each matrix the four bytes 4t .. 4t+3 of row gq (lane = 4 gq + t).
__device__ __forceinline__ void tc_ldsm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// Codes of a 4-bit lo word (already loaded) merged with the hi plane's bits: the two A registers of one row of one chunk.
template <int F>
__device__ __forceinline__ void tc_codes4(const unsigned char* smem, unsigned w, unsigned hi_a, int t, unsigned& q0, unsigned& q1) {
  constexpr int BH = wv_fmt_info(F).bits_hi;
  q0 = w & 0x0F0F0F0Fu; q1 = (w >> 4) & 0x0F0F0F0Fu;
  if constexpr (BH == 1) {
    const unsigned h = *reinterpret_cast<const unsigned*>(smem + hi_a) >> (2 * t);
    q0 |= (h << 4) & 0x10101010u; q1 |= ((h >> 1) << 4) & 0x10101010u;
  } else if constexpr (BH == 2) {
    const unsigned h = *reinterpret_cast<const unsigned*>(smem + hi_a) >> (4 * (t & 1));
    q0 |= (h << 4) & 0x30303030u; q1 |= ((h >> 2) << 4) & 0x30303030u;
  }
}
// Offset inside a block of the lo / hi word lane (gq, t) reads for row gq of chunk cs of the segment (row gq + 8: + 1024).
template <int F> __device__ __forceinline__ unsigned tc_lane_lo(const TcGeom& g, unsigned cs, unsigned gq, unsigned t) {
  constexpr int BL = wv_fmt_info(F).bits_lo;
  const unsigned w = BL >= 4 ? 4u * t : (BL == 2 ? 4u * (t >> 1) : 0u);
  return g.off[0] + tc_addr(1u, 0u, cs * (BL * 4u), gq) + w;
}
template <int F> __device__ __forceinline__ unsigned tc_lane_hi(const TcGeom& g, unsigned cs, unsigned gq, unsigned t) {
  constexpr int BH = wv_fmt_info(F).bits_hi;
  return g.off[1] + tc_addr(1u, 0u, cs * (BH * 4u), gq) + (BH == 2 ? 4u * (t >> 1) : 0u);
}

// Offsets inside a block of the parameter words of (row r, chunk cs of the segment), and the loads from them.
struct TcParamOff { unsigned a, b; };
template <int F>
__device__ __forceinline__ TcParamOff tc_param_off(const TcGeom& g, unsigned r, unsigned cs) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  auto at = [&](int p, unsigned o) { return g.off[p] + tc_addr(g.tiled[p], g.segb[p], o, r); };
  TcParamOff o{0u, 0u};
  if constexpr (fi.kind == WK_KQUANT) { o.a = at(2, (cs >> 3) * 8u); o.b = at(4, cs * (fi.has_min ? 4u : 2u)); }
  else if constexpr (fi.kind == WK_CLASSIC) { o.a = at(2, cs * 4u); if constexpr (fi.has_min) o.b = at(3, cs * 4u); }
  else if constexpr (fi.kind == WK_BINARY) { o.a = at(2, (cs >> g.gsh) * 4u); }
  else if constexpr (fi.kind == WK_AFFINE) { o.a = at(2, (cs >> g.gsh) * 4u); o.b = at(3, (cs >> g.gsh) * 4u); }
  else if constexpr (fi.pgroup == 16) { o.a = at(2, cs * 8u); }
  else { o.a = at(2, cs * 4u); }
  return o;
}
template <int F>
__device__ __forceinline__ void tc_load_params(FragT<F>& f, const unsigned char* smem, unsigned blk, const TcParamOff o) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  auto ld32 = [&](unsigned a) { return *reinterpret_cast<const unsigned*>(smem + a); };
  auto ld64 = [&](unsigned a) { return *reinterpret_cast<const uint2*>(smem + a); };
  auto ld16 = [&](unsigned a) { return (unsigned)*reinterpret_cast<const unsigned short*>(smem + a); };
  if constexpr (fi.kind == WK_KQUANT) {
    const uint2 dd = ld64(blk + o.a);
    f.pr[0] = dd.x; f.pr[1] = dd.y;
    if constexpr (fi.has_min) f.pr[2] = ld32(blk + o.b); else f.pr[2] = ld16(blk + o.b);
  } else if constexpr (fi.kind == WK_CLASSIC || fi.kind == WK_AFFINE) {
    f.pr[0] = ld32(blk + o.a);
    if constexpr (fi.has_min) f.pr[1] = ld32(blk + o.b);
  } else if constexpr (fi.pgroup == 16) {
    const uint2 v = ld64(blk + o.a);
    f.pr[0] = v.x; f.pr[1] = v.y;
  } else {
    f.pr[0] = ld32(blk + o.a);
  }
}

template <int F>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemv_tc_kernel(const WvDevBlob b, const unsigned char* __restrict__ xrec, float* __restrict__ y, int row_begin, const TcGeom g, int* __restrict__ err,
               const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, const __grid_constant__ CUtensorMap tm2,
               const __grid_constant__ CUtensorMap tm3, const __grid_constant__ CUtensorMap tm4) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi;
  constexpr bool HALVES = TcCfg<F>::HALVES, INT_MID = TcCfg<F>::INT_MID;
  constexpr int UNIT = TcCfg<F>::UNIT, UPW = TcCfg<F>::UPW;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ int s_npass;        // 0 until the consumers have decided: 1 or 2 passes over the matrix
  __shared__ float s_stat[TC_WARPS][2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bid = blockIdx.x;
  const int nblk = g.blk_base + (bid < g.blk_rem ? 1 : 0);
  const int blk0 = bid * g.blk_base + min(bid, g.blk_rem);
  const int ngrp = (nblk + g.rb - 1) / g.rb;
  // swizzled tiles want a 1024-byte aligned base
  const unsigned sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (sbase - smem_u32(smem_raw));
  const unsigned bar0 = sbase + g.bar_off;
  const unsigned stage_bytes = g.blk_bytes * (unsigned)g.rb;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (TC_MAX_STAGES + s); };

  if (tid == 0) {
    s_abort = 0;
    s_npass = 0;
    for (int s = 0; s < g.nstage; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), TC_WARPS); }
    mbar_init(bar0 + 8u * (2 * TC_MAX_STAGES), 1);   // arrival of the activation record
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == TC_WARPS) {
    // ------------------------------------------------------------ producer warp: lane 0 issues the copies
    if (lane != 0) return;
    const CUtensorMap* tm[5] = {&tm0, &tm1, &tm2, &tm3, &tm4};
    int ps = 0, issued = 0;
    unsigned ppar = 1;
    bool wrapped = false, dead = false;
    int npass = 1;
    for (int pass = 0; pass < npass && !dead; pass++) {
      for (int gi = 0; gi < ngrp && !dead; gi++) {
        const int nb = min(g.rb, nblk - gi * g.rb);
        for (int seg = 0; seg < g.nseg && !dead; seg++) {
          if (wrapped) {
            if (*(volatile int*)&s_abort || !mbar_wait(empty_bar(ps), ppar)) {
              if (!*(volatile int*)&s_abort) { atomicCAS_system(err, 0, 800 + ps); *(volatile int*)&s_abort = 1; }
              dead = true;
              break;
            }
          }
          mbar_expect_tx(full_bar(ps), g.tx_bytes * nb);
          for (int rb = 0; rb < nb; rb++) {
            const unsigned dst = sbase + (unsigned)ps * stage_bytes + (unsigned)rb * g.blk_bytes;
            const int row0 = row_begin + (blk0 + gi * g.rb + rb) * 16;
#pragma unroll
            for (int p = 0; p < 5; p++) {
              if (!g.segb[p]) continue;
              if (g.tiled[p]) tc_tma_3d(dst + g.off[p], tm[p], 0, row0, seg * (int)(g.segb[p] >> 7), full_bar(ps));
              else tc_tma_2d(dst + g.off[p], tm[p], seg * (int)g.segb[p], row0, full_bar(ps));
            }
          }
          issued++;
          if (++ps == g.nstage) { ps = 0; wrapped = true; ppar ^= 1u; }
        }
      }
      if (pass == 0 && !dead) {
        // the consumers decide in their prologue whether a residual pass follows
        int np = 0;
        for (unsigned i = 0; i < TMA_SPIN_LIMIT && !np; i++) np = *(volatile int*)&s_npass;
        if (!np) { atomicCAS_system(err, 0, 850); *(volatile int*)&s_abort = 1; dead = true; }
        npass = np;
      }
    }
    // drain: every copy issued must have landed before the CTA gives its shared memory back
    for (int t = max(0, issued - g.nstage); t < issued; t++) {
      if (!mbar_wait(full_bar(t % g.nstage), (unsigned)(t / g.nstage) & 1u)) { atomicCAS_system(err, 0, 900 + t % g.nstage); break; }
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int gq = lane >> 2, t = lane & 3;
  unsigned char* dig = smem + g.dig_off;                       // [chunk][2 digits][32 bytes in operand order]
  float4* meta = reinterpret_cast<float4*>(smem + g.meta_off);  // [chunk] {sf, sf SX, sf SX(first 16), sf SX(second 16)} {msx0, msx1, -, -}
  float* red = reinterpret_cast<float*>(smem + g.red_off);      // [2][TC_WARPS][TC_RB * 16]
  float* yb = y + (size_t)blockIdx.y * b.rows + row_begin;

  // ---- lane constants of the main loop (nothing here depends on x: it overlaps the previous kernel's tail)
  // A operand: the words this lane reads for row gq of the chunks of its units (row gq + 8 is 1024 bytes further)
  unsigned a_lo[UPW][UNIT], a_hi[UPW][UNIT];
  // 4- and 8-bit planes fetch their lo words with ldmatrix: the row address this lane supplies (4-bit: one instruction
  // covers rows 0-7 / 8-15 of two neighbouring chunks; 8-bit: rows 0-7 / 8-15 of the two 16-byte halves of one chunk)
  constexpr bool LDSM = BL == 4 || BL == 8;
  constexpr int NLM = BL == 4 ? UNIT / 2 : UNIT;
  unsigned a_lm[UPW][LDSM ? NLM : 1];
  // epilogue: parameter words of this lane's (row, chunk)
  TcParamOff p_off[UPW][HALVES ? 1 : 2];
  // B operand: lane (gq, t) supplies column n = gq. One group per chunk: column (chunk n >> 1, digit n & 1).
  // Two groups per chunk: column (chunk n >> 2, half (n >> 1) & 1, digit n & 1), zero outside the half's 16
  // weights, which are the operand positions of lanes t >> 1 == half.
  const int b_chunk = HALVES ? (gq >> 2) : (gq >> 1);
  const bool b_on = HALVES ? ((t >> 1) == ((gq >> 1) & 1)) : true;
  const unsigned b_off = (unsigned)(gq & 1) * 32u + (unsigned)t * 8u;
  const int e_chunk = HALVES ? (t >> 1) : t;                    // chunk of the unit this lane finishes
#pragma unroll
  for (int u = 0; u < UPW; u++) {
    const unsigned cs0 = (unsigned)(warp * UPW + u) * UNIT;
#pragma unroll
    for (int i = 0; i < UNIT; i++) {
      a_lo[u][i] = tc_lane_lo<F>(g, cs0 + i, (unsigned)gq, (unsigned)t);
      a_hi[u][i] = BH ? tc_lane_hi<F>(g, cs0 + i, (unsigned)gq, (unsigned)t) : 0u;
    }
    if constexpr (LDSM) {
      const unsigned lrow = (unsigned)(lane & 7) + 8u * (unsigned)((lane >> 3) & 1), lsel = (unsigned)(lane >> 4);
#pragma unroll
      for (int i = 0; i < NLM; i++) {
        if constexpr (BL == 4) a_lm[u][i] = g.off[0] + tc_addr(1u, 0u, (cs0 + 2 * i + lsel) * 16u, lrow);
        else a_lm[u][i] = g.off[0] + tc_addr(1u, 0u, (cs0 + i) * 32u + 16u * lsel, lrow);
      }
    }
    if constexpr (HALVES) p_off[u][0] = tc_param_off<F>(g, (unsigned)gq + ((t & 1) ? 8u : 0u), cs0 + e_chunk);
    else { p_off[u][0] = tc_param_off<F>(g, (unsigned)gq, cs0 + e_chunk); p_off[u][1] = tc_param_off<F>(g, (unsigned)gq + 8u, cs0 + e_chunk); }
  }

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // The activation record (digits in operand order, per-chunk scale factors and sums, pass count): either prepared
  // once for the whole grid by tc_xquant_kernel and brought in with one bulk copy (g.prequant), or built here by
  // the consumer threads straight from x (four rounds of tasks at a time, so that all their loads are in flight
  // before the first one is used).
  const unsigned rec_bytes = (unsigned)g.cpr * 96u + 16u;
  const unsigned xbar = bar0 + 8u * (2 * TC_MAX_STAGES);
  const unsigned char* rec0 = xrec + (size_t)blockIdx.y * g.rec_stride;
  const float* xrow = reinterpret_cast<const float*>(xrec) + (size_t)blockIdx.y * b.cols;   // in-kernel mode: xrec is x itself
  const int ntask = g.cpr * 4;
  const bool x_al32 = (reinterpret_cast<uintptr_t>(xrow) & 31) == 0;
  float st_a = 0.f, st_s = 0.f;
  auto quantise = [&](int pass) {
    constexpr int NT = TC_WARPS * 32;
    const int rot = (int)(((unsigned)bid * 97u) % (unsigned)g.cpr) * 4;   // CTAs start at different chunks: spreads the L2 requests
    for (int base = 0; base < ntask; base += 4 * NT) {
      float xv[4][8];
      int tk[4];
#pragma unroll
      for (int r = 0; r < 4; r++) {
        int task = base + r * NT + tid;
        const bool on = task < ntask;
        task += rot; if (task >= ntask) task -= ntask;
        tk[r] = on ? task : -1;
        tcx_load<BL>(xrow + (size_t)(on ? task >> 2 : 0) * 32, task & 3, x_al32, xv[r]);
      }
#pragma unroll
      for (int r = 0; r < 4; r++) {
        if (base + r * NT < ntask) {   // warp-uniform: the quads shuffle
          const bool on = tk[r] >= 0;
          if (!on) {
#pragma unroll
            for (int i = 0; i < 8; i++) xv[r][i] = 0.f;
          }
          const float2 stt = tcx_task(pass, on, on ? tk[r] >> 2 : 0, tid & 3, xv[r], smem + g.dig_off, g.cpr, INT_MID ? fi.mid : 0, HALVES ? 1 : 0);
          if (pass == 0) { st_a += stt.x; st_s += stt.y; }
        }
      }
    }
  };
  int npass;
  if (g.prequant) {
    if (tid == 0) {
      mbar_expect_tx(xbar, rec_bytes);
      bulk_g2s(sbase + g.dig_off, rec0, rec_bytes, xbar);
    }
    if (!mbar_wait(xbar, 0u)) { atomicCAS_system(err, 0, 1100); *(volatile int*)&s_abort = 1; }
    const int* rec_tail = reinterpret_cast<const int*>(smem + g.dig_off + (size_t)g.cpr * 96);
    npass = (rec_tail[0] == 2 || g.force_wide) ? 2 : 1;
  } else {
    quantise(0);
#pragma unroll
    for (int o = 16; o; o >>= 1) { st_a += __shfl_xor_sync(0xffffffffu, st_a, o); st_s += __shfl_xor_sync(0xffffffffu, st_s, o); }
    if (lane == 0) { s_stat[warp][0] = st_a; s_stat[warp][1] = st_s; }
    asm volatile("bar.sync 15, %0;" ::"n"(TC_WARPS * 32) : "memory");   // also: every chunk's digits are in place
    float ta = 0.f, ts = 0.f;
    for (int w = 0; w < TC_WARPS; w++) { ta += s_stat[w][0]; ts += s_stat[w][1]; }
    npass = (!(ta <= 0.25f * ts) || g.force_wide) ? 2 : 1;   // criterion: see tc_xquant_kernel; every thread computes the same value
  }
  if (tid == 0) *(volatile int*)&s_npass = npass;   // for the producer

  int fs = 0, par = 0;
  unsigned fpar = 0;
  bool dead = false;
  for (int pass = 0; pass < npass; pass++) {
    if (pass == 1) {
      asm volatile("bar.sync 15, %0;" ::"n"(TC_WARPS * 32) : "memory");   // every warp is done reading the first digits
      if (g.prequant) {
        if (tid == 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the generic reads above before the bulk write
          mbar_expect_tx(xbar, rec_bytes);
          bulk_g2s(sbase + g.dig_off, rec0 + g.rec_pass, rec_bytes, xbar);   // digits of the residual
        }
        if (!mbar_wait(xbar, 1u)) { atomicCAS_system(err, 0, 1101); *(volatile int*)&s_abort = 1; }
      } else {
        quantise(1);
        asm volatile("bar.sync 15, %0;" ::"n"(TC_WARPS * 32) : "memory");
      }
    }
    for (int gi = 0; gi < ngrp; gi++) {
      const int nb = min(g.rb, nblk - gi * g.rb);
      float acc[TC_RB][2];
#pragma unroll
      for (int rb = 0; rb < TC_RB; rb++) { acc[rb][0] = 0.f; acc[rb][1] = 0.f; }
      for (int seg = 0; seg < g.nseg; seg++) {
        if (!dead) {
          if (*(volatile int*)&s_abort) dead = true;
          else if (!mbar_wait(full_bar(fs), fpar)) { atomicCAS_system(err, 0, 1000 + fs); *(volatile int*)&s_abort = 1; dead = true; }
        }
        const unsigned st = (unsigned)fs * stage_bytes;   // offset of the stage from the aligned base
#pragma unroll
        for (int u = 0; u < UPW; u++) {
          const int cu = seg * TC_SEG + (warp * UPW + u) * UNIT;   // first chunk of the unit inside the row
          // B words of this lane for the unit, already placed: its own chunk's digits in "its" instruction, zero elsewhere
          // (and zero when the chunk lies past the end of the row)
          uint2 bw = make_uint2(0u, 0u);
          if (b_on && cu + b_chunk < g.cpr) bw = *reinterpret_cast<const uint2*>(dig + (size_t)(cu + b_chunk) * 64 + b_off);
          unsigned bx[UNIT], by[UNIT];
#pragma unroll
          for (int i = 0; i < UNIT; i++) { bx[i] = b_chunk == i ? bw.x : 0u; by[i] = b_chunk == i ? bw.y : 0u; }
          // this lane's chunk for the epilogue: past the end of the row its record reads as zero
          const int ce = cu + e_chunk;
          float4 mt = make_float4(0.f, 0.f, 0.f, 0.f);
          int msx0 = 0, msx1 = 0;
          if (ce < g.cpr) {
            mt = meta[(size_t)ce * 2];
            if constexpr (INT_MID) { const int2 mm = *reinterpret_cast<const int2*>(meta + (size_t)ce * 2 + 1); msx0 = mm.x; msx1 = mm.y; }
          }
#pragma unroll
          for (int rb = 0; rb < TC_RB; rb++) {
            if (rb < nb) {
              const unsigned blk = st + (unsigned)rb * g.blk_bytes;
              int c[4] = {0, 0, 0, 0};
              if constexpr (BL == 4) {
#pragma unroll
                for (int i = 0; i < UNIT; i += 2) {
                  unsigned w0, w1, w2, w3, a0, a1, a2, a3;
                  tc_ldsm4(sbase + blk + a_lm[u][i / 2], w0, w1, w2, w3);   // rows gq, gq + 8 of chunk i; rows gq, gq + 8 of chunk i + 1
                  tc_codes4<F>(smem, w0, blk + a_hi[u][i], t, a0, a2);
                  tc_codes4<F>(smem, w1, blk + a_hi[u][i] + 1024u, t, a1, a3);
                  mma_u8s8(c, a0, a1, a2, a3, bx[i], by[i]);
                  tc_codes4<F>(smem, w2, blk + a_hi[u][i + 1], t, a0, a2);
                  tc_codes4<F>(smem, w3, blk + a_hi[u][i + 1] + 1024u, t, a1, a3);
                  mma_u8s8(c, a0, a1, a2, a3, bx[i + 1], by[i + 1]);
                }
              } else if constexpr (BL == 8) {
#pragma unroll
                for (int i = 0; i < UNIT; i++) {
                  unsigned a0, a1, a2, a3;
                  tc_ldsm4(sbase + blk + a_lm[u][i], a0, a1, a2, a3);       // the fragment as it is: rows gq / gq + 8, words t / t + 4
                  mma_u8s8(c, a0, a1, a2, a3, bx[i], by[i]);
                }
              } else {
#pragma unroll
                for (int i = 0; i < UNIT; i++) {
                  unsigned a0, a1, a2, a3;
                  tc_load_a<F>(smem, blk + a_lo[u][i], blk + a_hi[u][i], t, a0, a2);
                  tc_load_a<F>(smem, blk + a_lo[u][i] + 1024u, blk + a_hi[u][i] + 1024u, t, a1, a3);
                  mma_u8s8(c, a0, a1, a2, a3, bx[i], by[i]);
                }
              }
              // c[0], c[1]: digit sums of this lane's chunk (or half chunk) for row gq; c[2], c[3]: row gq + 8
              int v0 = c[0] + (c[1] << 8), v1 = c[2] + (c[3] << 8);
              if constexpr (HALVES) {
                if constexpr (INT_MID) { const int mm = (t & 1) ? msx1 : msx0; v0 += mm; v1 += mm; }
                // lanes t and t ^ 1 hold the two halves of one chunk: the even lane finishes row gq, the odd one row gq + 8
                const int give = (t & 1) ? v0 : v1;
                const int got = __shfl_xor_sync(0xffffffffu, give, 1);
                float val[2];
                val[0] = (float)((t & 1) ? got : v0);
                val[1] = (float)((t & 1) ? v1 : got);
                FragT<F> f;
                tc_load_params<F>(f, smem, blk, p_off[u][0]);
                acc[rb][0] += idot_finish<F>(f, val, mt);
              } else {
                if constexpr (INT_MID) { v0 += msx0; v1 += msx0; }
                FragT<F> f0, f1;
                tc_load_params<F>(f0, smem, blk, p_off[u][0]);
                tc_load_params<F>(f1, smem, blk, p_off[u][1]);
                float val[2] = {(float)v0, 0.f};
                acc[rb][0] += idot_finish<F>(f0, val, mt);
                val[0] = (float)v1;
                acc[rb][1] += idot_finish<F>(f1, val, mt);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(fs));
        if (++fs == g.nstage) { fs = 0; fpar ^= 1u; }
      }
      // row sums of this group's blocks: over the quad, then over the warps
      float* mine = red + ((size_t)par * TC_WARPS + warp) * (TC_RB * 16);
#pragma unroll
      for (int rb = 0; rb < TC_RB; rb++) {
        if constexpr (HALVES) {
          float s = acc[rb][0];
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          if (t < 2) mine[rb * 16 + gq + 8 * t] = s;   // t = 0: row gq, t = 1: row gq + 8
        } else {
          float s0 = acc[rb][0], s1 = acc[rb][1];
          s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
          s0 += __shfl_xor_sync(0xffffffffu, s0, 2); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
          if (t == 0) { mine[rb * 16 + gq] = s0; mine[rb * 16 + gq + 8] = s1; }
        }
      }
      asm volatile("bar.sync 15, %0;" ::"n"(TC_WARPS * 32) : "memory");
      if (tid < nb * 16) {
        const float* base = red + (size_t)par * TC_WARPS * (TC_RB * 16) + tid;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < TC_WARPS; w++) sum += base[w * (TC_RB * 16)];
        const int row = (blk0 + gi * g.rb) * 16 + tid;
        if (row < g.nrows) {
          if (pass == 0) yb[row] = sum; else yb[row] += sum;   // the same thread stored this row in the first pass
        }
      }
      par ^= 1;
    }
  }
}

// ------------------------------------------------------------------ host side
static unsigned tc_align(unsigned v, unsigned a) { return (v + a - 1u) & ~(a - 1u); }

static PFN_cuTensorMapEncodeTiled_v12000 tc_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    else cudaGetLastError();
  }
  return fn;
}
// Plane of `rows` rows of `rb` bytes. tiled: seen as {128 B, rows, rb / 128 pieces}, one box = 128 B x 16 rows x np
// pieces, 128-byte swizzle. Otherwise {rb bytes, rows}, one box = segb bytes x 16 rows, no swizzle.
static bool tc_encode(CUtensorMap* out, const void* base, unsigned rb, int rows, bool tiled, unsigned segb) {
  auto fn = tc_encode_fn();
  if (!fn) return false;
  if (tiled) {
    cuuint64_t dims[3] = {128, (cuuint64_t)rows, (cuuint64_t)(rb / 128u)};
    cuuint64_t strides[2] = {(cuuint64_t)rb, 128};
    cuuint32_t box[3] = {128, 16, segb / 128u};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  cuuint64_t dims[2] = {(cuuint64_t)rb, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)rb};
  cuuint32_t box[2] = {segb, 16};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor maps are encoded once per blob plane set and kept: encoding goes through the driver entry point
// and is far too slow to repeat on every launch.
struct TcMaps { CUtensorMap m[5]; };
static std::mutex g_tc_mu;
static std::map<std::tuple<const void*, int, int, int, int>, TcMaps> g_tc_maps;

int wv_act_width();   // wv_gemv_tma.cu: development switch (3 = always take the wide path)
int wv_tc_prequant(); // wv_gemv_tma.cu: development switch (tuning code 31: activation record from the pre-kernel)

template <int F>
static int launch_tc(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb_, int re, cudaStream_t st) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  if constexpr (!TcCfg<F>::OK) { return 1; } else {
  if (b.cols & 31) return 1;
  TcGeom g{};
  g.cpr = b.cols >> 5;
  g.nseg = (g.cpr + TC_SEG - 1) / TC_SEG;
  int ratio = 1;
  if (fi.kind == WK_BINARY || fi.kind == WK_AFFINE) {
    if (b.group < 32 || (b.group % 32) || (b.cols % b.group)) return 1;
    ratio = b.group / 32;
    if ((ratio & (ratio - 1)) || ratio > 16) return 1;
  }
  while ((1 << g.gsh) < ratio) g.gsh++;
  // bytes per chunk of every plane, times TC_SEG = bytes per segment row
  unsigned bpc8[5] = {fi.bits_lo * 32u, fi.bits_hi * 32u, 0, 0, 0};   // bytes per 8 chunks
  switch (fi.kind) {
  case WK_CLASSIC: bpc8[2] = 32; bpc8[3] = fi.has_min ? 32 : 0; break;
  case WK_KQUANT: if (g.cpr % 8) return 1; bpc8[2] = 8; bpc8[4] = fi.has_min ? 32 : 16; break;
  case WK_IQ: case WK_TERNARY: bpc8[2] = fi.pgroup == 16 ? 64 : 32; break;
  case WK_BINARY: bpc8[2] = 32 / ratio; break;
  case WK_AFFINE: bpc8[2] = bpc8[3] = 32 / ratio; break;
  default: return 1;
  }
  const void* base[5] = {b.lo, b.hi, b.p0, b.p1, b.km};
  unsigned rowb[5];
  unsigned off = 0;
  for (int p = 0; p < 5; p++) {
    g.segb[p] = bpc8[p] * (TC_SEG / 8);
    rowb[p] = (unsigned)(((unsigned long long)bpc8[p] * g.cpr) / 8);
    if (!g.segb[p]) continue;
    if (!base[p] || (reinterpret_cast<uintptr_t>(base[p]) & 15)) return 1;
    g.tiled[p] = (g.segb[p] >= 128 && (g.segb[p] % 128) == 0 && (rowb[p] % 128) == 0) ? 1u : 0u;
    if (p < 2 && !g.tiled[p]) return 1;                                 // code planes are read through the swizzle
    if (!g.tiled[p] && (g.segb[p] > 256 || (g.segb[p] % 16) || (rowb[p] % 16))) return 1;
    g.off[p] = off;
    off += g.tiled[p] ? (g.segb[p] / 128u) * 2048u : tc_align(16u * g.segb[p], 1024u);
    g.tx_bytes += g.tiled[p] ? (g.segb[p] / 128u) * 2048u : 16u * g.segb[p];
  }
  g.blk_bytes = off;
  // the activation record in shared memory is the image of the one tc_xquant_kernel writes: digits, scale factors, tail
  const unsigned recb = tc_align((unsigned)g.cpr * 96u + 16u, 128u);
  const unsigned redb = 2u * TC_WARPS * TC_RB * 16u * 4u;
  const unsigned fixed = 1024u + recb + redb + (2u * TC_MAX_STAGES + 1u) * 8u + 128u;
  const unsigned avail = 225u * 1024u;
  // two blocks per stage when at least four such stages fit (the operand words of a unit are then reused for both
  // blocks), else one
  g.rb = ((unsigned long long)g.blk_bytes * 2 * 4 + fixed <= avail) ? 2 : 1;
  const unsigned stage_bytes = g.blk_bytes * (unsigned)g.rb;
  if (stage_bytes * 2 + fixed > avail) return 1;
  int ns = (int)((avail - fixed) / stage_bytes);
  if (ns > TC_MAX_STAGES) ns = TC_MAX_STAGES;
  g.nstage = ns;
  g.dig_off = stage_bytes * ns;
  g.meta_off = g.dig_off + (unsigned)g.cpr * 64u;
  g.red_off = g.dig_off + recb;
  g.bar_off = tc_align(g.red_off + redb, 128u);
  const size_t smem = 1024u + g.bar_off + (2 * TC_MAX_STAGES + 1) * 8;
  g.force_wide = wv_act_width() == 3;
  g.prequant = wv_tc_prequant();
  // scratch for the activation records (first pass and residual per batch row) and the pre-kernel's counters
  if (batch > 256) return 1;
  const unsigned rec_one = tc_align((unsigned)g.cpr * 96u + 16u + TCX_MAX_CTAS * 8u, 256u);
  g.rec_pass = rec_one;
  g.rec_stride = 2u * rec_one;
  unsigned char* recs = reinterpret_cast<unsigned char*>(wv_scratch_take((size_t)batch * g.rec_stride));
  if (!recs) return 1;
  static unsigned* counters = nullptr;
  static unsigned seq = 0;
  static std::mutex cmu;
  unsigned cbase;
  {
    std::lock_guard<std::mutex> lk(cmu);
    if (!counters) {   // first call (set-up, before any capture): 16 groups of 256 zeroed counters
      if (cudaMalloc(&counters, 4096 * sizeof(unsigned)) != cudaSuccess) { cudaGetLastError(); return 1; }
      cudaMemset(counters, 0, 4096 * sizeof(unsigned));
    }
    cbase = (seq++ & 15u) * 256u;
  }

  TcMaps maps;
  {
    std::lock_guard<std::mutex> lk(g_tc_mu);
    const auto key = std::make_tuple((const void*)b.lo, b.rows, b.cols, b.format, b.group);
    auto it = g_tc_maps.find(key);
    if (it == g_tc_maps.end()) {
      TcMaps m{};
      for (int p = 0; p < 5; p++) {
        const int q = g.segb[p] ? p : 0;   // absent planes carry a copy of the lo map (never used)
        if (!tc_encode(&m.m[p], base[q], rowb[q], b.rows, g.tiled[q] != 0, g.segb[q])) {
          static bool warned = false;
          if (!warned) { warned = true; fprintf(stderr, "welvet_cuda: tensor-map encoding failed, using the dp4a kernel\n"); }
          return 1;
        }
      }
      if (g_tc_maps.size() > 4096) g_tc_maps.clear();
      it = g_tc_maps.emplace(key, m).first;
    }
    maps = it->second;
  }

  g.nrows = re - rb_;
  const int total_blk = (g.nrows + 15) / 16;
  int grid = wv_sm_count();
  if (grid > total_blk) grid = total_blk;
  g.blk_base = total_blk / grid;
  g.blk_rem = total_blk % grid;
  int dev = 0; cudaGetDevice(&dev);
  auto kern = gemv_tc_kernel<F>;
  static unsigned attr_mask = 0;
  if (!(attr_mask & (1u << dev))) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) { wv_set_error("gemv (tc): cannot raise the shared-memory limit"); return WV_ECUDA; }
    attr_mask |= 1u << dev;
  }
  if (g.prequant) {
    const int ntask = g.cpr * 4;
    int nx = (ntask + TCX_THREADS - 1) / TCX_THREADS;
    if (nx > TCX_MAX_CTAS) nx = TCX_MAX_CTAS;
    cudaError_t ex = launch_pdl(tc_xquant_kernel<fi.bits_lo>, dim3(nx, batch), dim3(TCX_THREADS), 0, st, dx, b.cols,
                                TcCfg<F>::INT_MID ? fi.mid : 0, TcCfg<F>::HALVES ? 1 : 0, recs, g.rec_stride, g.rec_pass, counters + cbase, g.force_wide);
    if (ex != cudaSuccess) { wv_set_error("gemv (tc) activation record launch: %s", cudaGetErrorString(ex)); return WV_ECUDA; }
  }
  cudaError_t e = launch_pdl(kern, dim3(grid, batch), dim3(TC_THREADS), smem, st, b, g.prequant ? (const unsigned char*)recs : reinterpret_cast<const unsigned char*>(dx), dy, rb_, g, wv_tma_err_ptr(),
                             maps.m[0], maps.m[1], maps.m[2], maps.m[3], maps.m[4]);
  if (e != cudaSuccess) { wv_set_error("gemv (tc) launch: %s", cudaGetErrorString(e)); return WV_ECUDA; }
  return WV_OK;
  }
}

// Returns WV_OK, an error, or 1 when the format or shape is not served by this kernel.
int wv_launch_gemv_tc(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st) {
  switch (b.format) {
#define WV_F(f) case f: return launch_tc<f>(b, dx, dy, batch, row_begin, row_end, st);
  WV_F(WV_Q8_0) WV_F(WV_Q4_0) WV_F(WV_Q4_1) WV_F(WV_Q5_0) WV_F(WV_Q5_1)
  WV_F(WV_Q2_K) WV_F(WV_Q3_K) WV_F(WV_Q4_K) WV_F(WV_Q5_K) WV_F(WV_Q6_K)
  WV_F(WV_IQ1_S) WV_F(WV_IQ2_XXS) WV_F(WV_IQ2_XS) WV_F(WV_IQ3_XXS) WV_F(WV_IQ3_S) WV_F(WV_IQ4_XS)
  WV_F(WV_TERNARY) WV_F(WV_BINARY) WV_F(WV_AFFINE)
#undef WV_F
  }
  return 1;
}
