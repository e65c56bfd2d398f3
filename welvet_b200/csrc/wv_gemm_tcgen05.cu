// Batched Dense MatVec (batch >= 2 activation rows against one packed matrix) on the fifth-generation tensor
// cores: Y[batch][rows] = X[batch][cols] * W^T with W streamed and dequantised once, whatever the batch.
//
// The reference runs dense.Forward row by row over the batch (layers/dense/simd.go:557-614 per row,
// gemv_parallel.go:12-391); its WebGPU shaders do the same per dispatch. Here the batch is the N dimension of a
// tcgen05.mma: a CTA owns 128 rows of W (the MMA's M) and a range of the columns (split-K); per 32 columns its 512
// producer threads dequantise a 128 x 32 slice of W to TF32 values in the canonical K-major 128-byte-swizzled
// operand layout in shared memory and stage the matching slice of X (rounded to TF32) beside it, one elected thread
// issues four tcgen05.mma (M 128, N = batch padded to 16, K 8) per slice into a TMEM accumulator, tcgen05.commit
// hands the stage back, and at the end four warps read the accumulator with tcgen05.ld and store Y (or the split's
// partial, which the last split of the row tile to finish adds up in split order).
//
// Arithmetic: both operands are rounded to TF32 (round to nearest, 11 significant bits) by the producers, so the
// hardware's truncation of the low mantissa bits drops zeros; products are exact in the FP32 accumulator. Each term
// is off by at most 2^-11 + 2^-11 + 2^-22 of |w x|, i.e. |y - y_ref| <= 9.8e-4 * sum |w x| before accumulation
// rounding. TF32 keeps FP32's exponent range, so no operand needs scaling.
//
// Every wait is bounded: a wait that runs out records a code in the mapped error word, raises the CTA's abort flag,
// and all roles fall through to the common exit, where the TMEM columns are released.
#include "wv_common.cuh"
#include "wv_tma_common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <mutex>

#define TCG_PRODUCERS 512
#define TCG_THREADS (TCG_PRODUCERS + 64)     // + the MMA warp and the warp whose first lane issues the X copies
#define TCG_MAX_STAGES 6
#define TCG_M 128
#define TCG_KB 2            // 32-column slices per pipeline stage

__constant__ float c_tcg_iq4nl[16] = WV_IQ4NL_GRID;

// ------------------------------------------------------------------ dequantisation of a quarter chunk (8 weights)
// The unpack kernel's arithmetic with the parameters of the 8 weights hoisted. The values are rounded to TF32 right
// after, so the two places where the reference divides (k-quant scale / 255, min / 127) multiply by the reciprocal
// here: the difference is one unit in the 24th bit, against the rounding to 11 bits that follows.
struct TcgRaw { unsigned lo[2]; unsigned hi[2]; float p0, p1; unsigned km; };

// q (0..3) names the 8 weights of chunk ch; the four threads that share a chunk are neighbouring lanes, so that a
// warp's loads fall into whole 32-byte sectors (8 rows x 4 quarters per warp).
template <int F>
__device__ __forceinline__ void tcg_load_raw(TcgRaw& r, const WvDevBlob& b, long long ch, int q) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi;
  const int half = q >> 1;
  if constexpr (BL == 8) { const uint2 v = __ldg(reinterpret_cast<const uint2*>(b.lo + ch * 8) + q); r.lo[0] = v.x; r.lo[1] = v.y; }
  else if constexpr (BL == 4) r.lo[0] = __ldg(b.lo + ch * 4 + q);
  else if constexpr (BL == 2) r.lo[0] = __ldg(b.lo + ch * 2 + half) >> (16 * (q & 1));
  else r.lo[0] = __ldg(b.lo + ch) >> (8 * q);
  if constexpr (BH >= 1) r.hi[0] = __ldg(b.hi + ch * BH);
  if constexpr (BH == 2) r.hi[1] = __ldg(b.hi + ch * BH + 1);
  const long long i = ch * 32 + q * 8;   // flat index of the first weight
  if constexpr (fi.kind == WK_CLASSIC) {
    r.p0 = __ldg(b.p0 + ch);
    if constexpr (fi.has_min) r.p1 = __ldg(b.p1 + ch);
  } else if constexpr (fi.kind == WK_KQUANT) {
    const float2 dd = __ldg(reinterpret_cast<const float2*>(b.p0) + (ch >> 3));
    r.p0 = dd.x; r.p1 = dd.y;
    if constexpr (fi.has_min) r.km = __ldg(b.km + ch);
    else r.km = __ldg(reinterpret_cast<const unsigned short*>(b.km) + ch);
  } else if constexpr (fi.kind == WK_IQ || fi.kind == WK_TERNARY) {
    r.p0 = __ldg(b.p0 + (fi.pgroup == 16 ? ch * 2 + half : ch));
  } else if constexpr (fi.kind == WK_BINARY) {
    r.p0 = __ldg(b.p0 + i / b.group);
  } else if constexpr (fi.kind == WK_AFFINE) {
    r.p0 = __ldg(b.p0 + i / b.group);
    r.p1 = __ldg(b.p1 + i / b.group);
  }
}

template <int F>
__device__ __forceinline__ void tcg_convert(const TcgRaw& r, int q, float (&w)[8]) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi;
  const int half = q >> 1;
  float sc = r.p0, mn = 0.f;
  if constexpr (fi.kind == WK_CLASSIC) { if constexpr (fi.has_min) mn = r.p1; }
  if constexpr (fi.kind == WK_AFFINE) mn = r.p1;
  if constexpr (fi.kind == WK_KQUANT) {
    const unsigned su = (r.km >> (8 * half)) & 0xffu;
    sc = r.p0 * (float)(su ? su : 1u) * (1.0f / 255.0f);    // a zero scale byte stands for d / 255 (quant/kquant.go:180-182)
    if constexpr (fi.has_min) {
      const unsigned mu = (r.km >> (16 + 8 * half)) & 0xffu;
      mn = r.p1 * (float)(int)(signed char)mu * (1.0f / 127.0f);
    }
  }
  // code -> float without an integer conversion: the code lands in the mantissa of 2^23, and subtracting
  // 2^23 + mid leaves (code - mid) exactly
  constexpr float magic = 8388608.0f + (float)((fi.kind == WK_CLASSIC || fi.kind == WK_KQUANT) && !fi.has_min ? fi.mid : 0);
#pragma unroll
  for (int j = 0; j < 8; j++) {
    constexpr unsigned mask = (1u << BL) - 1u;
    unsigned u = (r.lo[(j * BL) >> 5] >> ((j * BL) & 31)) & mask;
    unsigned ubits = u | 0x4B000000u;
    if constexpr (BL == 8 && BH == 0) ubits = __byte_perm(r.lo[j >> 2], 0x4B000000u, 0x7440u + (unsigned)(j & 3));   // one instruction: byte j under the exponent of 2^23
    if constexpr (BH > 0) {
      const int jj = q * 8 + j;
      const int k = wv_k_of(BL, jj), m = wv_m_of(BL, jj);
      const unsigned hw = (BH == 2 && wv_hi_word(BH, k)) ? r.hi[1] : r.hi[0];
      u |= ((hw >> wv_hi_bit(BH, k, m)) & ((1u << BH) - 1u)) << BL;
    }
    if constexpr (BH > 0) ubits = u | 0x4B000000u;
    const float uf = __uint_as_float(ubits) - magic;     // (code - mid) for the symmetric block formats, the code otherwise
    float v;
    if constexpr (fi.kind == WK_CLASSIC || fi.kind == WK_KQUANT) v = fi.has_min ? fmaf(uf, sc, mn) : uf * sc;
    else if constexpr (fi.kind == WK_IQ) {
      if constexpr (fi.table) v = sc * c_tcg_iq4nl[u & 15];
      else if constexpr (fi.sign) v = (u & 1) ? sc : -sc;
      else v = sc * (uf - ((float)fi.mid + 0.5f));
    }
    else if constexpr (fi.kind == WK_TERNARY) v = u == 0 ? -sc : (u == 2 ? sc : 0.0f);
    else if constexpr (fi.kind == WK_BINARY) v = (u & 1) ? sc : -sc;
    else v = fmaf(sc, uf, mn);   // affine
    w[j] = v;
  }
}

__device__ __forceinline__ float tcg_tf32(float v) {
  unsigned o;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(o) : "f"(v));
  return __uint_as_float(o);
}

// ------------------------------------------------------------------ tcgen05 plumbing
__device__ __forceinline__ void tcg_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcg_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Shared-memory operand descriptor: K-major, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long tcg_desc(unsigned saddr) {
  return (unsigned long long)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((unsigned long long)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tcg_mma_tf32(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tcg_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcg_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

struct TcgGeom {
  int row_begin, row_end;     // rows of the blob this launch covers
  int cpr;                    // chunks (32 columns) per row
  int batch, npad;            // activation rows, and that padded to a multiple of 16 (the MMA's N)
  int ksplit, cps;            // column splits and chunks per split
  int nstage;
  unsigned a_bytes, b_bytes, stage_bytes;   // one slice of A (128 rows x 128 bytes) and of B; a stage holds TCG_KB of each
  unsigned tmem_cols;         // power of two >= max(32, npad)
  int y_stride;               // floats between consecutive activation rows' outputs
};

template <int F, int D>   // D: stages whose weight loads are in flight
__global__ void __launch_bounds__(TCG_THREADS, 1)
gemm_tcgen05_kernel(const WvDevBlob b, const __grid_constant__ CUtensorMap xmap, float* __restrict__ y, float* __restrict__ part,
                    unsigned* __restrict__ counters, const TcgGeom g, int* __restrict__ err) {
  extern __shared__ __align__(1024) unsigned char tcg_smem[];
  __shared__ __align__(8) unsigned long long s_bar[2 * TCG_MAX_STAGES + 1];
  __shared__ unsigned s_tmem;
  __shared__ int s_abort;
  __shared__ unsigned s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mt = blockIdx.x, sp = blockIdx.y;
  const int m0 = g.row_begin + mt * TCG_M;
  const int kc0 = sp * g.cps, kc1 = min(g.cpr, kc0 + g.cps);
  const int nk = max(0, kc1 - kc0);
  const int nst = (nk + TCG_KB - 1) / TCG_KB;    // pipeline stages to work through
  // the dynamic segment is declared 1024-byte aligned; round up all the same (the swizzle pattern is relative to 1024 bytes)
  const unsigned sbase = (smem_u32(tcg_smem) + 1023u) & ~1023u;
  auto full_bar = [&](int s) { return smem_u32(&s_bar[s]); };
  auto empty_bar = [&](int s) { return smem_u32(&s_bar[TCG_MAX_STAGES + s]); };
  const unsigned done_bar = smem_u32(&s_bar[2 * TCG_MAX_STAGES]);

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < g.nstage; s++) { mbar_init(full_bar(s), TCG_PRODUCERS / 32 + 1); mbar_init(empty_bar(s), 1); }
    mbar_init(done_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == TCG_PRODUCERS / 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(g.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcg_fence_before();
  __syncthreads();
  tcg_fence_after();
  const unsigned tmem = *(volatile unsigned*)&s_tmem;
  // The weights do not depend on the preceding kernel: the producers start at once. Only the thread that copies X waits
  // for it (X was rounded by the kernel right before this one), and nothing is stored before X has arrived.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp < TCG_PRODUCERS / 32) {
    // ------------------------------------------------------------ producers
    const int row_l = tid >> 2;
    const int quarter = tid & 3;                                 // which 8 of a chunk's 32 weights
    const int row = min(m0 + row_l, g.row_end - 1);              // rows past the end repeat the last one and are not stored
    const long long ch_row = (long long)row * g.cpr;
    // this thread's part of the A slice: 32 bytes of row row_l, 16-byte pieces quarter*2, quarter*2+1, swizzled by the row
    const unsigned a_off = (unsigned)(row_l >> 3) * 1024u + (unsigned)(row_l & 7) * 128u;
    // A stage holds TCG_KB consecutive 32-column slices (the barrier traffic and the loop's bookkeeping are paid per
    // stage, not per slice). Loads run D stages ahead of the conversion (they take about a microsecond to come back):
    // D register sets, the stage loop unrolled by D so that they are indexed statically.
    TcgRaw raw[D][TCG_KB];
    auto load = [&](TcgRaw (&r)[TCG_KB], int it) {
#pragma unroll
      for (int kb = 0; kb < TCG_KB; kb++) {
        const int kc = kc0 + it * TCG_KB + kb;
        if (kc < kc1) tcg_load_raw<F>(r[kb], b, ch_row + kc, quarter);
      }
    };
#pragma unroll
    for (int d = 0; d < D; d++) if (d < nst) load(raw[d], d);
    int s = 0;
    unsigned epar = 1;     // parity of the "empty" phase to wait for once the ring has wrapped
    bool wrapped = false;
    bool dead = false;
    for (int it0 = 0; it0 < nst && !dead; it0 += D) {
#pragma unroll
      for (int d = 0; d < D; d++) {
        const int it = it0 + d;
        if (it >= nst || dead) break;
        bool bad = *(volatile int*)&s_abort != 0;
        if (!bad && wrapped && !mbar_wait(empty_bar(s), epar)) { atomicCAS_system(err, 0, 500 + s); *(volatile int*)&s_abort = 1; bad = true; }
        if (__any_sync(0xffffffffu, bad)) { dead = true; break; }     // the whole warp leaves together (it meets at __syncwarp below)
        const unsigned st = sbase + (unsigned)s * g.stage_bytes;
#pragma unroll
        for (int kb = 0; kb < TCG_KB; kb++) {
          if (kc0 + it * TCG_KB + kb >= kc1) break;    // past the split's last slice: the MMA thread skips it too
          float w[8];
          tcg_convert<F>(raw[d][kb], quarter, w);
#pragma unroll
          for (int p = 0; p < 2; p++) {
            const unsigned piece = (unsigned)(quarter * 2 + p) ^ (unsigned)(row_l & 7);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(st + kb * g.a_bytes + a_off + piece * 16u), "f"(tcg_tf32(w[4 * p])),
                         "f"(tcg_tf32(w[4 * p + 1])), "f"(tcg_tf32(w[4 * p + 2])), "f"(tcg_tf32(w[4 * p + 3])) : "memory");
          }
        }
        if (it + D < nst) load(raw[d], it + D);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(s));      // one arrival per warp
        if (++s == g.nstage) { s = 0; wrapped = true; epar ^= 1u; }
      }
    }
  } else if (warp == TCG_PRODUCERS / 32 + 1) {
    // ------------------------------------------------------------ X copies (one thread): a stage's slices of the rounded
    // activations arrive by tensor-map copies with the 128-byte swizzle, i.e. already in the operand layout; rows past
    // the batch are zero-filled by the copy engine
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      int s = 0;
      unsigned epar = 1;
      bool wrapped = false;
      for (int it = 0; it < nst; it++) {
        if (*(volatile int*)&s_abort) break;
        if (wrapped && !mbar_wait(empty_bar(s), epar)) { atomicCAS_system(err, 0, 530 + s); *(volatile int*)&s_abort = 1; break; }
        const int nkb = min(TCG_KB, nk - it * TCG_KB);
        mbar_expect_tx(full_bar(s), (unsigned)nkb * g.b_bytes);
        const unsigned st = sbase + (unsigned)s * g.stage_bytes + TCG_KB * g.a_bytes;
        for (int kb = 0; kb < nkb; kb++) tma_load_2d(st + kb * g.b_bytes, &xmap, (kc0 + it * TCG_KB + kb) * 32, 0, full_bar(s));
        if (++s == g.nstage) { s = 0; wrapped = true; epar ^= 1u; }
      }
    }
  } else if (lane == 0) {
    // ------------------------------------------------------------ MMA issuer (one thread)
    const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(g.npad >> 3) << 17) | ((unsigned)(TCG_M >> 4) << 24);
    int s = 0;
    unsigned fpar = 0;
    for (int it = 0; it < nst; it++) {
      if (*(volatile int*)&s_abort) break;
      if (!mbar_wait(full_bar(s), fpar)) { atomicCAS_system(err, 0, 510 + s); *(volatile int*)&s_abort = 1; break; }
      tcg_fence_after();
      const unsigned st = sbase + (unsigned)s * g.stage_bytes;
#pragma unroll
      for (int kb = 0; kb < TCG_KB; kb++) {
        if (it * TCG_KB + kb >= nk) break;       // the split's last stage may hold one slice only
        const unsigned long long da = tcg_desc(st + kb * g.a_bytes), db = tcg_desc(st + TCG_KB * g.a_bytes + kb * g.b_bytes);
#pragma unroll
        for (int k = 0; k < 4; k++)   // 8 TF32 values = 32 bytes further along K inside the swizzled row
          tcg_mma_tf32(tmem, da + (unsigned long long)(2 * k), db + (unsigned long long)(2 * k), idesc, (it > 0 || kb > 0 || k > 0) ? 1u : 0u);
      }
      tcg_commit(empty_bar(s));        // arrives when these MMAs have read the stage
      if (++s == g.nstage) { s = 0; fpar ^= 1u; }
    }
    tcg_commit(done_bar);               // arrives when every MMA issued above has finished
  }

  // ---------------------------------------------------------------- epilogue: warps 0-3 own TMEM lanes 32 w .. 32 w + 31
  float* dst = g.ksplit == 1 ? y : part + ((size_t)mt * g.ksplit + sp) * (size_t)g.batch * TCG_M;
  if (warp < 4) {
    bool ok = !*(volatile int*)&s_abort;
    if (ok && nk > 0 && !mbar_wait(done_bar, 0)) { atomicCAS_system(err, 0, 520); *(volatile int*)&s_abort = 1; ok = false; }
    ok = __all_sync(0xffffffffu, ok);     // tcgen05.ld is warp-wide
    tcg_fence_after();
    const int row_l = warp * 32 + lane;
    const bool row_ok = m0 + row_l < g.row_end;
    for (int c0 = 0; c0 < g.npad; c0 += 16) {
      float v[16];
      if (ok && nk > 0) tcg_ld16(tmem + ((unsigned)(warp * 32) << 16) + (unsigned)c0, v);
      else {
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int m = c0 + j;
        if (m < g.batch) {
          if (g.ksplit == 1) { if (row_ok) dst[(size_t)m * g.y_stride + m0 + row_l] = v[j]; }
          else dst[(size_t)m * TCG_M + row_l] = v[j];
        }
      }
    }
  }
  tcg_fence_before();
  if (g.ksplit > 1) __threadfence();
  __syncthreads();
  if (warp == TCG_PRODUCERS / 32) {
    tcg_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(g.tmem_cols) : "memory");
  }
  if (g.ksplit == 1) return;
  // ---------------------------------------------------------------- the last split of this row tile adds the partials up, in split order
  if (tid == 0) {
    const unsigned prev = atomicAdd(&counters[mt], 1u);
    s_last = (prev == (unsigned)g.ksplit - 1u);
    if (s_last) counters[mt] = 0u;   // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* base = part + (size_t)mt * g.ksplit * (size_t)g.batch * TCG_M;
  const size_t per = (size_t)g.batch * TCG_M;
  for (int e = tid; e < g.batch * TCG_M; e += TCG_THREADS) {
    const int m = e / TCG_M, row_l = e - m * TCG_M;
    float v[8];
    float sum = 0.f;
    for (int s0 = 0; s0 < g.ksplit; s0 += 8) {
#pragma unroll
      for (int u = 0; u < 8; u++) v[u] = s0 + u < g.ksplit ? __ldcg(base + (size_t)(s0 + u) * per + e) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; u++) if (s0 + u < g.ksplit) sum += v[u];
    }
    if (m0 + row_l < g.row_end) y[(size_t)m * g.y_stride + m0 + row_l] = sum;
  }
}

// X rounded to TF32 (round to nearest), element for element.
__global__ void __launch_bounds__(256) tcg_round_x_kernel(const float4* __restrict__ x, float4* __restrict__ xr, size_t n4) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = x[i];
    xr[i] = make_float4(tcg_tf32(v.x), tcg_tf32(v.y), tcg_tf32(v.z), tcg_tf32(v.w));
  }
}

// ------------------------------------------------------------------ host side
static float* g_tcg_xr = nullptr;
static size_t g_tcg_xr_floats = 0;
static PFN_cuTensorMapEncodeTiled_v12000 tcg_encode_fn() {
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
static float* g_tcg_part = nullptr;
static size_t g_tcg_part_floats = 0;
static unsigned* g_tcg_cnt = nullptr;
static int g_tcg_cnt_n = 0;
static std::mutex g_tcg_mu;

int wv_sm_count();

template <int F>
static int launch_tcg(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb, int re, cudaStream_t st) {
  TcgGeom g{};
  g.row_begin = rb; g.row_end = re;
  g.cpr = b.cols >> 5;
  g.batch = batch;
  g.npad = (batch + 15) & ~15;
  g.y_stride = b.rows;
  const int rows = re - rb;
  const int mtiles = (rows + TCG_M - 1) / TCG_M;
  // column splits: enough CTAs for the SMs, at least 8 chunks (256 columns) per split
  int ks = wv_sm_count() / mtiles;
  if (ks > g.cpr / 8) ks = g.cpr / 8;
  if (ks < 1) ks = 1;
  g.cps = (g.cpr + ks - 1) / ks;
  g.ksplit = (g.cpr + g.cps - 1) / g.cps;
  g.a_bytes = TCG_M * 128u;
  g.b_bytes = (unsigned)g.npad * 128u;
  g.stage_bytes = TCG_KB * (g.a_bytes + g.b_bytes);
  int ns = (int)((200u * 1024u) / g.stage_bytes);
  if (ns > TCG_MAX_STAGES) ns = TCG_MAX_STAGES;
  if (ns < 2) return 1;
  g.nstage = ns;
  g.tmem_cols = 32;
  while ((int)g.tmem_cols < g.npad) g.tmem_cols *= 2;
  const size_t smem = (size_t)ns * g.stage_bytes + 1024;
  float* part = nullptr;
  unsigned* cnt = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_tcg_mu);
    if (g.ksplit > 1) {
      const size_t need = (size_t)mtiles * g.ksplit * batch * TCG_M;
      if (need > g_tcg_part_floats) {       // grows when a larger shape arrives (set-up time: not capturable)
        cudaStreamSynchronize(st);
        if (g_tcg_part) cudaFree(g_tcg_part);
        g_tcg_part = nullptr; g_tcg_part_floats = 0;
        if (cudaMalloc(&g_tcg_part, need * 4) != cudaSuccess) { cudaGetLastError(); wv_set_error("batched matvec: %zu bytes of split scratch unavailable", need * 4); return WV_ENOMEM; }
        g_tcg_part_floats = need;
      }
      if (mtiles > g_tcg_cnt_n) {
        cudaStreamSynchronize(st);
        if (g_tcg_cnt) cudaFree(g_tcg_cnt);
        g_tcg_cnt = nullptr; g_tcg_cnt_n = 0;
        const int n = mtiles < 4096 ? 4096 : mtiles;
        if (cudaMalloc(&g_tcg_cnt, (size_t)n * 4) != cudaSuccess) { cudaGetLastError(); wv_set_error("batched matvec: counter allocation failed"); return WV_ENOMEM; }
        cudaMemset(g_tcg_cnt, 0, (size_t)n * 4);
        g_tcg_cnt_n = n;
      }
    }
    part = g_tcg_part; cnt = g_tcg_cnt;
  }
  // X rounded to TF32 once, by a small kernel in front (each of the row tiles would otherwise round it again), into a
  // buffer of the library; the main kernel fetches it through a tensor map encoded per call.
  float* xr = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_tcg_mu);
    const size_t need = (size_t)batch * b.cols;
    if (need > g_tcg_xr_floats) {
      cudaStreamSynchronize(st);
      if (g_tcg_xr) cudaFree(g_tcg_xr);
      g_tcg_xr = nullptr; g_tcg_xr_floats = 0;
      if (cudaMalloc(&g_tcg_xr, need * 4) != cudaSuccess) { cudaGetLastError(); wv_set_error("batched matvec: %zu bytes for the rounded activations unavailable", need * 4); return WV_ENOMEM; }
      g_tcg_xr_floats = need;
    }
    xr = g_tcg_xr;
  }
  auto enc = tcg_encode_fn();
  if (!enc) return 1;
  CUtensorMap xmap;
  {
    cuuint64_t dims[2] = {(cuuint64_t)b.cols, (cuuint64_t)batch};
    cuuint64_t strides[1] = {(cuuint64_t)b.cols * 4};
    cuuint32_t box[2] = {32, (cuuint32_t)g.npad};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, xr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return 1;
  }
  auto kern = gemm_tcgen05_kernel<F, 4>;
  static unsigned attr_mask = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_mask & (1u << (dev & 31)))) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024) != cudaSuccess) { wv_set_error("batched matvec: cannot raise the shared-memory limit"); return WV_ECUDA; }
    attr_mask |= 1u << (dev & 31);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(mtiles, g.ksplit); cfg.blockDim = dim3(TCG_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  int* err = wv_tma_err_ptr();
  {
    const size_t n4 = (size_t)batch * b.cols / 4;
    cudaLaunchConfig_t rc_ = {};
    int blocks = (int)((n4 + 255) / 256);
    if (blocks > 2 * 148) blocks = 2 * 148;
    rc_.gridDim = dim3(blocks); rc_.blockDim = dim3(256); rc_.stream = st;
    rc_.attrs = at; rc_.numAttrs = 1;
    if (cudaLaunchKernelEx(&rc_, tcg_round_x_kernel, reinterpret_cast<const float4*>(dx), reinterpret_cast<float4*>(xr), n4) != cudaSuccess) {
      wv_set_error("batched matvec (rounding) launch: %s", cudaGetErrorString(cudaGetLastError())); return WV_ECUDA;
    }
  }
  if (cudaLaunchKernelEx(&cfg, kern, b, xmap, dy, part, cnt, g, err) != cudaSuccess) { wv_set_error("batched matvec launch: %s", cudaGetErrorString(cudaGetLastError())); return WV_ECUDA; }
  return WV_OK;
}

// Batched y[m][rows] = x[m][cols] W^T for 2 <= batch <= 256 activation rows. Returns 1 for what this kernel does not
// take (FormatNone, rows that do not start on chunk boundaries, unaligned x), so that the caller runs the rows one by one.
int wv_launch_gemm_tcgen05(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st) {
  if (batch < 2 || batch > 256 || !b.fast || b.format == WV_NONE || (b.cols & 31) || row_end <= row_begin) return 1;
  if ((reinterpret_cast<uintptr_t>(dx) & 15) || !wv_tma_err_ptr()) return 1;
  switch (b.format) {
#define WV_F(f) case f: return launch_tcg<f>(b, dx, dy, batch, row_begin, row_end, st);
  WV_F(WV_Q8_0) WV_F(WV_Q4_0) WV_F(WV_Q4_1) WV_F(WV_Q5_0) WV_F(WV_Q5_1)
  WV_F(WV_Q2_K) WV_F(WV_Q3_K) WV_F(WV_Q4_K) WV_F(WV_Q5_K) WV_F(WV_Q6_K)
  WV_F(WV_IQ1_S) WV_F(WV_IQ2_XXS) WV_F(WV_IQ2_XS) WV_F(WV_IQ3_XXS) WV_F(WV_IQ3_S) WV_F(WV_IQ4_NL) WV_F(WV_IQ4_XS)
  WV_F(WV_TERNARY) WV_F(WV_BINARY) WV_F(WV_AFFINE)
#undef WV_F
  }
  return 1;
}
