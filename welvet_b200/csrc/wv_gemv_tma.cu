// TMA-fed GEMV for sm_100a: the packed planes of a band of rows are pulled into a shared-memory
// ring by bulk asynchronous copies (cp.async.bulk + mbarrier), so the bytes in flight per SM
// are set by the ring depth (100-200 KB) rather than by registers, and the consumer warps never
// compute a global address.
//
//   * one CTA per SM owns a contiguous band of output rows; a producer thread streams the band
//     tile by tile (TR rows of every plane, each plane's rows contiguous -> one bulk copy per
//     plane per tile) through STAGES buffers guarded by full/empty mbarriers;
//   * weights do not depend on the preceding kernel, so the producer starts before
//     griddepcontrol.wait (programmatic dependent launch overlaps the previous kernel's tail);
//   * every consumer lane owns one 32-column chunk for the whole kernel and keeps that chunk's
//     quantised activations in registers (no per-step activation loads); a row's partial sums
//     are reduced with warp shuffles and then across the column warps through shared memory,
//     32 rows at a time, so y is written with coalesced stores;
//   * all waits on mbarriers are bounded: when a wait runs out the CTA records an error code,
//     stops issuing copies, drains the ones in flight (bounded again) and returns.
#include "wv_gemv_common.cuh"
#include "wv_dev_hooks.h"
#include "wv_tma_common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <array>
#include <map>
#include <mutex>
#include <tuple>

#ifndef TMA_CONSUMER_WARPS
#define TMA_CONSUMER_WARPS 16
#endif
#define TMA_THREADS ((TMA_CONSUMER_WARPS + 1) * 32)
#define TMA_MAX_STAGES 8
#ifndef TMA_MAX_ROW_GROUPS
#define TMA_MAX_ROW_GROUPS 8
#endif

struct TmaGeom {
  int cpr;           // chunks per row
  int nwc;           // column warps per row (ceil(cpr/32))
  int nrg;           // row groups working side by side on one tile
  int tr;            // rows per tile = nrg * RT
  int nstage;
  unsigned stage_bytes;
  unsigned off[5];   // lo, hi, p0, p1, km section offsets inside a stage
  unsigned rb[5];    // bytes per row of each plane (0 = plane absent)
  int rows_base, rows_rem;  // single matrix: CTA b owns rows_base (+1 if b < rows_rem) consecutive rows
  int lead;          // tiles issued before the producer waits for the activation loads to be on their way
  int force3;        // development switch: always use the 24-bit activation records
  unsigned x_off;    // staged activations: 33 floats per chunk (32 + one of padding)
  unsigned red_off;  // float red[2][nrg][nwc][32]
  unsigned gate_off; // gate | up launches: the gate's row sums of this CTA's band (TMA_GATE_ROWS floats)
  unsigned bar_off;  // full[nstage], empty[nstage]
  // Rows wider than the consumer warps cover (more than 16384 columns) are worked through in ncp column passes
  // (grouped instance only): cpr and rb[] then describe one pass's slice of a row, pitch[] the whole row, and the
  // passes' partial row sums wait in shared memory (TMA_GATE_ROWS floats per matrix at part_off).
  int ncp;
  unsigned pitch[5];
  unsigned part_off;
  unsigned nsegp[5];   // column passes: a row slice of plane i is nsegp[i] innermost boxes of its tensor map
  const void* maps;    // column passes: five tensor maps in device memory, plane i seen as {box bytes, pieces of a row, rows}
};

// The matrices one launch works through (same format, columns and group; they share x): the
// planes, output vector and row split of each. A plain GEMV is a group of one.
#define TMA_MAX_GROUP 4
#define TMA_GATE_ROWS 512
struct TmaGroup {
  int n;
  int rows[TMA_MAX_GROUP];
  int rows_base[TMA_MAX_GROUP], rows_rem[TMA_MAX_GROUP];   // CTA b owns rows_base (+1 if b < rows_rem) consecutive rows of matrix i
  const void* plane[TMA_MAX_GROUP][5];                      // lo, hi, p0, p1, km
  float* y[TMA_MAX_GROUP];
};

// What only the grouped launch and the peer-storing epilogue need. The plain GEMV is instantiated
// without it: the extra parameters and loop nest cost 0.3-0.6 us per launch when they were always there.
struct TmaExt {
  TmaGroup grp;
  int mode;                 // 0: y_i = W_i x;  1: matrices 0 | 1 are gate | up and the one output is silu(W_0 x) * (W_1 x)
  int npeers;               // > 0: every output row goes to all ranks' vectors py[matrix][rank] instead of grp.y[matrix]
  const float* residual;    // single matrix: added to each row sum before the store (may alias the output)
  float* py[TMA_MAX_GROUP][WV_MAX_PEERS];
  const float* norm_gamma;  // NORM instance: RMSNorm weights; x is normalised between the copy into shared memory and the records
  double norm_eps;
};
struct TmaNoExt {};
template <bool EXT> struct TmaExtArgs { using type = TmaNoExt; };
template <> struct TmaExtArgs<true> { using type = TmaExt; };

// Sticky code of the first bounded wait that ran out, in mapped pinned host memory so that the
// host can poll it without a CUDA call.
static int* g_err_host = nullptr;
static int* g_err_dev = nullptr;

// Per-lane shared-memory addresses (32-bit) of this lane's chunk in row 0 of its row group,
// relative to a stage base; a row further down adds the plane's row bytes.
struct LaneOff { unsigned lo, hi, p0, p1, km; };

template <int F>
__device__ __forceinline__ LaneOff lane_offsets(const TmaGeom& g, int row0, int c, int group) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  LaneOff o;
  o.lo = g.off[0] + row0 * g.rb[0] + c * fi.bits_lo * 4;
  o.hi = g.off[1] + row0 * g.rb[1] + c * fi.bits_hi * 4;
  unsigned pi;
  if constexpr (fi.kind == WK_KQUANT) pi = (c >> 3) * 8;
  else if constexpr (fi.kind == WK_BINARY || fi.kind == WK_AFFINE) pi = ((c * 32) / group) * 4;
  else if constexpr (fi.pgroup == 16) pi = c * 8;
  else pi = c * 4;
  o.p0 = g.off[2] + row0 * g.rb[2] + pi;
  o.p1 = g.off[3] + row0 * g.rb[3] + pi;
  o.km = g.off[4] + row0 * g.rb[4] + c * (fi.has_min ? 4 : 2);
  return o;
}

// Weight fragment at addresses a.* (already advanced to the wanted row and stage).
template <int F>
__device__ __forceinline__ void load_frag_smem(FragT<F>& f, const LaneOff& a) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi;
  if constexpr (BL == 1) f.lo[0] = lds32(a.lo);
  else if constexpr (BL == 2) { const uint2 v = lds64(a.lo); f.lo[0] = v.x; f.lo[1] = v.y; }
  else if constexpr (BL == 4) { const uint4 v = lds128(a.lo); f.lo[0] = v.x; f.lo[1] = v.y; f.lo[2] = v.z; f.lo[3] = v.w; }
  else {
    // a.lo is the chunk's 32 bytes, or their upper half for the lanes that read the halves in the
    // opposite order (see the kernel): the other half is always at a.lo ^ 16
    const uint4 v = lds128(a.lo), u = lds128(a.lo ^ 16u);
    f.lo[0] = v.x; f.lo[1] = v.y; f.lo[2] = v.z; f.lo[3] = v.w; f.lo[4] = u.x; f.lo[5] = u.y; f.lo[6] = u.z; f.lo[7] = u.w;
  }
  if constexpr (BH == 1) f.hi[0] = lds32(a.hi);
  if constexpr (BH == 2) { const uint2 v = lds64(a.hi); f.hi[0] = v.x; f.hi[1] = v.y; }
  if constexpr (fi.kind == WK_KQUANT) {
    const uint2 dd = lds64(a.p0);
    f.pr[0] = dd.x; f.pr[1] = dd.y;
    if constexpr (fi.has_min) f.pr[2] = lds32(a.km); else f.pr[2] = lds16(a.km);
  } else if constexpr (fi.kind == WK_CLASSIC || fi.kind == WK_AFFINE) {
    f.pr[0] = lds32(a.p0);
    if constexpr (fi.has_min) f.pr[1] = lds32(a.p1);
  } else if constexpr (fi.pgroup == 16) {
    const uint2 v = lds64(a.p0);
    f.pr[0] = v.x; f.pr[1] = v.y;
  } else {
    f.pr[0] = lds32(a.p0);
  }
}

template <int F, int RT, bool PREFETCH, bool EXT, bool MP = false, bool NORM = false>   // MP: column passes (rows wider than 16384 columns); NORM: RMSNorm of x in the prologue
__global__ void __launch_bounds__(TMA_THREADS, 1)
gemv_tma_kernel(const WvDevBlob b, const uint4* __restrict__ xqg, const float* __restrict__ xf, float* __restrict__ y,
                int row_begin, int row_end, const TmaGeom g, int* __restrict__ err, const typename TmaExtArgs<EXT>::type ext) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_abort;
  __shared__ unsigned s_xissued;   // consumer warps that have issued their loads of x
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // band of this CTA in matrix i, without divisions: the host splits the rows as evenly as possible
  const int bid = blockIdx.x;
  int band, c_lo, c_hi, ntiles;
  auto set_band = [&](int i) {
    int rbase = g.rows_base, rrem = g.rows_rem;
    if constexpr (EXT) { rbase = ext.grp.rows_base[i]; rrem = ext.grp.rows_rem[i]; }
    band = rbase + (bid < rrem ? 1 : 0);
    c_lo = bid * rbase + min(bid, rrem);
    c_hi = c_lo + band;
    ntiles = (band + g.tr - 1) / g.tr;
  };
  int nmat = 1;
  if constexpr (EXT) nmat = ext.grp.n;
  (void)y;
  (void)row_end; (void)xqg;
  const unsigned bar0 = smem_u32(smem + g.bar_off);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (g.nstage + s); };
  const int nactive = g.nrg * g.nwc;  // consumer warps that take part

  if (tid == 0) {
    s_abort = 0;
    s_xissued = 0;
    for (int s = 0; s < g.nstage; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), nactive); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if constexpr (fi.table) {
    // [256 code pairs][32 lanes] of float2 {grid[low nibble], grid[high nibble]}: a plane byte addresses both of its weights
    float2* tbl = reinterpret_cast<float2*>(smem + g.red_off + 2u * g.nrg * g.nwc * 32 * 4);
    for (int i = tid; i < 256 * 32; i += TMA_THREADS) tbl[i] = make_float2(c_grid4nl[(i >> 5) & 15], c_grid4nl[i >> 9]);
  }
  __syncthreads();

  if (warp == TMA_CONSUMER_WARPS) {
    // ------------------------------------------------------------ producer
    // One thread issues the copies; the other lanes of the warp have nothing to do.
    const void* src[5] = {b.lo, b.hi, b.p0, b.p1, b.km};
    bool dead = false;
    int issued = 0;        // tiles issued so far, over all matrices
    int ps = 0;            // stage of the tile being issued
    unsigned ppar = 1;     // parity of the "empty" phase to wait for once the ring has wrapped
    bool wrapped = false;
    int bi = 0;            // matrix being streamed
    int pcp = 0;           // column pass being streamed
    auto issue_tile = [&](int t) {
      const int s = ps;
      if (wrapped) {
        if (*(volatile int*)&s_abort || !mbar_wait(empty_bar(s), ppar)) {
          if (!*(volatile int*)&s_abort) { atomicCAS_system(err, 0, 100 + s); *(volatile int*)&s_abort = 1; }
          dead = true;
          return;
        }
      }
      const int r0 = c_lo + t * g.tr;
      const int nr = min(g.tr, c_hi - r0);
      unsigned bytes = 0;
#pragma unroll
      for (int i = 0; i < 5; i++) bytes += g.rb[i] * nr;
      mbar_expect_tx(full_bar(s), bytes);
      const unsigned dst = smem_u32(smem) + (unsigned)s * g.stage_bytes;
#pragma unroll
      for (int i = 0; i < 5; i++) {
        const void* pl = src[i];
        if constexpr (EXT) pl = ext.grp.plane[bi][i];
        if (!g.rb[i]) continue;
        bulk_g2s(dst + g.off[i], (const unsigned char*)pl + (size_t)(row_begin + r0) * g.rb[i], g.rb[i] * nr, full_bar(s));
      }
      issued++;
      if (++ps == g.nstage) { ps = 0; wrapped = true; ppar ^= 1u; }
    };
    if constexpr (MP) {
      // Column passes: a tile is a slice of each of its rows, fetched by one tensor-map copy per plane (one bulk copy
      // per row and plane measured 40 us at 8192 x 28672, spread over the lanes 54 us: the copy engine pays per copy).
      (void)issue_tile; (void)pcp;
      bool held = false;
      for (int cpass = 0; cpass < g.ncp && !dead; cpass++)
      for (bi = 0; bi < nmat && !dead; bi++) {
        set_band(bi);
        for (int t = 0; t < ntiles && !dead; t++) {
          const int s = ps;
          const int r0 = c_lo + t * g.tr;
          const int nr = min(g.tr, c_hi - r0);
          int ok = 1;
          if (lane == 0) {
            if (!held && issued >= g.lead) {
              held = true;
              for (unsigned i = 0; i < TMA_SPIN_LIMIT; i++) {
                if (*(volatile unsigned*)&s_xissued >= TMA_CONSUMER_WARPS) break;
              }
            }
            if (wrapped && (*(volatile int*)&s_abort || !mbar_wait(empty_bar(s), ppar))) {
              if (!*(volatile int*)&s_abort) { atomicCAS_system(err, 0, 100 + s); *(volatile int*)&s_abort = 1; }
              ok = 0;
            }
            if (ok) {
              // one tensor-map copy per plane brings the tile's row slices in as [row][slice]; the box always has
              // g.tr rows (rows past the matrix are zero-filled and count towards the barrier's bytes)
              unsigned bytes = 0;
#pragma unroll
              for (int i = 0; i < 5; i++) bytes += g.rb[i] * g.tr;
              mbar_expect_tx(full_bar(s), bytes);
              const unsigned dst = smem_u32(smem) + (unsigned)s * g.stage_bytes;
#pragma unroll
              for (int i = 0; i < 5; i++)
                if (g.rb[i]) tma_load_3d(dst + g.off[i], (const unsigned char*)g.maps + 128 * i, 0, cpass * (int)g.nsegp[i], row_begin + r0, full_bar(s));
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { dead = true; break; }
          (void)nr;
          issued++;
          if (++ps == g.nstage) { ps = 0; wrapped = true; ppar ^= 1u; }
        }
      }
      __syncwarp();
      if (lane == 0) {
        for (int t = max(0, issued - g.nstage); t < issued; t++) {
          if (!mbar_wait(full_bar(t % g.nstage), (t / g.nstage) & 1)) { atomicCAS_system(err, 0, 200 + t % g.nstage); break; }
        }
      }
      return;
    }
    if (lane == 0) {
      bool held = false;
      const int npass = 1;
      for (pcp = 0; pcp < npass && !dead; pcp++)
      for (bi = 0; bi < nmat && !dead; bi++) {
        set_band(bi);
        for (int t = 0; t < ntiles && !dead; t++) {
          if (!held && issued >= g.lead) {
            // The activation loads must not queue behind a full ring of weight traffic: after the
            // first tiles, hold further copies until every consumer warp has issued its loads of x
            // (a relaxed counter: a barrier here would wait for the loads to complete).
            held = true;
            for (unsigned i = 0; i < TMA_SPIN_LIMIT; i++) {
              if (*(volatile unsigned*)&s_xissued >= TMA_CONSUMER_WARPS) break;
            }
          }
          issue_tile(t);
        }
      }
      // drain: every copy issued must have landed before the CTA gives its shared memory back
      for (int t = max(0, issued - g.nstage); t < issued; t++) {
        if (!mbar_wait(full_bar(t % g.nstage), (t / g.nstage) & 1)) { atomicCAS_system(err, 0, 200 + t % g.nstage); break; }
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int wc = warp % g.nwc, rg = warp / g.nwc;
  const int c = wc * 32 + lane;
  const bool live = c < g.cpr;

  // RMSNorm fused into the prologue: the norm's weights do not depend on the preceding kernel, so this lane's 32 of
  // them are requested before the wait and are there when x is
  float4 gam[NORM ? 8 : 1];
  if constexpr (NORM) {
    const float4* gp = reinterpret_cast<const float4*>(ext.norm_gamma + (size_t)(live ? c : 0) * 32);
#pragma unroll
    for (int k = 0; k < 8; k++) gam[k] = __ldg(gp + k);
  }
  __shared__ double s_norm[NORM ? TMA_CONSUMER_WARPS : 1];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // All consumer warps copy x into shared memory with coalesced loads; each chunk of 32
  // floats gets a 33-float slot so that lanes reading their own chunks element by element
  // hit 32 different banks. Every CTA starts its copy at a different place of x: all SMs
  // asking for the same lines in the same order would queue up at one L2 slice after the other.
  // With column passes, pass cp brings in its own slice of x (after every warp is done with the previous one).
  const int npass = MP ? g.ncp : 1;
  int cp = 0;
  auto copy_x = [&]() {
    if (cp > 0) asm volatile("bar.sync 15, %0;" ::"n"(TMA_CONSUMER_WARPS * 32) : "memory");
    const float* xrow = xf + (size_t)blockIdx.y * b.cols + (size_t)cp * g.cpr * 32;
    float* xs = reinterpret_cast<float*>(smem + g.x_off);
    const int nv = g.cpr * 8;
    if ((reinterpret_cast<uintptr_t>(xrow) & 15) == 0) {
      // cols <= 16384: at most 8 vectors per thread; all loads are issued before the first
      // store so that the copy costs one memory round trip, not eight
      const int rot = (int)(((unsigned)bid * 211u) % (unsigned)nv) & ~7;   // whole chunks (8 vectors)
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i0 = tid + u * TMA_CONSUMER_WARPS * 32;
        int i = i0 + rot;
        if (i >= nv) i -= nv;
        if (i0 < nv) v[u] = __ldg(reinterpret_cast<const float4*>(xrow) + i);
      }
      if (lane == 0) asm volatile("red.relaxed.cta.shared::cta.add.u32 [%0], 1;" ::"r"(smem_u32(&s_xissued)) : "memory");
      if constexpr (NORM) {
        // Sum of squares (the reference's RMSNorm sums in float64, layers/rmsnorm/cpu.go:76-85): a thread's at most 32
        // squares in float32 (conversions to float64 issue at a sixteenth of the float32 rate), then float64 over the
        // warp and, by every thread after the barrier, over the 16 warp sums in a fixed order. The float32 partial sums
        // are off by a few 1e-7 of their value; the normalised x inherits half of that.
        float sf = 0.f;
#pragma unroll
        for (int u = 0; u < 8; u++) {
          if (tid + u * TMA_CONSUMER_WARPS * 32 < nv) sf += (v[u].x * v[u].x + v[u].y * v[u].y) + (v[u].z * v[u].z + v[u].w * v[u].w);
        }
        double ss = (double)sf;
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_norm[warp] = ss;
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i0 = tid + u * TMA_CONSUMER_WARPS * 32;
        int i = i0 + rot;
        if (i >= nv) i -= nv;
        if (i0 < nv) { float* d = xs + (i >> 3) * 33 + (i & 7) * 4; d[0] = v[u].x; d[1] = v[u].y; d[2] = v[u].z; d[3] = v[u].w; }
      }
    } else {
      if (lane == 0) asm volatile("red.relaxed.cta.shared::cta.add.u32 [%0], 1;" ::"r"(smem_u32(&s_xissued)) : "memory");
      double ss = 0.0;
      for (int i = tid; i < g.cpr * 32; i += TMA_CONSUMER_WARPS * 32) {
        const float xv1 = __ldg(xrow + i);
        xs[(i >> 5) * 33 + (i & 31)] = xv1;
        if constexpr (NORM) ss += (double)xv1 * (double)xv1;
      }
      if constexpr (NORM) {
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_norm[warp] = ss;
      }
    }
    asm volatile("bar.sync 15, %0;" ::"n"(TMA_CONSUMER_WARPS * 32) : "memory");
  };
  if (rg >= g.nrg) {   // warps without a row group only help with the copies
    for (cp = 0; cp < npass; cp++) copy_x();
    return;
  }

  float* red = reinterpret_cast<float*>(smem + g.red_off);
  float* yb = nullptr;
  float keep = 0.f;
  int par = 0;
  bool dead = false;
  int nslots = 0;
  int cur_mat = 0;   // matrix of the group being worked on
  auto flush = [&](int batch_base) {
    float* mine = red + (((size_t)par * g.nrg + rg) * g.nwc + wc) * 32;
    mine[lane] = keep;
    asm volatile("bar.sync %0, %1;" ::"r"(rg + 1), "r"(g.nwc * 32) : "memory");
    if (wc == 0) {
      const float* base = red + ((size_t)par * g.nrg + rg) * g.nwc * 32;
      float sum = 0.f;
      for (int q = 0; q < g.nwc; q++) sum += base[q * 32 + lane];
      const int n = batch_base + lane;
      const int row = c_lo + (n / RT) * g.tr + rg * RT + (n % RT);
      if (n < nslots && (n / RT) * g.tr + rg * RT + (n % RT) < band && rg * RT + (n % RT) < g.tr) {
        if constexpr (EXT) {
          bool skip = false;
          if constexpr (MP) {
            float* sp = reinterpret_cast<float*>(smem + g.part_off) + cur_mat * TMA_GATE_ROWS + (n / RT) * g.tr + rg * RT + (n % RT);
            if (cp > 0) sum += *sp;
            if (cp < g.ncp - 1) { *sp = sum; skip = true; }
          }
          if (!skip && ext.mode == 1) {
            // SwiGLU gate product (simd/silu.go:14-27) in the epilogue: this thread owns the same row of the
            // gate matrix and of the up matrix, so the gate's sum waits in shared memory for the up row
            float* sg = reinterpret_cast<float*>(smem + g.gate_off);
            const int rib = (n / RT) * g.tr + rg * RT + (n % RT);
            if (cur_mat == 0) { sg[rib] = sum; skip = true; }
            else { const double gt = (double)sg[rib]; sum = (float)(gt / (1.0 + exp(-gt)) * (double)sum); }
          }
          if (!skip) {
            if (ext.residual) sum += ext.residual[(size_t)blockIdx.y * ext.grp.rows[cur_mat] + row_begin + row];
            if (ext.npeers) {
              for (int q = 0; q < ext.npeers; q++) ext.py[cur_mat][q][row_begin + row] = sum;   // own and peers' copies of y
            } else {
              yb[row] = sum;
            }
          }
        } else {
          yb[row] = sum;
        }
      }
    }
    par ^= 1;
    keep = 0.f;
  };

  const unsigned sbase = smem_u32(smem);
  LaneOff lo0 = lane_offsets<F>(g, rg * RT, live ? c : g.cpr - 1, b.group);
  if constexpr (BL == 8) {
    // 8-bit codes: a lane's chunk is 32 bytes, so the 16-byte loads of lanes i and i+4 of a quarter
    // warp would fall into the same banks. Every second group of four lanes reads the two halves
    // in the opposite order and keeps its activation words swapped to match.
    if (lane & 4) lo0.lo ^= 16u;
  }
  // Fetch the fragments of tile t from the ring into registers, then hand the stage back.
  // stage index and phase parity of the tile being fetched, advanced incrementally (no divisions
  // in the loop)
  int fs = 0;
  unsigned fpar = 0;
  auto wait_tile = [&](bool block) -> bool {
    if (dead || *(volatile int*)&s_abort) { dead = true; return true; }
    if (!block) {
      unsigned ok;
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(ok) : "r"(full_bar(fs)), "r"(fpar) : "memory");
      return __all_sync(0xffffffffu, ok != 0);
    }
    if (!mbar_wait(full_bar(fs), fpar)) {
      atomicCAS_system(err, 0, 300 + fs); *(volatile int*)&s_abort = 1; dead = true;
    }
    return true;
  };
  auto fetch_tile = [&](FragT<F> (&fr)[RT]) {
    LaneOff a = lo0;
    const unsigned st = sbase + (unsigned)fs * g.stage_bytes;
    a.lo += st; a.hi += st; a.p0 += st; a.p1 += st; a.km += st;
#pragma unroll
    for (int rr = 0; rr < RT; rr++) {
      load_frag_smem<F>(fr[rr], a);   // unconditional: rows past the band read stale ring data and are never stored
      a.lo += g.rb[0]; a.hi += g.rb[1]; a.p0 += g.rb[2]; a.p1 += g.rb[3]; a.km += g.rb[4];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(fs));  // the fragments are in registers: hand the stage back
    if (++fs == g.nstage) { fs = 0; fpar ^= 1u; }
  };

  // The main loop, instantiated once per activation record type: `dot(fragment)` is the chunk-row's
  // share of its output row.
  auto main_loop = [&](auto dot) {
    for (int bi = 0; bi < nmat; bi++) {   // one matrix after the other; ring position and x registers carry over
      set_band(bi);
      cur_mat = bi;
      nslots = ntiles * RT;
      if constexpr (EXT) yb = ext.grp.y[bi] + (size_t)blockIdx.y * ext.grp.rows[bi] + row_begin;
      else yb = y + (size_t)blockIdx.y * b.rows + row_begin;
      FragT<F> nxt[PREFETCH ? RT : 1];
      if constexpr (PREFETCH) { if (ntiles > 0) { wait_tile(true); fetch_tile(nxt); } }
      for (int t = 0; t < ntiles; t++) {
        FragT<F> fr[RT];
        bool fetched = true;
        if constexpr (PREFETCH) {
#pragma unroll
          for (int rr = 0; rr < RT; rr++) fr[rr] = nxt[rr];
          // prefetch the next tile's fragments before computing when they have already landed
          if (t + 1 < ntiles) {
            fetched = wait_tile(false);
            if (fetched) fetch_tile(nxt);
          }
        } else {
          wait_tile(true);
          fetch_tile(fr);
        }
        float v[RT];
        // No per-row branch: the RT chunk-rows form one block of independent dependency chains.
        // Lanes past the last chunk hold zeroed activations and contribute exactly 0.
#pragma unroll
        for (int rr = 0; rr < RT; rr++) v[rr] = dot(fr[rr]);
        // Transposing reduction: RT row sums per lane -> every lane ends with the warp total of one
        // row; the lane whose index equals the row's slot (n & 31) keeps it.
        float tot;
        if constexpr (RT == 4) {
          const bool b4 = lane & 16, b3 = lane & 8;
          float a0 = b4 ? v[2] : v[0], a1 = b4 ? v[3] : v[1];
          a0 += __shfl_xor_sync(0xffffffffu, b4 ? v[0] : v[2], 16);
          a1 += __shfl_xor_sync(0xffffffffu, b4 ? v[1] : v[3], 16);
          tot = b3 ? a1 : a0;
          tot += __shfl_xor_sync(0xffffffffu, b3 ? a0 : a1, 8);
#pragma unroll
          for (int o = 4; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
          tot = __shfl_sync(0xffffffffu, tot, (lane & 3) * 8);  // row (lane & 3) lives in lanes [8*(lane&3), +8)
          if ((lane >> 2) == (t & 7)) keep = tot;
        } else if constexpr (RT == 8) {
          const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
          float a[4];
#pragma unroll
          for (int i = 0; i < 4; i++) a[i] = (b4 ? v[4 + i] : v[i]) + __shfl_xor_sync(0xffffffffu, b4 ? v[i] : v[4 + i], 16);
          float c0 = (b3 ? a[2] : a[0]) + __shfl_xor_sync(0xffffffffu, b3 ? a[0] : a[2], 8);
          float c1 = (b3 ? a[3] : a[1]) + __shfl_xor_sync(0xffffffffu, b3 ? a[1] : a[3], 8);
          tot = (b2 ? c1 : c0) + __shfl_xor_sync(0xffffffffu, b2 ? c0 : c1, 4);
          tot += __shfl_xor_sync(0xffffffffu, tot, 2);
          tot += __shfl_xor_sync(0xffffffffu, tot, 1);
          // row r = 4*b4 + 2*b3 + b2 lives in lanes [4r, 4r+4): lane wants row (lane & 7)
          tot = __shfl_sync(0xffffffffu, tot, ((lane & 4) ? 16 : 0) + ((lane & 2) ? 8 : 0) + ((lane & 1) ? 4 : 0));
          if ((lane >> 3) == (t & 3)) keep = tot;
        } else if constexpr (RT == 2) {
          const bool b4 = lane & 16;
          tot = b4 ? v[1] : v[0];
          tot += __shfl_xor_sync(0xffffffffu, b4 ? v[0] : v[1], 16);
#pragma unroll
          for (int o = 8; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
          tot = __shfl_sync(0xffffffffu, tot, (lane & 1) * 16);
          if ((lane >> 1) == (t & 15)) keep = tot;
        } else {
          tot = v[0];
#pragma unroll
          for (int o = 16; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
          if (lane == (t & 31)) keep = tot;
        }
        if (((t * RT + RT - 1) & 31) == 31) flush(t * RT + RT - 32);
        if constexpr (PREFETCH) { if (!fetched) { wait_tile(true); fetch_tile(nxt); } }
      }
      if (nslots & 31) flush(nslots & ~31);
    }
  };

  const float* xc = reinterpret_cast<const float*>(smem + g.x_off) + (size_t)(live ? c : 0) * 33;
  for (cp = 0; cp < npass; cp++) {
  copy_x();
  if constexpr (NORM) {
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < TMA_CONSUMER_WARPS; w++) t += s_norm[w];
    const float inv = 1.0f / sqrtf((float)(t / (double)b.cols + ext.norm_eps));
    // every chunk is normalised in place by the one lane of row group 0 that owns it; the other row groups' warps
    // read it after the barrier (all warps that have a row group take part; the others have left)
    if (rg == 0 && live) {
      float* xw = reinterpret_cast<float*>(smem + g.x_off) + (size_t)c * 33;
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const float gq[4] = {gam[k].x, gam[k].y, gam[k].z, gam[k].w};
#pragma unroll
        for (int m = 0; m < 4; m++) xw[4 * k + m] = (xw[4 * k + m] * inv) * gq[m];
      }
    }
    asm volatile("bar.sync 14, %0;" ::"r"(nactive * 32) : "memory");
  }
  if constexpr (fi.table) {
    // IQ4_NL: f32 grid values from a shared-memory table, activations stay f32. xfr[2w + h] holds, for bytes 2h and
    // 2h + 1 of plane word w, the activations of the byte's low-nibble and high-nibble weight.
    const unsigned char* tbl = smem + g.red_off + 2u * g.nrg * g.nwc * 32 * 4;
    float4 xfr[8];
#pragma unroll
    for (int k = 0; k < 8; k++) xfr[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
#pragma unroll
      for (int w = 0; w < 4; w++)
#pragma unroll
        for (int h = 0; h < 2; h++)
          xfr[2 * w + h] = make_float4(xc[WvLane<BL>::j_of(2 * w, 2 * h)], xc[WvLane<BL>::j_of(2 * w + 1, 2 * h)],
                                       xc[WvLane<BL>::j_of(2 * w, 2 * h + 1)], xc[WvLane<BL>::j_of(2 * w + 1, 2 * h + 1)]);
    }
    const unsigned lane4 = (unsigned)lane * 8u;
    main_loop([&](const FragT<F>& f) { return chunk_value_tbl<F>(f, xfr, tbl, lane4); });
  } else {
    // Statistics of x that decide the width of the activation records, per warp, i.e. per 1024 columns (a warp's
    // chunks are the same columns on every CTA and every row shard, so all of them reach the same decision):
    // A = sum over the warp's chunks of the chunk's largest magnitude, S = sum |x_j| over the same columns.
    // With 16-bit records an element is off by at most amax_chunk / 65024, so these columns' share of a row's error
    // is at most sum_chunks amax_c / 65024 * sum_{j in c} |w_j|, about w_mean * 4.9e-4 * A for weights that are not
    // concentrated on a chunk's small elements, against a budget of 1e-3 * w_mean * S. A <= S / 4 keeps an eightfold
    // margin (N(0,1) data: A / S = 0.09); columns with isolated outliers, inf or NaN fail the test and take 24-bit
    // records, whose error is 2^-9 of that. Weights that sit exactly on the small elements of outlier chunks can
    // exceed either bound: no criterion on x alone excludes that.
    float xv[32];
#pragma unroll
    for (int j = 0; j < 32; j++) xv[j] = xc[j];
    float am[4] = {0.f, 0.f, 0.f, 0.f}, as[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 32; j++) { const float a = fabsf(xv[j]); am[j & 3] = fmaxf(am[j & 3], a); as[j & 3] += a; }
    float amax = fmaxf(fmaxf(am[0], am[1]), fmaxf(am[2], am[3]));
    float asum = (as[0] + as[1]) + (as[2] + as[3]);   // inf / NaN anywhere in the chunk makes this inf / NaN
    if (!live) { amax = 0.f; asum = 0.f; }
    float ta = amax, ts = asum;
#pragma unroll
    for (int o = 16; o; o >>= 1) { ta += __shfl_xor_sync(0xffffffffu, ta, o); ts += __shfl_xor_sync(0xffffffffu, ts, o); }
    const bool wide = !(ta <= 0.25f * ts) || g.force3;   // NaN compares false: non-finite input takes the wide path
    if (!wide) {
      XQRegs2 xr;
      if (live) {
        quantize_chunk2<F>(xr, xv, amax, false);
        if constexpr (BL == 8) {
          const bool sw = lane & 4;
#pragma unroll
          for (int l = 0; l < 2; l++) {
#pragma unroll
            for (int k = 0; k < 4; k++) {
              const unsigned a0 = xr.xw[8 * l + k], a1 = xr.xw[8 * l + k + 4];
              xr.xw[8 * l + k] = sw ? a1 : a0;
              xr.xw[8 * l + k + 4] = sw ? a0 : a1;
            }
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < 16; t++) xr.xw[t] = 0u;
        xr.mt = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; i++) xr.iv[i] = 0;
      }
      main_loop([&](const FragT<F>& f) { return idot_chunk2<F>(f, xr); });
    } else {
      XQRegs xr;
      if (live) {
        quantize_chunk<F>(xr, xc);
        if constexpr (BL == 8) {
          const bool sw = lane & 4;
#pragma unroll
          for (int l = 0; l < 3; l++) {
#pragma unroll
            for (int k = 0; k < 4; k++) {
              const unsigned a0 = xr.xw[8 * l + k], a1 = xr.xw[8 * l + k + 4];
              xr.xw[8 * l + k] = sw ? a1 : a0;
              xr.xw[8 * l + k + 4] = sw ? a0 : a1;
            }
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < 24; t++) xr.xw[t] = 0u;
        xr.mt = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 6; i++) xr.iv[i] = 0;
      }
      main_loop([&](const FragT<F>& f) { return idot_chunk<F>(f, xr); });
    }
  }
  }
}

// ------------------------------------------------------------------ host side
static unsigned align128(unsigned v) { return (v + 127u) & ~127u; }

// Bytes per row of each plane in the device layout; false when a plane's rows are not
// 16-byte multiples (then consecutive rows cannot be fetched by bulk copies).
static bool plane_row_bytes(const WvDevBlob& b, unsigned rb[5]) {
  const WvFmtInfo fi = wv_fmt_info(b.format);
  const unsigned cpr = (unsigned)(b.cols >> 5);
  rb[0] = cpr * fi.bits_lo * 4; rb[1] = cpr * fi.bits_hi * 4; rb[2] = rb[3] = rb[4] = 0;
  switch (fi.kind) {
  case WK_CLASSIC: rb[2] = cpr * 4; rb[3] = fi.has_min ? cpr * 4 : 0; break;
  case WK_KQUANT: if (cpr % 8) return false; rb[2] = cpr; rb[4] = cpr * (fi.has_min ? 4 : 2); break;
  case WK_IQ: case WK_TERNARY: rb[2] = cpr * (fi.pgroup == 16 ? 8 : 4); break;
  case WK_BINARY: if ((b.cols % b.group) || (b.group % 32)) return false; rb[2] = (unsigned)(b.cols / b.group) * 4; break;
  case WK_AFFINE: if ((b.cols % b.group) || (b.group % 32)) return false; rb[2] = rb[3] = (unsigned)(b.cols / b.group) * 4; break;
  default: return false;
  }
  for (int i = 0; i < 5; i++) if (rb[i] % 16) return false;
  return true;
}

static int g_tma_rt = 0, g_tma_stages = 0;
#ifdef WV_DEV_HOOKS
extern "C" void wv_set_tma_tuning(int rows_per_group, int stages) { g_tma_rt = rows_per_group; g_tma_stages = stages; }
#endif
int wv_tma_tuning_stages() { return g_tma_stages; }
int wv_tma_tuning_rt() { return g_tma_rt; }
static int g_act_width = 0;
#ifdef WV_DEV_HOOKS
extern "C" void wv_set_act_width(int limbs) { g_act_width = limbs; }
#endif
int wv_act_width() { return g_act_width; }
int wv_tc_prequant() { return g_tma_rt == 31 ? 1 : 0; }

// Tensor maps for the column passes, five per matrix (one per plane), encoded once and kept in device memory: plane i is
// seen as {box bytes, pieces of a row, rows} with a row `pitch` bytes long; a box of {box bytes, pieces per slice, tile
// rows} is one pass's slice of a tile's rows and lands in shared memory as [row][slice]. Returns null when the driver
// entry point or memory is missing.
struct PassMaps { CUtensorMap m[5]; };
static std::mutex g_pm_mu;
static std::map<std::tuple<std::array<const void*, 5>, std::array<unsigned, 5>, unsigned, int, int>, std::pair<const void*, std::array<unsigned, 5>>> g_pass_maps;
static const void* pass_maps(const void* const planes[5], const unsigned pitch[5], const unsigned rb[5], int rows, int tr, unsigned nsegp[5]) {
  std::lock_guard<std::mutex> lk(g_pm_mu);
  // every plane's address and pitch is part of the key: a later blob may reuse one plane's address but not all five
  const auto key = std::make_tuple(std::array<const void*, 5>{planes[0], planes[1], planes[2], planes[3], planes[4]},
                                   std::array<unsigned, 5>{pitch[0], pitch[1], pitch[2], pitch[3], pitch[4]}, rb[0], rows, tr);
  auto it = g_pass_maps.find(key);
  if (it != g_pass_maps.end()) { for (int i = 0; i < 5; i++) nsegp[i] = it->second.second[i]; return it->second.first; }
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) { cudaGetLastError(); return nullptr; }
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  PassMaps host{};
  std::array<unsigned, 5> nseg{};
  for (int i = 0; i < 5; i++) {
    if (!rb[i]) continue;
    unsigned inner = 256;
    while (inner >= 16 && rb[i] % inner) inner -= 16;
    if (inner < 16 || rb[i] / inner > 256 || tr > 256) return nullptr;
    nseg[i] = rb[i] / inner;
    cuuint64_t dims[3] = {inner, (cuuint64_t)(pitch[i] / inner), (cuuint64_t)rows};
    cuuint64_t strides[2] = {inner, pitch[i]};
    cuuint32_t box[3] = {inner, nseg[i], (cuuint32_t)tr};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&host.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(planes[i]), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return nullptr;
  }
  void* dev = nullptr;
  if (cudaMalloc(&dev, sizeof(PassMaps)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  if (cudaMemcpy(dev, &host, sizeof(PassMaps), cudaMemcpyHostToDevice) != cudaSuccess) { cudaGetLastError(); cudaFree(dev); return nullptr; }
  g_pass_maps[key] = {dev, nseg};
  for (int i = 0; i < 5; i++) nsegp[i] = nseg[i];
  return dev;
}

template <int F, int RT, bool PF>
static int launch_tma(const WvDevBlob* bl, int nb, const float* dx, float* const* dys, int batch, int rb_, int re, cudaStream_t st) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  const WvDevBlob& b = bl[0];   // the matrices of a group agree in everything but their row count
  TmaGeom g{};
  if (!plane_row_bytes(b, g.pitch)) return 1;
  const int cpr_row = b.cols >> 5;
  // rows wider than the consumer warps cover go through in column passes of equal width (whole super-blocks)
  g.ncp = 1;
  while ((cpr_row + g.ncp - 1) / g.ncp > TMA_CONSUMER_WARPS * 32) g.ncp++;
  if (g.ncp > 1 && (cpr_row % (g.ncp * 8) || g.ncp > 8)) return 1;
  g.cpr = cpr_row / g.ncp;
  for (int i = 0; i < 5; i++) {
    g.rb[i] = g.pitch[i] / g.ncp;
    if (g.pitch[i] % g.ncp || g.rb[i] % 16) return 1;
  }
  g.nwc = (g.cpr + 31) / 32;
  if (g.nwc > TMA_CONSUMER_WARPS) return 1;
  g.nrg = TMA_CONSUMER_WARPS / g.nwc;
  if (g.nrg > TMA_MAX_ROW_GROUPS) g.nrg = TMA_MAX_ROW_GROUPS;
  g.tr = g.nrg * RT;
  unsigned off = 0;
  for (int i = 0; i < 5; i++) { g.off[i] = off; off = align128(off + g.rb[i] * g.tr); }
  g.stage_bytes = off;
  const unsigned xbytes = align128((unsigned)g.cpr * 132u);
  const WvFuse* fuse = wv_cur_fuse;
  const bool gated = fuse && fuse->mode == 1;
  const unsigned gate_bytes = gated ? TMA_GATE_ROWS * 4u : 0u;
  const unsigned part_bytes = g.ncp > 1 ? (unsigned)nb * TMA_GATE_ROWS * 4u : 0u;
  const unsigned fixed = xbytes + align128(2u * g.nrg * g.nwc * 32 * 4 + (fi.table ? 65536u : 0u)) + gate_bytes + part_bytes + 2 * TMA_MAX_STAGES * 8 + 128;
  const unsigned avail = 225u * 1024u;  // 227 KB per CTA minus static shared memory and slack
  if (g.stage_bytes * 2 + fixed > avail) return 1;
  int ns = (int)((avail - fixed) / g.stage_bytes);
  if (ns > TMA_MAX_STAGES) ns = TMA_MAX_STAGES;
  if (g_tma_stages % 100 > 1 && g_tma_stages % 100 < ns) ns = g_tma_stages % 100;
  g.lead = g_tma_stages >= 100 ? g_tma_stages / 100 : 1;
  g.force3 = g_act_width == 3;
  g.nstage = ns;
  g.x_off = g.stage_bytes * ns;
  g.red_off = g.x_off + xbytes;
  g.gate_off = align128(g.red_off + 2u * g.nrg * g.nwc * 32 * 4 + (fi.table ? 65536u : 0u));
  g.part_off = g.gate_off + gate_bytes;
  g.bar_off = g.part_off + part_bytes;
  const size_t smem = g.bar_off + 2 * TMA_MAX_STAGES * 8;

  int grid = wv_sm_count();
  if (nb == 1 && grid > re - rb_) grid = re - rb_;
  g.rows_base = (re - rb_) / grid;
  g.rows_rem = (re - rb_) % grid;
  const uint4* xq = nullptr;  // activations are quantised inside the kernel
  int dev = 0; cudaGetDevice(&dev);
  cudaError_t e;
  if (gated) {
    if (nb != 2 || bl[0].rows != bl[1].rows || batch != 1) return WV_ESHAPE;
    if (bl[0].rows / grid + 1 > TMA_GATE_ROWS) return 1;
  }
  if (g.ncp > 1) {
    // the partial sums of a CTA's band wait in shared memory between the passes
    if (nb != 1) return 1;
    if ((re - rb_) / grid + 1 > TMA_GATE_ROWS) return 1;
    const void* planes[5] = {b.lo, b.hi, b.p0, b.p1, b.km};
    g.maps = pass_maps(planes, g.pitch, g.rb, b.rows, g.tr, g.nsegp);
    if (!g.maps) return 1;
  }
  if (nb == 1 && !wv_cur_peers && !fuse && g.ncp == 1) {
    auto kern = gemv_tma_kernel<F, RT, PF, false>;
    static unsigned attr_mask = 0;
    if (!(attr_mask & (1u << dev))) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) { wv_set_error("gemv (tma): cannot raise the shared-memory limit"); return WV_ECUDA; }
      attr_mask |= 1u << dev;
    }
    e = launch_pdl(kern, dim3(grid, batch), dim3(TMA_THREADS), smem, st, b, xq, dx, dys[0], rb_, re, g, g_err_dev, TmaNoExt{});
  } else {
    if constexpr (RT == 4 && !PF) {   // the grouped / peer-storing variant exists for the default configuration only
      const bool norm = fuse && fuse->norm_gamma;
      if (norm && g.ncp > 1) return WV_ESHAPE;      // the fused norm needs the whole row of x at once
      const int variant = g.ncp > 1 ? 1 : (norm ? 2 : 0);
      auto kern = variant == 1 ? gemv_tma_kernel<F, RT, PF, true, true, false>
                : variant == 2 ? gemv_tma_kernel<F, RT, PF, true, false, true> : gemv_tma_kernel<F, RT, PF, true, false, false>;
      static unsigned attr_mask[3] = {0, 0, 0};
      if (!(attr_mask[variant] & (1u << dev))) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) { wv_set_error("gemv (tma): cannot raise the shared-memory limit"); return WV_ECUDA; }
        attr_mask[variant] |= 1u << dev;
      }
      TmaExt ext{};
      ext.grp.n = nb;
      for (int i = 0; i < nb; i++) {
        const int nrows = nb == 1 ? re - rb_ : bl[i].rows;
        ext.grp.rows[i] = bl[i].rows;
        ext.grp.rows_base[i] = nrows / grid;
        ext.grp.rows_rem[i] = nrows % grid;
        ext.grp.plane[i][0] = bl[i].lo; ext.grp.plane[i][1] = bl[i].hi; ext.grp.plane[i][2] = bl[i].p0; ext.grp.plane[i][3] = bl[i].p1; ext.grp.plane[i][4] = bl[i].km;
        ext.grp.y[i] = dys[i];
      }
      if (wv_cur_peers) {
        if (batch != 1 || nb != 1) return WV_ESHAPE;
        ext.npeers = wv_cur_peers->n;
        for (int q = 0; q < ext.npeers; q++) ext.py[0][q] = wv_cur_peers->y[q];
      }
      if (fuse) {
        ext.mode = fuse->mode;
        ext.residual = fuse->residual;
        ext.norm_gamma = fuse->norm_gamma;
        ext.norm_eps = fuse->norm_eps;
        if (fuse->residual && nb != 1) return WV_ESHAPE;
        if (fuse->npeers) {
          if (batch != 1) return WV_ESHAPE;
          ext.npeers = fuse->npeers;
          for (int i = 0; i < nb; i++) for (int q = 0; q < ext.npeers; q++) ext.py[i][q] = fuse->py[i][q];
        }
      }
      e = launch_pdl(kern, dim3(grid, batch), dim3(TMA_THREADS), smem, st, b, xq, dx, dys[0], rb_, re, g, g_err_dev, ext);
    } else {
      return 1;
    }
  }
  if (e != cudaSuccess) { wv_set_error("gemv (tma) launch: %s", cudaGetErrorString(e)); return WV_ECUDA; }
  return WV_OK;
}

template <int F>
static int launch_tma_format(const WvDevBlob* b, int nb, const float* dx, float* const* dy, int batch, int rb, int re, cudaStream_t st) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  // tuning codes: 1, 2, 4 = rows per group with register prefetch of the next tile; 11, 12, 14, 8 = without
  // measured best everywhere: four rows per group, fragments fetched right before use (a second
  // fragment set in registers costs more in register pressure than it hides in latency)
  int rt = (g_tma_rt && g_tma_rt < 20) ? g_tma_rt : 14;
  switch (rt) {
  case 1: return launch_tma<F, 1, true>(b, nb, dx, dy, batch, rb, re, st);
  case 2: return launch_tma<F, 2, true>(b, nb, dx, dy, batch, rb, re, st);
  case 12: return launch_tma<F, 2, false>(b, nb, dx, dy, batch, rb, re, st);
  case 8: if constexpr (fi.bits_lo < 8) return launch_tma<F, 8, false>(b, nb, dx, dy, batch, rb, re, st); break;
  }
  if (rt == 4) return launch_tma<F, 4, true>(b, nb, dx, dy, batch, rb, re, st);
  return launch_tma<F, 4, false>(b, nb, dx, dy, batch, rb, re, st);
}

int wv_launch_gemv_tma(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st) {
  // Formats with one parameter group per chunk: rows of at most 4096 columns go to the tensor-pipe
  // kernel (one column segment per 16-row block; measured 3-10 % faster there, level or slower on
  // wider rows and for IQ3_XXS). Tuning codes 21, 22, 24 force it with that many chunk pairs per
  // warp; any other non-zero code keeps everything on the dp4a kernel.
  if (wv_cur_fuse) {   // fused epilogues live in the grouped instance of the dp4a kernel
    float* dys1[1] = {dy};
    return wv_launch_gemv_tma_group(&b, 1, dx, dys1, batch, row_begin, row_end, st);
  }
  // Tuning code 30 routes everything the tensor-pipe kernel of wv_gemv_tc.cu serves through it.
  if (g_tma_rt == 30 || g_tma_rt == 31) {
    const int rc = wv_launch_gemv_tc(b, dx, dy, batch, row_begin, row_end, st);
    if (rc != 1) return rc;
  }
  if ((g_tma_rt >= 20 && g_tma_rt < 30) || ((g_tma_rt == 0 || g_tma_rt >= 30) && b.cols <= 4096 && b.format != WV_IQ3_XXS)) {
    const int rc = wv_launch_gemv_mma(b, dx, dy, batch, row_begin, row_end, st, (g_tma_rt >= 20 && g_tma_rt < 30) ? g_tma_rt - 20 : 4);
    if (rc != 1) return rc;
  } else if (g_tma_rt == 0 && b.format == WV_Q8_0) {
    // 8-bit codes need no unpacking, so the tensor-pipe kernel also wins on wider rows (two chunk pairs per warp
    // and tile: 12.2 vs 12.6 us at 4096x14336); shapes it does not serve come back with 1
    const int rc = wv_launch_gemv_mma(b, dx, dy, batch, row_begin, row_end, st, 2);
    if (rc != 1) return rc;
  }
  float* dys[1] = {dy};
  return wv_launch_gemv_tma_group(&b, 1, dx, dys, batch, row_begin, row_end, st);
}

// Several matrices of one format, column count and group that share x (Q|K|V, gate|up) in one
// launch: the prologue (wait for the preceding kernel, bring x in, quantise it) is paid once.
// Returns 1 when the group cannot run as one launch of this kernel.
int wv_launch_gemv_tma_group(const WvDevBlob* b, int nb, const float* dx, float* const* dy, int batch, int row_begin, int row_end,
                             cudaStream_t st) {
  if (nb < 1 || nb > TMA_MAX_GROUP) return 1;
  for (int i = 1; i < nb; i++)
    if (b[i].format != b[0].format || b[i].cols != b[0].cols || b[i].group != b[0].group || b[i].dtype != b[0].dtype || !b[i].fast) return 1;
  switch (b[0].format) {
#define WV_F(f) case f: return launch_tma_format<f>(b, nb, dx, dy, batch, row_begin, row_end, st);
  WV_F(WV_Q8_0) WV_F(WV_Q4_0) WV_F(WV_Q4_1) WV_F(WV_Q5_0) WV_F(WV_Q5_1)
  WV_F(WV_Q2_K) WV_F(WV_Q3_K) WV_F(WV_Q4_K) WV_F(WV_Q5_K) WV_F(WV_Q6_K)
  WV_F(WV_IQ1_S) WV_F(WV_IQ2_XXS) WV_F(WV_IQ2_XS) WV_F(WV_IQ3_XXS) WV_F(WV_IQ3_S) WV_F(WV_IQ4_NL) WV_F(WV_IQ4_XS)
  WV_F(WV_TERNARY) WV_F(WV_BINARY) WV_F(WV_AFFINE)
#undef WV_F
  }
  return 1;
}

// Code of the first bounded device wait that ran out (0 = none); reading clears it.
int wv_tma_take_error() {
  if (!g_err_host) return 0;
  const int v = *(volatile int*)g_err_host;
  if (v) *(volatile int*)g_err_host = 0;
  return v;
}
int* wv_tma_err_ptr() { return g_err_dev; }
int wv_tma_init() {
  if (g_err_host) return WV_OK;
  if (cudaHostAlloc(&g_err_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) { cudaGetLastError(); return WV_ENOMEM; }
  *g_err_host = 0;
  if (cudaHostGetDevicePointer(&g_err_dev, g_err_host, 0) != cudaSuccess) { cudaGetLastError(); return WV_ECUDA; }
  return WV_OK;
}
