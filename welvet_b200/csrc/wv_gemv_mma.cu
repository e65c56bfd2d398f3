// GEMV for the formats with one parameter group per 32 weights (or wider), with the dot
// products on the tensor pipe: the integer pipe of an SM issues dp4a at half rate, and at three
// activation limbs per weight it is what bounds the dp4a kernel; mma.sync m16n8k32 (u8 x u8 ->
// s32) does the same sums for 16 rows x 32 columns x 8 operand columns in one instruction.
//
//   * A operand = 16 rows x one 32-column chunk of unsigned codes, unpacked from the bit planes by
//     the lane that holds that fragment (one 32-bit word of the lo plane per row per lane);
//   * B operand = the chunk's activations as block fixed point X' = rint(x 2^(22-e)) + 2^22 in
//     [0, 2^23], split into three unsigned byte digits (columns 0..2) plus a column of ones
//     (column 3), so that  sum code*X = n0 + 256 n1 + 65536 n2 - 2^22 n3  exactly;
//   * two chunks are chained into one accumulator: the second chunk's digits sit in columns 4..7,
//     so all four lanes of a quad end up with useful sums (chunk A/B x low/high digits) and the
//     scale is applied once per pair of instructions;
//   * symmetric formats start the accumulator at -mid * (digit sums), which keeps all-zero
//     weights at exactly 0;
//   * the planes of a tile (16 rows x one column segment) are fetched by one tensor-map copy per
//     plane (cp.async.bulk.tensor, 128-byte swizzle) into a shared-memory ring (full / empty
//     mbarriers, bounded waits). Each plane is described as {128 bytes, rows, 128-byte pieces of
//     a row}, so a tile lands as [piece][row][128 B] and the swizzle spreads the eight rows a
//     warp reads together over different banks. Rows and pieces past the end are zero-filled
//     by the copy engine, which is what makes ragged last segments and row blocks harmless.
//
// Every warp owns a fixed set of chunk pairs in each segment and keeps two row sums per lane
// (rows g and g+8 of the 16-row block); the sums are reduced over the quad and then across the
// warps through shared memory once per 16 rows.
#include "wv_gemv_common.cuh"
#include "wv_tma_common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>

#define MMA_WARPS 16
#define MMA_THREADS ((MMA_WARPS + 1) * 32)
#define MMA_MAX_STAGES 8
#define MMA_SLOT 144u       // bytes per chunk slot: 96 digits, 16 accumulator start, 16 meta, 16 of padding (bank spread)
#define MMA_SLOT_K 96u
#define MMA_SLOT_META 112u


struct MmaGeom {
  int cpr;              // chunks per row
  int nseg;             // column segments per 16-row block
  int seg_chunks;       // chunks per segment (32 * PW)
  int gsh;              // log2(chunks per parameter group)
  int nstage;
  unsigned stage_bytes;
  unsigned off[4];      // lo, hi, p0, p1 offsets inside a stage (multiples of 2048)
  unsigned np[4];       // 128-byte pieces per row segment of each plane (0 = plane absent)
  unsigned tx_bytes;    // bytes one tile brings in
  int mt_base, mt_rem;  // CTA b owns mt_base (+1 if b < mt_rem) blocks of 16 rows
  int nrows;
  int lead;             // tiles issued before the producer waits for the activation loads to be on their way
  unsigned x_off, const_off, red_off, bar_off;
  unsigned ysm_off;     // peer-storing variant: the band's row sums wait here until the main loop is over
};

__device__ __forceinline__ void mma_u8u8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8u8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void sts128(unsigned a, unsigned x, unsigned y, unsigned z, unsigned w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

template <int F> struct MmaCfg {
  static constexpr WvFmtInfo fi = wv_fmt_info(F);
  // Q4_0 / Q8_0 store code ^ mid, i.e. the reference's own two's-complement code with the top bit
  // flipped: flipping it back yields the signed code (times 16 for the nibbles, which sit in the
  // high half of their byte), so these formats multiply signed codes and need no -mid start value.
  static constexpr bool SIGNED_A = F == WV_Q4_0 || F == WV_Q8_0;
  static constexpr float A_SCALE = F == WV_Q4_0 ? 1.0f / 16.0f : 1.0f;
  static constexpr bool INT_MID = fi.mid != 0 && !fi.half_mid && !SIGNED_A;
  static constexpr bool USES_SX = fi.has_min || fi.sign || fi.half_mid;
  static constexpr bool OK = !fi.table && fi.pgroup != 16 && fi.kind != WK_KQUANT && fi.kind != WK_TERNARY &&
                             fi.kind != WK_NONE && fi.bits_hi <= 1;
};

// One thread turns the 32 activations of its slot into the chunk's B-operand digits, the
// accumulator start values and the scale factors, in place (slots are 144 bytes apart, so the
// 16-byte accesses of neighbouring threads fall into different banks).
template <int F>
__device__ __forceinline__ void mma_quantize_slot(unsigned slot) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo;
  float xv[32];
#pragma unroll
  for (int q = 0; q < 8; q++) {
    const uint4 v = lds128(slot + 16u * q);
    xv[4 * q] = __uint_as_float(v.x); xv[4 * q + 1] = __uint_as_float(v.y); xv[4 * q + 2] = __uint_as_float(v.z); xv[4 * q + 3] = __uint_as_float(v.w);
  }
  float am[4] = {0.f, 0.f, 0.f, 0.f}, pr[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 32; j++) { am[j & 3] = fmaxf(am[j & 3], fabsf(xv[j])); pr[j & 3] = fmaf(xv[j], 0.f, pr[j & 3]); }  // pr: NaN iff any inf / NaN
  const float amax = fmaxf(fmaxf(am[0], am[1]), fmaxf(am[2], am[3]));
  const float probe = (pr[0] + pr[1]) + (pr[2] + pr[3]);
  const unsigned eb = (__float_as_uint(amax) >> 23) & 0xffu;
  float sf = 0.f, inv = 0.f;
  if (probe != 0.f || eb == 255u) sf = __uint_as_float(0x7fc00000u);  // inf / NaN in x: the row sums become NaN
  else if (eb >= 22u) { sf = __uint_as_float((eb - 21u) << 23); inv = __uint_as_float((275u - eb) << 23); }
  unsigned D[3][8];
  int sl[3] = {0, 0, 0};
  float fsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int k = 0; k < 8; k++) {
    unsigned X[4];
    // the low 23 bits of 1.5*2^23 + rint(v) are rint(v) + 2^22: bytes 0..2 are the digits
#pragma unroll
    for (int m = 0; m < 4; m++) {
      const float r = fmaf(xv[WvLane<BL>::j_of(k, m)], inv, 12582912.0f);
      X[m] = __float_as_uint(r);
      if constexpr (MmaCfg<F>::USES_SX && !MmaCfg<F>::INT_MID) fsum[m] += r - 12582912.0f;
    }
    const unsigned a01 = __byte_perm(X[0], X[1], 0x6240), a23 = __byte_perm(X[2], X[3], 0x6240);   // {b0,b0',b2,b2'}
    D[0][k] = __byte_perm(a01, a23, 0x5410);
    D[2][k] = __byte_perm(a01, a23, 0x7632);
    D[1][k] = __byte_perm(__byte_perm(X[0], X[1], 0x0051), __byte_perm(X[2], X[3], 0x0051), 0x5410);
    if constexpr (MmaCfg<F>::INT_MID) {
#pragma unroll
      for (int l = 0; l < 3; l++) sl[l] = dp4a_uu(D[l][k], 0x01010101u, sl[l]);
    }
  }
#pragma unroll
  for (int l = 0; l < 3; l++) {
    if constexpr (BL == 8) {   // a lane of the 8-bit A operand holds groups p and p + 4 (see load_a): same pairing here
      sts128(slot + 32u * l, D[l][0], D[l][4], D[l][1], D[l][5]);
      sts128(slot + 32u * l + 16u, D[l][2], D[l][6], D[l][3], D[l][7]);
    } else {
      sts128(slot + 32u * l, D[l][0], D[l][1], D[l][2], D[l][3]);
      sts128(slot + 32u * l + 16u, D[l][4], D[l][5], D[l][6], D[l][7]);
    }
  }
  if constexpr (MmaCfg<F>::INT_MID)
    sts128(slot + MMA_SLOT_K, (unsigned)(-fi.mid * sl[0]), (unsigned)(-fi.mid * sl[1]), (unsigned)(-fi.mid * sl[2]), (unsigned)(-fi.mid * 32));
  float sx = 0.f;
  if constexpr (MmaCfg<F>::USES_SX) {
    float tot;
    if constexpr (MmaCfg<F>::INT_MID) tot = (float)(sl[0] + (sl[1] << 8) + ((sl[2] - 32 * 64) << 16));
    else tot = (fsum[0] + fsum[1]) + (fsum[2] + fsum[3]);
    constexpr float coef = fi.has_min ? 1.0f : (fi.sign ? -1.0f : -((float)fi.mid + 0.5f));
    sx = coef * (sf * tot);
  }
  const float f0 = (fi.sign ? 2.0f * sf : sf) * MmaCfg<F>::A_SCALE;
  if constexpr (!MmaCfg<F>::INT_MID) sts128(slot + MMA_SLOT_K, 0u, 0u, 0u, 0u);
  sts128(slot + MMA_SLOT_META, __float_as_uint(f0), __float_as_uint(f0 * 65536.0f), __float_as_uint(sx), 0u);
}

// Offset of byte o of row r inside a plane's [piece][row][128 B] tile under the 128-byte swizzle
// (the 16-byte unit index is XORed with the row index modulo 8).
__device__ __forceinline__ unsigned mma_swz(unsigned o, unsigned r) {
  return (o >> 7) * 2048u + r * 128u + ((((o >> 4) & 7u) ^ (r & 7u)) << 4) + (o & 15u);
}

__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* tm, int c0, int c1, int c2, unsigned bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(tm)), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

// Peer vectors only in the instantiation that stores to them: the plain GEMV keeps a short parameter list.
struct MmaNoPeers {};
template <bool P> struct MmaPeerArgs { using type = MmaNoPeers; };
template <> struct MmaPeerArgs<true> { using type = WvPeers; };

template <int F, int PW, int NSEG, bool PEERS>
__global__ void __launch_bounds__(MMA_THREADS, 1)
gemv_mma_kernel(const WvDevBlob b, const float* __restrict__ xf, float* __restrict__ y, int row_begin, const MmaGeom g,
                int* __restrict__ err, const __grid_constant__ CUtensorMap tm_lo, const __grid_constant__ CUtensorMap tm_hi,
                const __grid_constant__ CUtensorMap tm_p0, const __grid_constant__ CUtensorMap tm_p1,
                const typename MmaPeerArgs<PEERS>::type peers) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  constexpr int BL = fi.bits_lo, BH = fi.bits_hi;
  constexpr bool INT_MID = MmaCfg<F>::INT_MID, SIGNED_A = MmaCfg<F>::SIGNED_A;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ unsigned s_xissued;   // consumer warps that have issued their loads of x
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bid = blockIdx.x;
  const int nmt = g.mt_base + (bid < g.mt_rem ? 1 : 0);
  const int c_lo = (bid * g.mt_base + min(bid, g.mt_rem)) * 16;
  const int band = min(nmt * 16, g.nrows - c_lo);
  // swizzled tiles want a 1024-byte aligned base
  const unsigned sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (sbase - smem_u32(smem_raw));
  const unsigned bar0 = sbase + g.bar_off;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (MMA_MAX_STAGES + s); };

  if (tid == 0) {
    s_abort = 0;
    s_xissued = 0;
    for (int s = 0; s < g.nstage; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), MMA_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < 12) reinterpret_cast<unsigned*>(smem + g.const_off)[tid] = tid < 4 ? 0u : 0x01010101u;  // 16 B of zeros, 32 B of ones
  __syncthreads();

  if (warp == MMA_WARPS) {
    // ------------------------------------------------------------ producer warp
    // Lane 0 issues one tensor-map copy per plane per tile.
    const CUtensorMap* tm[4] = {&tm_lo, &tm_hi, &tm_p0, &tm_p1};
    int ps = 0, issued = 0;
    unsigned ppar = 1;
    bool wrapped = false, dead = false;
    auto issue_tile = [&](int mt, int seg) {   // lane 0 only
      if (wrapped) {
        if (*(volatile int*)&s_abort || !mbar_wait(empty_bar(ps), ppar)) {
          if (!*(volatile int*)&s_abort) { atomicCAS_system(err, 0, 400 + ps); *(volatile int*)&s_abort = 1; }
          dead = true;
          return;
        }
      }
      mbar_expect_tx(full_bar(ps), g.tx_bytes);
      const unsigned dst = sbase + (unsigned)ps * g.stage_bytes;
      const int row0 = row_begin + c_lo + mt * 16;
#pragma unroll
      for (int i = 0; i < 4; i++)
        if (g.np[i]) tma_load_3d(dst + g.off[i], tm[i], 0, row0, seg * (int)g.np[i], full_bar(ps));
      issued++;
      if (++ps == g.nstage) { ps = 0; wrapped = true; ppar ^= 1u; }
    };
    if (lane == 0) {
      int mt = 0, seg = 0;
      for (int t = 0; t < g.lead && mt < nmt && !dead; t++) {
        issue_tile(mt, seg);
        if (++seg == g.nseg) { seg = 0; mt++; }
      }
      // The activation loads must not queue behind a full ring of weight traffic: after the
      // first tiles, hold further copies until every consumer warp has issued its loads of x
      // (a relaxed counter: a barrier here would wait for the loads to complete).
      for (unsigned i = 0; i < TMA_SPIN_LIMIT; i++) {
        if (*(volatile unsigned*)&s_xissued >= MMA_WARPS) break;
      }
      while (mt < nmt && !dead) {
        issue_tile(mt, seg);
        if (++seg == g.nseg) { seg = 0; mt++; }
      }
      // drain: every copy issued must have landed before the CTA gives its shared memory back
      for (int t = max(0, issued - g.nstage); t < issued; t++) {
        if (!mbar_wait(full_bar(t % g.nstage), (unsigned)(t / g.nstage) & 1u)) { atomicCAS_system(err, 0, 500 + t % g.nstage); break; }
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  // Everything that does not depend on x comes first: it overlaps the tail of the previous kernel.
  const unsigned xs0 = sbase + g.x_off;
  const int gr = lane >> 2, p = lane & 3, sel = p >> 1, part = p & 1;
  const int mulp = part ? -64 : 256;
  // B operand: lanes 0-15 carry columns 0..3 (chunk A: three digit columns and the ones), lanes
  // 16-31 columns 4..7 (chunk B). A lane keeps the words of its own chunk of every pair in
  // registers (loaded once after quantisation) and presents zeros for the other chunk.
  const int ncol = gr & 3;
  const unsigned dig = g.x_off + (unsigned)ncol * 32u + (unsigned)p * 8u;   // offset from the aligned base
  const unsigned maskA = lane < 16 ? 0xffffffffu : 0u, maskB = ~maskA;
  // A operand: this lane's word inside a chunk's lo / hi data and the shifts that bring its two
  // code groups (2p, 2p+1) down to bit 0
  const unsigned lo_lane = BL >= 4 ? p * 4u : (BL == 2 ? (p >> 1) * 4u : 0u);
  const int sh_lo = BL == 2 ? (p & 1) * 4 : (BL == 1 ? 2 * p : 0);
  const int sh_hi = 2 * p;
  constexpr unsigned MASK = 0x01010101u * ((1u << (BL & 7)) - 1u);
  constexpr unsigned MASKH = BH ? (0x01010101u << BL) : 0u;
  // The main loop reads shared memory through ordinary pointers (offsets from the aligned base),
  // so that the compiler can batch the loads of several chunk pairs ahead of their use.
  auto ld32 = [&](unsigned o) { return *reinterpret_cast<const unsigned*>(smem + o); };
  auto ld64 = [&](unsigned o) { return *reinterpret_cast<const uint2*>(smem + o); };
  auto ldf = [&](unsigned o) { return *reinterpret_cast<const float*>(smem + o); };
  auto load_a = [&](unsigned lo_o, unsigned hi_o, unsigned& q0, unsigned& q1) {
    if constexpr (BL == 8) {
      // words p and p + 4 of the chunk's eight: the second sits in the neighbouring 16-byte unit, which the
      // swizzle puts at the address with bit 4 flipped. Two 4-byte loads whose eight rows hit eight different
      // units, where one 8-byte load of words 2p, 2p + 1 would put rows g and g ^ 1 on the same banks.
      const unsigned w0 = ld32(lo_o), w1 = ld32(lo_o ^ 16u);
      q0 = SIGNED_A ? w0 ^ 0x80808080u : w0; q1 = SIGNED_A ? w1 ^ 0x80808080u : w1;
    } else if constexpr (SIGNED_A) {   // 4-bit: signed code * 16 in each byte
      const unsigned w = ld32(lo_o);
      q0 = ((w << 4) & 0xF0F0F0F0u) ^ 0x80808080u; q1 = (w & 0xF0F0F0F0u) ^ 0x80808080u;
    } else {
      const unsigned w = ld32(lo_o) >> sh_lo;
      q0 = w & MASK; q1 = (w >> BL) & MASK;
    }
    if constexpr (BH == 1) {
      const unsigned h = ld32(hi_o) >> sh_hi;
      q0 |= (h << BL) & MASKH; q1 |= ((h >> 1) << BL) & MASKH;
    }
  };
  // Swizzled offsets (row gr; row gr+8 is 1024 bytes further) of everything this lane reads from
  // a stage: fixed for the whole kernel because a warp owns the same chunks of every segment.
  const int wq = warp * PW * 2;   // first chunk of this warp inside a segment
  unsigned o_lo[2 * PW], o_hi[2 * PW], o_p[PW];
#pragma unroll
  for (int q = 0; q < 2 * PW; q++) {
    o_lo[q] = g.off[0] + mma_swz((unsigned)(wq + q) * (BL * 4u) + lo_lane, (unsigned)gr);
    o_hi[q] = g.off[1] + mma_swz((unsigned)(wq + q) * 4u, (unsigned)gr);
  }
#pragma unroll
  for (int i = 0; i < PW; i++) o_p[i] = mma_swz((unsigned)((wq + 2 * i + sel) >> g.gsh) * 4u, (unsigned)gr);


  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  {
    // x goes into the slots; all loads are issued before the first store
    const float* xrow = xf + (size_t)blockIdx.y * b.cols;
    const int nv = b.cols >> 2;
    if ((reinterpret_cast<uintptr_t>(xrow) & 15) == 0) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i = tid + u * MMA_WARPS * 32;
        if (i < nv) v[u] = __ldg(reinterpret_cast<const float4*>(xrow) + i);
      }
      if (lane == 0) asm volatile("red.relaxed.cta.shared::cta.add.u32 [%0], 1;" ::"r"(smem_u32(&s_xissued)) : "memory");
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i = tid + u * MMA_WARPS * 32;
        const unsigned ch = (unsigned)(i >> 3);
        if (i < nv) sts128(xs0 + ch * MMA_SLOT + (((unsigned)i & 7u) << 4), __float_as_uint(v[u].x), __float_as_uint(v[u].y),
                           __float_as_uint(v[u].z), __float_as_uint(v[u].w));
      }
    } else {
      if (lane == 0) asm volatile("red.relaxed.cta.shared::cta.add.u32 [%0], 1;" ::"r"(smem_u32(&s_xissued)) : "memory");
      for (int i = tid; i < b.cols; i += MMA_WARPS * 32) {
        const unsigned ch = (unsigned)(i >> 5), q = (unsigned)(i >> 2) & 7u;
        *reinterpret_cast<float*>(smem + g.x_off + ch * MMA_SLOT + (q << 4) + ((unsigned)i & 3u) * 4u) = __ldg(xrow + i);
      }
    }
  }
  asm volatile("bar.sync 15, %0;" ::"n"(MMA_WARPS * 32) : "memory");
  if (tid < g.cpr) mma_quantize_slot<F>(xs0 + (unsigned)tid * MMA_SLOT);
  asm volatile("bar.sync 15, %0;" ::"n"(MMA_WARPS * 32) : "memory");
  // this lane's B words and scale factor for each of its NSEG * PW chunk pairs
  // (the factors stay in shared memory when there are too many pairs for the register file)
  constexpr bool FR_REGS = NSEG * PW <= 8;
  unsigned bo0[NSEG * PW], bo1[NSEG * PW];
  float fr[FR_REGS ? NSEG * PW : 1];
#pragma unroll
  for (int sg = 0; sg < NSEG; sg++) {
#pragma unroll
    for (int i = 0; i < PW; i++) {
      const int jg = sg * (32 * PW) + wq + 2 * i;                 // chunk A of the pair
      const int jb = jg + (lane < 16 ? 0 : 1), js = jg + sel;
      uint2 w = make_uint2(0x01010101u, 0x01010101u);            // column 3 / 7: ones
      if (ncol < 3) w = jb < g.cpr ? ld64(dig + (unsigned)jb * MMA_SLOT) : make_uint2(0u, 0u);
      bo0[sg * PW + i] = w.x; bo1[sg * PW + i] = w.y;
      if constexpr (FR_REGS) fr[sg * PW + i] = js < g.cpr ? ldf(g.x_off + (unsigned)js * MMA_SLOT + MMA_SLOT_META + (unsigned)part * 4u) : 0.f;
      (void)js;
    }
  }

  float* red = reinterpret_cast<float*>(smem + g.red_off);
  float* yb = y + (size_t)blockIdx.y * b.rows + row_begin + c_lo;
  int fs = 0, par = 0;
  unsigned fpar = 0;
  bool dead = false;
  for (int mt = 0; mt < nmt; mt++) {
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int seg = 0; seg < NSEG; seg++) {
      if (!dead) {
        if (*(volatile int*)&s_abort) dead = true;
        else if (!mbar_wait(full_bar(fs), fpar)) { atomicCAS_system(err, 0, 600 + fs); *(volatile int*)&s_abort = 1; dead = true; }
      }
      const unsigned st = (unsigned)fs * g.stage_bytes;   // offset of the stage from the aligned base
      const int jseg = seg * (32 * PW) + wq;   // slot index of this warp's first chunk in the segment
#pragma unroll
      for (int i = 0; i < PW; i++) {
        // Chunk A = jseg + 2i, chunk B the next one. Pairs past the end of the row (last segment
        // only) read zero-filled codes and scales and carry zero B words and factors.
        const int jg = min(jseg + 2 * i, g.cpr - 2);
        const unsigned slot = g.x_off + (unsigned)(jg + sel) * MMA_SLOT;
        int c[4] = {0, 0, 0, 0};
        if constexpr (INT_MID) {
          const uint2 kk = ld64(slot + MMA_SLOT_K + (unsigned)part * 8u);
          c[0] = (int)kk.x; c[1] = (int)kk.y; c[2] = (int)kk.x; c[3] = (int)kk.y;
        }
        const unsigned b0 = bo0[seg * PW + i], b1 = bo1[seg * PW + i];
#pragma unroll
        for (int ch = 0; ch < 2; ch++) {
          unsigned a0, a1, a2, a3;
          const unsigned la = st + o_lo[2 * i + ch], ha = st + o_hi[2 * i + ch];
          load_a(la, ha, a0, a2);
          load_a(la + 1024u, ha + 1024u, a1, a3);
          const unsigned m = ch == 0 ? maskA : maskB;
          if constexpr (SIGNED_A) mma_s8u8(c, a0, a1, a2, a3, b0 & m, b1 & m);
          else mma_u8u8(c, a0, a1, a2, a3, b0 & m, b1 & m);
        }
        // lane (sel, part): chunk jg+sel, digits 0-1 (part 0) or digit 2 and the ones column (part 1)
        const unsigned pa = st + g.off[2] + o_p[i];
        const float s0 = ldf(pa), s1 = ldf(pa + 1024u);
        float f;
        if constexpr (FR_REGS) f = fr[seg * PW + i];
        else f = ldf(slot + MMA_SLOT_META + (unsigned)part * 4u);   // dead pairs: the scale read from the tile is zero
        const float t0 = (float)(c[0] + c[1] * mulp), t1 = (float)(c[2] + c[3] * mulp);
        acc0 = fmaf(s0 * f, t0, acc0);
        acc1 = fmaf(s1 * f, t1, acc1);
        if constexpr (MmaCfg<F>::USES_SX) {
          const float sxp = ldf(slot + MMA_SLOT_META + 8u + (unsigned)part * 4u);
          if constexpr (fi.has_min) {
            const unsigned pb = st + g.off[3] + o_p[i];
            acc0 = fmaf(ldf(pb), sxp, acc0);
            acc1 = fmaf(ldf(pb + 1024u), sxp, acc1);
          } else {
            acc0 = fmaf(s0, sxp, acc0);
            acc1 = fmaf(s1, sxp, acc1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(fs));
      if (++fs == g.nstage) { fs = 0; fpar ^= 1u; }
    }
    // 16 row sums of this block: over the quad, then over the warps
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1); acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2); acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    float* mine = red + ((size_t)par * MMA_WARPS + warp) * 16;
    if (p == 0) { mine[gr] = acc0; mine[gr + 8] = acc1; }
    asm volatile("bar.sync 15, %0;" ::"n"(MMA_WARPS * 32) : "memory");
    if (warp == (mt & (MMA_WARPS - 1)) && lane < 16) {
      const float* base = red + (size_t)par * MMA_WARPS * 16 + lane;
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < MMA_WARPS; q++) sum += base[q * 16];
      const int row = mt * 16 + lane;
      if (row < band) {
        if constexpr (PEERS) {
          reinterpret_cast<float*>(smem + g.ysm_off)[row] = sum;
        } else {
          yb[row] = sum;
        }
      }
    }
    par ^= 1;
  }
  if constexpr (PEERS) {
    // Own and peers' copies of y, after the main loop: a store to a peer issued between two tiles holds its warp, and
    // through the per-tile barrier the whole CTA, for as long as the first access to that peer's mapping takes
    // (measured with eight ranks: 43 us against 31 us for a 148 MB shard).
    asm volatile("bar.sync 15, %0;" ::"n"(MMA_WARPS * 32) : "memory");
    const float* ysm = reinterpret_cast<const float*>(smem + g.ysm_off);
    for (int q = warp; q < peers.n; q += MMA_WARPS) {      // a warp per peer: their first accesses wait side by side
      float* yq = peers.y[q] + row_begin + c_lo;
      for (int r = lane; r < band; r += 32) yq[r] = ysm[r];
    }
  }
}

// ------------------------------------------------------------------ host side
int wv_tma_tuning_stages();   // wv_gemv_tma.cu: ring-depth cap (low two digits) and lead tiles (hundreds) of the experiment hook
static unsigned align128u(unsigned v) { return (v + 127u) & ~127u; }

// Tensor maps are encoded once per (plane, shape, segment width) and kept: encoding goes through
// the driver entry point and is far too slow to repeat on every launch.
struct MmaMaps { CUtensorMap m[4]; };
static std::mutex g_maps_mu;
static std::map<std::tuple<const void*, int, int, int, int, int>, MmaMaps> g_maps;

static PFN_cuTensorMapEncodeTiled_v12000 mma_encode_fn() {
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

// Plane of `rows` rows of `rb` bytes (rb a multiple of 128) seen as {128 B, rows, rb/128 pieces};
// one box = 128 B x 16 rows x np pieces.
static bool mma_encode_plane(CUtensorMap* out, const void* base, unsigned rb, int rows, unsigned np) {
  auto fn = mma_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {128, (cuuint64_t)rows, (cuuint64_t)(rb / 128u)};
  cuuint64_t strides[2] = {(cuuint64_t)rb, 128};
  cuuint32_t box[3] = {128, 16, np};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int F, int PW, int NSEG>
static int launch_mma(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb_, int re, cudaStream_t st) {
  constexpr WvFmtInfo fi = wv_fmt_info(F);
  MmaGeom g{};
  if (b.cols & 31) return 1;
  g.cpr = b.cols >> 5;
  g.seg_chunks = 32 * PW;
  g.nseg = (g.cpr + g.seg_chunks - 1) / g.seg_chunks;
  if (g.nseg != NSEG) return 1;
  if (g.cpr > MMA_WARPS * 32 || (g.cpr & 1)) return 1;   // one quantising thread per chunk; chunks are used in pairs
  const unsigned bpc[4] = {fi.bits_lo * 4u, fi.bits_hi * 4u, 4u, fi.has_min ? 4u : 0u};  // bytes per chunk (p0 / p1: per group)
  int ratio = 1;
  if (fi.kind == WK_BINARY || fi.kind == WK_AFFINE) {
    if (b.group < 32 || (b.group % 32) || (b.cols % b.group)) return 1;
    ratio = b.group / 32;
    if ((ratio & (ratio - 1)) || ratio > 16) return 1;
  }
  g.gsh = 0;
  while ((1 << g.gsh) < ratio) g.gsh++;
  unsigned rb[4];
  const void* base[4] = {b.lo, b.hi, b.p0, b.p1};
  unsigned off = 0;
  for (int i = 0; i < 4; i++) {
    const unsigned per_seg = i < 2 ? bpc[i] * g.seg_chunks : bpc[i] * g.seg_chunks / ratio;
    rb[i] = i < 2 ? bpc[i] * g.cpr : bpc[i] * g.cpr / ratio;
    if ((rb[i] % 128) || (per_seg % 128) || (reinterpret_cast<uintptr_t>(base[i]) & 15)) return 1;
    g.np[i] = per_seg / 128u;
    if (g.np[i] > 256) return 1;
    g.off[i] = off;
    off += g.np[i] * 2048u;
  }
  g.stage_bytes = off;
  g.tx_bytes = off;
  g.nrows = re - rb_;
  const int total_mt = (g.nrows + 15) / 16;
  int grid = wv_sm_count();
  if (grid > total_mt) grid = total_mt;
  g.mt_base = total_mt / grid;
  g.mt_rem = total_mt % grid;
  const unsigned ybytes = wv_cur_peers ? align128u((unsigned)(g.mt_base + 1) * 16u * 4u) : 0u;
  if (ybytes > 32768u) return 1;
  const unsigned xbytes = align128u((unsigned)g.cpr * MMA_SLOT);
  const unsigned fixed = 1024u + xbytes + 128u + 2u * MMA_WARPS * 16u * 4u + ybytes + 2u * MMA_MAX_STAGES * 8u + 128u;
  const unsigned avail = 225u * 1024u;
  if (g.stage_bytes * 2 + fixed > avail) return 1;
  int ns = (int)((avail - fixed) / g.stage_bytes);
  if (ns > MMA_MAX_STAGES) ns = MMA_MAX_STAGES;
  g.nstage = ns;
  const int knob = wv_tma_tuning_stages();
  if (knob % 100 > 1 && knob % 100 < ns) g.nstage = ns = knob % 100;
  g.lead = knob >= 100 ? knob / 100 : 1;
  g.x_off = g.stage_bytes * ns;
  g.const_off = g.x_off + xbytes;
  g.red_off = g.const_off + 128u;
  g.ysm_off = align128u(g.red_off + 2u * MMA_WARPS * 16u * 4u);
  g.bar_off = g.ysm_off + ybytes;
  const size_t smem = 1024u + g.bar_off + 2 * MMA_MAX_STAGES * 8;

  MmaMaps maps;
  {
    std::lock_guard<std::mutex> lk(g_maps_mu);
    const auto key = std::make_tuple((const void*)b.lo, b.rows, b.cols, b.format, b.group, PW);
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
      MmaMaps m{};
      for (int i = 0; i < 4; i++) {
        const bool ok = g.np[i] ? mma_encode_plane(&m.m[i], base[i], rb[i], b.rows, g.np[i])
                                : mma_encode_plane(&m.m[i], base[0], rb[0], b.rows, g.np[0]);   // placeholder, never used
        if (!ok) {
          static bool warned = false;
          if (!warned) { warned = true; fprintf(stderr, "welvet_cuda: tensor-map encoding failed, using the dp4a kernel\n"); }
          return 1;
        }
      }
      if (g_maps.size() > 4096) g_maps.clear();
      it = g_maps.emplace(key, m).first;
    }
    maps = it->second;
  }

  int dev = 0; cudaGetDevice(&dev);
  cudaError_t e;
  if (!wv_cur_peers) {
    auto kern = gemv_mma_kernel<F, PW, NSEG, false>;
    static unsigned attr_mask = 0;
    if (!(attr_mask & (1u << dev))) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) { wv_set_error("gemv (mma): cannot raise the shared-memory limit"); return WV_ECUDA; }
      attr_mask |= 1u << dev;
    }
    e = launch_pdl(kern, dim3(grid, batch), dim3(MMA_THREADS), smem, st, b, dx, dy, rb_, g, wv_tma_err_ptr(),
                   maps.m[0], maps.m[1], maps.m[2], maps.m[3], MmaNoPeers{});
  } else if constexpr (PW != 4 && !(PW == 2 && F == WV_Q8_0)) {
    return 1;   // the peer-storing variant exists for the default configurations only
  } else {
    if (batch != 1) return WV_ESHAPE;
    auto kern = gemv_mma_kernel<F, PW, NSEG, true>;
    static unsigned attr_mask = 0;
    if (!(attr_mask & (1u << dev))) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) { wv_set_error("gemv (mma): cannot raise the shared-memory limit"); return WV_ECUDA; }
      attr_mask |= 1u << dev;
    }
    e = launch_pdl(kern, dim3(grid, batch), dim3(MMA_THREADS), smem, st, b, dx, dy, rb_, g, wv_tma_err_ptr(),
                   maps.m[0], maps.m[1], maps.m[2], maps.m[3], *wv_cur_peers);
  }
  if (e != cudaSuccess) { wv_set_error("gemv (mma) launch: %s", cudaGetErrorString(e)); return WV_ECUDA; }
  return WV_OK;
}

template <int F>
static int launch_mma_format(const WvDevBlob& b, const float* dx, float* dy, int batch, int rb, int re, cudaStream_t st, int pw) {
  if constexpr (MmaCfg<F>::OK) {
    // the segment count is a template parameter: per-pair operands live in registers
    const int cpr = b.cols >> 5;
    if (pw == 2) {
      switch ((cpr + 63) / 64) {
      case 1: return launch_mma<F, 2, 1>(b, dx, dy, batch, rb, re, st);
      case 2: return launch_mma<F, 2, 2>(b, dx, dy, batch, rb, re, st);
      case 4: return launch_mma<F, 2, 4>(b, dx, dy, batch, rb, re, st);
      case 7: return launch_mma<F, 2, 7>(b, dx, dy, batch, rb, re, st);
      }
      return 1;
    }
    switch ((cpr + 127) / 128) {
    case 1: return launch_mma<F, 4, 1>(b, dx, dy, batch, rb, re, st);
    case 2: return launch_mma<F, 4, 2>(b, dx, dy, batch, rb, re, st);
    case 3: return launch_mma<F, 4, 3>(b, dx, dy, batch, rb, re, st);
    case 4: return launch_mma<F, 4, 4>(b, dx, dy, batch, rb, re, st);
    }
  }
  return 1;
}

// Returns WV_OK, an error, or 1 when the format or shape is not served by this kernel.
int wv_launch_gemv_mma(const WvDevBlob& b, const float* dx, float* dy, int batch, int row_begin, int row_end, cudaStream_t st, int pw) {
  switch (b.format) {
#define WV_F(f) case f: return launch_mma_format<f>(b, dx, dy, batch, row_begin, row_end, st, pw);
  WV_F(WV_Q8_0) WV_F(WV_Q4_0) WV_F(WV_Q4_1) WV_F(WV_Q5_0) WV_F(WV_Q5_1)
  WV_F(WV_IQ1_S) WV_F(WV_IQ2_XXS) WV_F(WV_IQ3_XXS) WV_F(WV_BINARY) WV_F(WV_AFFINE)
#undef WV_F
  }
  return 1;
}
