// The host-ALU steps that sit between the Dense GEMVs of a decoder block in single-token decode,
// on the device, so that activations never leave HBM between projections: RMSNorm, rotary
// position embedding with the KV-cache write, grouped-query attention over the cache, the SwiGLU
// gate product and the residual add. The reference runs all of them in float64 on the host
// (layers/rmsnorm/cpu.go:32-90, layers/mha/rope.go:6-21, layers/mha/cpu.go:184-207,
// layers/mha/attn.go:15-120, simd/silu.go:14-27, model/transformer/scratch.go:33-41); here sums that
// decide a normalisation are kept in float64 and the rest is float32.
#include "wv_common.cuh"
#include <math.h>
#include <stdlib.h>

// ------------------------------------------------------------------ RMSNorm
// y[i] = x[i] * inv * gamma[i], inv = 1 / sqrt(sum(x^2) / dim + eps)  (rmsnorm/cpu.go:76-85).
// One CTA per token row; the sum of squares and the scale are float64 as in the reference.
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                       float* __restrict__ y, int dim, double eps) {
  __shared__ double s_part[32];
  __shared__ double s_inv;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float* xr = x + (size_t)blockIdx.x * dim;
  float* yr = y + (size_t)blockIdx.x * dim;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  double acc = 0.0;
  for (int i = tid; i < dim; i += blockDim.x) { const double v = (double)xr[i]; acc += v * v; }
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) s_part[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    double t = lane < (int)(blockDim.x >> 5) ? s_part[lane] : 0.0;
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) s_inv = 1.0 / sqrt(t / (double)dim + eps);
  }
  __syncthreads();
  const double inv = s_inv;
  for (int i = tid; i < dim; i += blockDim.x) yr[i] = (float)(((double)xr[i] * inv) * (double)gamma[i]);
}

int wv_launch_rmsnorm(const float* dx, const float* dgamma, float* dy, int rows, int dim, double eps, cudaStream_t st) {
  int threads = dim >= 4096 ? 1024 : (dim >= 1024 ? 512 : 128);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows); cfg.blockDim = dim3(threads); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, rmsnorm_kernel, dx, dgamma, dy, dim, eps) == cudaSuccess ? WV_OK : WV_ECUDA;
}

// ------------------------------------------------------------------ RoPE + KV-cache write
// applyRoPE (mha/rope.go:6-21) on the new token's Q (in place) and K, then K and V go into slot
// pos % msl of the caches (mha/cpu.go:184-207: the rotated K row is what the cache keeps).
// angle = pos / theta^(2d/headDim), pairs (d, d + headDim/2), float64 trigonometry.
__global__ void __launch_bounds__(256) rope_cache_kernel(float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                         float* __restrict__ cache_k, float* __restrict__ cache_v, int pos, int msl,
                                                         int num_heads, int num_kv_heads, int head_dim, double theta) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int half = head_dim >> 1;
  const int nq = num_heads * half, nk = num_kv_heads * half;
  const size_t slot = (size_t)(pos % msl) * num_kv_heads * head_dim;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nq + nk; i += gridDim.x * blockDim.x) {
    const bool is_q = i < nq;
    const int j = is_q ? i : i - nq;
    const int h = j / half, d = j % half;
    double c = 1.0, s = 0.0;
    if (half > 0 && theta > 0.0) {
      const double angle = (double)pos / pow(theta, (double)(2 * d) / (double)head_dim);
      sincos(angle, &s, &c);
    }
    const int base = h * head_dim;
    if (is_q) {
      const double v0 = q[base + d], v1 = q[base + d + half];
      q[base + d] = (float)(v0 * c - v1 * s);
      q[base + d + half] = (float)(v0 * s + v1 * c);
    } else {
      const double v0 = k[base + d], v1 = k[base + d + half];
      cache_k[slot + base + d] = (float)(v0 * c - v1 * s);
      cache_k[slot + base + d + half] = (float)(v0 * s + v1 * c);
      cache_v[slot + base + d] = v[base + d];
      cache_v[slot + base + d + half] = v[base + d + half];
    }
  }
}

int wv_launch_rope_cache(float* dq, const float* dk, const float* dv, float* dcache_k, float* dcache_v, int pos, int msl,
                         int num_heads, int num_kv_heads, int head_dim, double theta, cudaStream_t st) {
  const int n = (num_heads + num_kv_heads) * (head_dim / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((n + 255) / 256 > 0 ? (n + 255) / 256 : 1); cfg.blockDim = dim3(256); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, rope_cache_kernel, dq, dk, dv, dcache_k, dcache_v, pos, msl, num_heads, num_kv_heads, head_dim, theta) ==
                 cudaSuccess ? WV_OK : WV_ECUDA;
}

// ------------------------------------------------------------------ single-token attention over the cache
// attnForward (mha/attn.go:15-120) for seqLen 1 under the causal mask: the query at position
// kv_len - 1 sees cache rows 0 .. kv_len-1 (row kPos lives in slot kPos % msl), grouped-query heads
// share kv head h / (heads / kv_heads), scores = q.k * scale, max-subtracted softmax, out = sum w v.
//
// Two launches. attn_split_kernel: one CTA per (group of GC query heads that share a kv head, split of the
// positions), about two CTAs per SM; a K or V row is read once for the GC heads, a warp's K rows are all in flight
// together and its first V rows are requested before the softmax of the scores. Each CTA leaves one record
// {max, sum, acc[head_dim]} per head. attn_merge_kernel: one CTA per head, one thread per dimension, merges the
// records in split order (the result does not depend on the order the CTAs ran in) with every load of a batch of
// splits in flight at once. Every step of this kernel pair is a round trip to L2, so the structure is chosen to
// keep their number small: q, K, (V), records out | records in, result out. head_dim <= 256, multiple of 4.
#define ATT_THREADS 256
#define ATT_WARPS (ATT_THREADS / 32)
#define ATT_CHUNK 256        // positions per split at most
#define ATT_MERGE_BATCH 40
template <int GC, bool WIDE>
__global__ void __launch_bounds__(ATT_THREADS, 2) attn_split_kernel(const float* __restrict__ q, const float* __restrict__ cache_k,
                                                                 const float* __restrict__ cache_v, float* __restrict__ out,
                                                                 float* __restrict__ part, int num_heads, int num_kv_heads,
                                                                 int head_dim, int kv_len, int msl, float scale, int nsplit) {
  constexpr int UN = WIDE ? 4 : 8;                        // rows a warp has in flight
  constexpr bool EARLY_V = GC * (WIDE ? 2 : 1) <= 4;       // registers allow requesting the first V rows before the softmax
  extern __shared__ __align__(16) float att_smem[];
  float* s_score = att_smem;                              // [GC][ATT_CHUNK]
  float* s_acc = att_smem + GC * ATT_CHUNK;               // [ATT_WARPS][GC][head_dim]
  __shared__ float s_max[GC], s_sum[GC];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int grp = blockIdx.x, sp = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h0 = grp * GC;
  const int kvh = h0 / (num_heads / num_kv_heads);
  const int kv_dim = num_kv_heads * head_dim;
  const int per = (kv_len + nsplit - 1) / nsplit;
  const int p0 = sp * per, p1 = min(kv_len, p0 + per);
  const int n = max(0, p1 - p0);
  const int vec = head_dim >> 2;           // float4 per row; lanes beyond it idle
  const bool on0 = lane < vec, on1 = WIDE && lane + 32 < vec;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  auto row_of = [&](const float* cache, int i) {
    return reinterpret_cast<const float4*>(cache + (size_t)((p0 + min(i, max(n - 1, 0))) % msl) * kv_dim + (size_t)kvh * head_dim);
  };
  float4 vv[UN], vw[WIDE ? UN : 1];          // V rows of the warp's first positions, requested early
  {
    // scores: a warp takes positions warp, warp + 8, ...
    float4 qv[GC], qw[WIDE ? GC : 1];
#pragma unroll
    for (int g = 0; g < GC; g++) {
      const float4* qh = reinterpret_cast<const float4*>(q + (size_t)(h0 + g) * head_dim);
      qv[g] = on0 ? qh[lane] : zero4;
      if (WIDE) qw[g] = on1 ? qh[lane + 32] : zero4;
    }
    for (int i0 = warp; i0 < n; i0 += ATT_WARPS * UN) {
      float4 kk[UN], kw[WIDE ? UN : 1];
#pragma unroll
      for (int u = 0; u < UN; u++) {
        const float4* kr = row_of(cache_k, i0 + u * ATT_WARPS);
        kk[u] = on0 ? kr[lane] : zero4;
        if (WIDE) kw[u] = on1 ? kr[lane + 32] : zero4;
      }
      if (EARLY_V && i0 == warp) {
#pragma unroll
        for (int u = 0; u < UN; u++) {
          const float4* vr = row_of(cache_v, i0 + u * ATT_WARPS);
          vv[u] = on0 ? vr[lane] : zero4;
          if (WIDE) vw[u] = on1 ? vr[lane + 32] : zero4;
        }
      }
#pragma unroll
      for (int u = 0; u < UN; u++) {
        const int i = i0 + u * ATT_WARPS;
#pragma unroll
        for (int g = 0; g < GC; g++) {
          float d = qv[g].x * kk[u].x + qv[g].y * kk[u].y + qv[g].z * kk[u].z + qv[g].w * kk[u].w;
          if (WIDE) d += qw[g].x * kw[u].x + qw[g].y * kw[u].y + qw[g].z * kw[u].z + qw[g].w * kw[u].w;
#pragma unroll
          for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          if (lane == 0 && i < n) s_score[g * ATT_CHUNK + i] = d * scale;
        }
      }
    }
  }
  __syncthreads();
  // max-subtracted exponentials: warp g takes head g
  for (int g = warp; g < GC; g += ATT_WARPS) {
    float m = -3.0e38f;
    for (int i = lane; i < n; i += 32) m = fmaxf(m, s_score[g * ATT_CHUNK + i]);
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float t = 0.f;
    for (int i = lane; i < n; i += 32) { const float e = __expf(s_score[g * ATT_CHUNK + i] - m); s_score[g * ATT_CHUNK + i] = e; t += e; }
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) { s_max[g] = m; s_sum[g] = t; }
  }
  __syncthreads();
  {
    // weighted sum of the V rows: a lane keeps its 4 (+4) dimensions of every head
    float4 a0[GC], a1[WIDE ? GC : 1];
#pragma unroll
    for (int g = 0; g < GC; g++) { a0[g] = zero4; if (WIDE) a1[g] = zero4; }
    for (int i0 = warp; i0 < n; i0 += ATT_WARPS * UN) {
      if (!EARLY_V || i0 != warp) {
#pragma unroll
        for (int u = 0; u < UN; u++) {
          const float4* vr = row_of(cache_v, i0 + u * ATT_WARPS);
          vv[u] = on0 ? vr[lane] : zero4;
          if (WIDE) vw[u] = on1 ? vr[lane + 32] : zero4;
        }
      }
#pragma unroll
      for (int u = 0; u < UN; u++) {
        const int i = i0 + u * ATT_WARPS;
        if (i < n) {
#pragma unroll
          for (int g = 0; g < GC; g++) {
            const float w = s_score[g * ATT_CHUNK + i];
            a0[g].x += w * vv[u].x; a0[g].y += w * vv[u].y; a0[g].z += w * vv[u].z; a0[g].w += w * vv[u].w;
            if (WIDE) { a1[g].x += w * vw[u].x; a1[g].y += w * vw[u].y; a1[g].z += w * vw[u].z; a1[g].w += w * vw[u].w; }
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < GC; g++) {
      float4* d = reinterpret_cast<float4*>(s_acc + ((size_t)warp * GC + g) * head_dim);
      if (on0) d[lane] = a0[g];
      if (WIDE) { if (on1) d[lane + 32] = a1[g]; }
    }
  }
  __syncthreads();
  // this split's records, one per head: [0] max, [1] sum, [2 ..] unnormalised accumulators (warps summed in order)
  for (int e = tid; e < GC * head_dim; e += ATT_THREADS) {
    const int g = e / head_dim, dim = e - g * head_dim;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) t += s_acc[((size_t)w * GC + g) * head_dim + dim];
    if (nsplit == 1) out[(size_t)(h0 + g) * head_dim + dim] = n > 0 ? t / s_sum[g] : 0.f;
    else part[((size_t)(h0 + g) * nsplit + sp) * (head_dim + 2) + 2 + dim] = t;
  }
  if (nsplit > 1 && tid < GC) {
    float* rec = part + ((size_t)(h0 + tid) * nsplit + sp) * (head_dim + 2);
    rec[0] = n > 0 ? s_max[tid] : -3.0e38f;
    rec[1] = n > 0 ? s_sum[tid] : 0.f;
  }
}

// Merge of the splits' records of one head (blockIdx.x), one thread per dimension, in split order.
__global__ void __launch_bounds__(256) attn_merge_kernel(const float* __restrict__ part, float* __restrict__ out, int head_dim, int nsplit) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int h = blockIdx.x, dim = threadIdx.x;
  if (dim >= head_dim) return;
  const float* base = part + (size_t)h * nsplit * (head_dim + 2);
  float gm = -3.0e38f, tot = 0.f, acc = 0.f;
  for (int s0 = 0; s0 < nsplit; s0 += ATT_MERGE_BATCH) {
    float m[ATT_MERGE_BATCH], t[ATT_MERGE_BATCH], v[ATT_MERGE_BATCH];
#pragma unroll
    for (int u = 0; u < ATT_MERGE_BATCH; u++) {
      const bool on = s0 + u < nsplit;
      const float* r = base + (size_t)(on ? s0 + u : s0) * (head_dim + 2);
      m[u] = on ? r[0] : -3.0e38f;
      t[u] = on ? r[1] : 0.f;
      v[u] = on ? r[2 + dim] : 0.f;
    }
    float bm = gm;
#pragma unroll
    for (int u = 0; u < ATT_MERGE_BATCH; u++) bm = fmaxf(bm, m[u]);
    const float resc = __expf(gm - bm);     // 1 for the first batch's gm = -3e38 start as well: tot and acc are 0 then
    tot *= resc; acc *= resc; gm = bm;
#pragma unroll
    for (int u = 0; u < ATT_MERGE_BATCH; u++) {
      const float f = __expf(m[u] - gm);
      tot += f * t[u];
      acc += f * v[u];
    }
  }
  out[(size_t)h * head_dim + dim] = tot > 0.f ? acc / tot : 0.f;
}

// Records of the splits: nsplit per head, owned by the library.
static float* g_att_part = nullptr;
static size_t g_att_part_floats = 0;

template <int GC, bool WIDE>
static int attn_launch(cudaLaunchConfig_t& cfg, size_t smem, const float* dq, const float* dk, const float* dv, float* dout, int num_heads,
                       int num_kv_heads, int head_dim, int kv_len, int msl, float scale, int nsplit) {
  static unsigned attr_mask = 0;   // per device: opt in to more than 48 KB of dynamic shared memory once
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && !(attr_mask & (1u << (dev & 31)))) {
    if (cudaFuncSetAttribute(attn_split_kernel<GC, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return WV_ECUDA;
    attr_mask |= 1u << (dev & 31);
  }
  cfg.dynamicSmemBytes = smem;
  return cudaLaunchKernelEx(&cfg, attn_split_kernel<GC, WIDE>, dq, dk, dv, dout, g_att_part, num_heads, num_kv_heads, head_dim,
                            kv_len, msl, scale, nsplit) == cudaSuccess ? WV_OK : WV_ECUDA;
}

int wv_launch_attn_decode(const float* dq, const float* dcache_k, const float* dcache_v, float* dout, int num_heads, int num_kv_heads,
                          int head_dim, int kv_len, int msl, float scale, cudaStream_t st) {
  if (head_dim > 256 || (head_dim & 3) || num_heads % num_kv_heads) { wv_set_error("attention: head_dim %d / heads %d:%d not supported", head_dim, num_heads, num_kv_heads); return WV_ESHAPE; }
  // query heads per CTA: the largest power of two <= 8 that divides the group of heads sharing a kv head
  const int G = num_heads / num_kv_heads;
  int gc = 1;
  while (gc < 8 && G % (gc * 2) == 0) gc *= 2;
  const int ngroups = num_heads / gc;
  // splits: about two CTAs per SM, at least 8 positions and at most ATT_CHUNK positions each
  int ctas = 2 * 148;
#ifdef WV_DEV_HOOKS
  if (const char* e = getenv("WV_ATT_CTAS")) ctas = atoi(e);
#endif
  int nsplit = (ctas + ngroups - 1) / ngroups;
  if (nsplit > kv_len / 8) nsplit = kv_len / 8;
  if (nsplit < 1) nsplit = 1;
  if ((kv_len + nsplit - 1) / nsplit > ATT_CHUNK) nsplit = (kv_len + ATT_CHUNK - 1) / ATT_CHUNK;
  if (nsplit > 65536) { wv_set_error("attention: kv_len %d too long", kv_len); return WV_ESHAPE; }
  const size_t need = (size_t)num_heads * nsplit * (head_dim + 2);
  if (need > g_att_part_floats) {
    // grows only when a larger shape arrives (set-up time: not capturable)
    cudaStreamSynchronize(st);
    if (g_att_part) cudaFree(g_att_part);
    g_att_part = nullptr;
    const size_t want = need * 2;
    if (cudaMalloc(&g_att_part, want * 4) != cudaSuccess) { cudaGetLastError(); g_att_part_floats = 0; wv_set_error("attention: scratch allocation failed"); return WV_ENOMEM; }
    g_att_part_floats = want;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ngroups, nsplit); cfg.blockDim = dim3(ATT_THREADS); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  const size_t smem = ((size_t)gc * ATT_CHUNK + (size_t)ATT_WARPS * gc * head_dim) * sizeof(float);
  const bool wide = head_dim > 128;
  int rc;
#define ATT_GO(GC_) (wide ? attn_launch<GC_, true>(cfg, smem, dq, dcache_k, dcache_v, dout, num_heads, num_kv_heads, head_dim, kv_len, msl, scale, nsplit) \
                          : attn_launch<GC_, false>(cfg, smem, dq, dcache_k, dcache_v, dout, num_heads, num_kv_heads, head_dim, kv_len, msl, scale, nsplit))
  switch (gc) {
    case 8: rc = ATT_GO(8); break;
    case 4: rc = ATT_GO(4); break;
    case 2: rc = ATT_GO(2); break;
    default: rc = ATT_GO(1); break;
  }
#undef ATT_GO
  if (rc || nsplit == 1) return rc;
  cudaLaunchConfig_t mc = {};
  mc.gridDim = dim3(num_heads); mc.blockDim = dim3((head_dim + 31) & ~31); mc.stream = st;
  mc.attrs = at; mc.numAttrs = 1;
  const float* cpart = g_att_part;
  return cudaLaunchKernelEx(&mc, attn_merge_kernel, cpart, dout, head_dim, nsplit) == cudaSuccess ? WV_OK : WV_ECUDA;
}

// ------------------------------------------------------------------ SwiGLU gate product and residual add
// out[i] = float32(g / (1 + exp(-g)) * up[i]) with g = float64(gate[i])  (simd/silu.go:14-27).
__global__ void silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ out, int n) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const double g = (double)gate[i];
    out[i] = (float)(g / (1.0 + exp(-g)) * (double)up[i]);
  }
}
// dst[i] += add[i]  (model/transformer/scratch.go:33-41)
__global__ void residual_add_kernel(float* __restrict__ dst, const float* __restrict__ add, int n) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] += add[i];
}

template <typename... KArgs, typename... Args>
static int launch_small(void (*kern)(KArgs...), int n, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  int blocks = (n + 255) / 256;
  if (blocks > 592) blocks = 592;
  if (blocks < 1) blocks = 1;
  cfg.gridDim = dim3(blocks); cfg.blockDim = dim3(256); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...) == cudaSuccess ? WV_OK : WV_ECUDA;
}
int wv_launch_silu_mul(const float* dgate, const float* dup, float* dout, int n, cudaStream_t st) {
  return launch_small(silu_mul_kernel, n, st, dgate, dup, dout, n);
}
int wv_launch_residual_add(float* ddst, const float* dadd, int n, cudaStream_t st) {
  return launch_small(residual_add_kernel, n, st, ddst, dadd, n);
}

// ------------------------------------------------------------------ top-K sampling over the logits
// sampling.SampleTopK (model/sampling/topk.go:11-50) for 1 <= K <= 1024 without reading the logits back:
// candidates are v / temperature (a float32 divide), ordered by value descending; p_i = exp(float64(val_i - max))
// with the subtraction in float32; the draw r = u * sum(p) walks the running sum in that order and the first
// candidate with r <= acc wins, the last one otherwise. The reference takes u from math/rand's global source; here
// the caller passes it, so that the host keeps the one random stream. sort.Slice leaves the order of equal values
// open; here equal values go by rising index. A NaN logit is ordered by its bit pattern (the reference's order with
// NaN is whatever its sort happens to do).
//
// One CTA. Each logit becomes a 64-bit word (ordered value bits : ~index), all distinct; a most-significant-digit
// radix select (8 bits a pass, stopping as soon as a bucket holds exactly what is still needed) finds the K-th
// largest word, the K words at or above it are gathered and sorted by a bitonic network in shared memory, and
// thread 0 does the two short sequential float64 walks so that the sums round as the reference's do.
#define TOPK_MAX 1024
__device__ __forceinline__ unsigned long long topk_word(float v, float temperature, int i) {
  const float val = __fdiv_rn(v, temperature);
  unsigned u = __float_as_uint(val);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)i);
}
__global__ void __launch_bounds__(1024, 1) topk_sample_kernel(const float* __restrict__ v, int n, int k, float temperature, double u01,
                                                              int* __restrict__ out) {
  __shared__ unsigned s_hist[256];
  __shared__ unsigned long long s_cand[TOPK_MAX];
  __shared__ double s_p[TOPK_MAX];
  __shared__ unsigned long long s_prefix;
  __shared__ unsigned s_need, s_done, s_count;
  const int tid = threadIdx.x;
  if (tid == 0) { s_prefix = 0ull; s_need = (unsigned)k; s_done = 0u; s_count = 0u; }
  __syncthreads();
  unsigned long long thresh = 0ull;
  for (int pass = 0; pass < 8; pass++) {
    const int shift = 56 - 8 * pass;
    if (tid < 256) s_hist[tid] = 0u;
    __syncthreads();
    const unsigned long long prefix = s_prefix;
    const unsigned long long himask = pass == 0 ? 0ull : (~0ull << (shift + 8));
    for (int i = tid; i < n; i += 1024) {
      const unsigned long long w = topk_word(v[i], temperature, i);
      if ((w & himask) == prefix) atomicAdd(&s_hist[(unsigned)(w >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned need = s_need, d = 255u;
      for (;; d--) {               // from the top digit down: the bucket where the running count reaches `need`
        const unsigned c = s_hist[d];
        if (c >= need || d == 0u) { if (c == need) s_done = 1u; break; }
        need -= c;
      }
      s_need = need;
      s_prefix = prefix | ((unsigned long long)d << shift);
    }
    __syncthreads();
    thresh = s_prefix;             // low digits still zero: every word of the chosen bucket is >= thresh
    if (s_done) break;
  }
  for (int i = tid; i < n; i += 1024) {
    const unsigned long long w = topk_word(v[i], temperature, i);
    if (w >= thresh) { const unsigned slot = atomicAdd(&s_count, 1u); if (slot < TOPK_MAX) s_cand[slot] = w; }
  }
  __syncthreads();
  const int cnt = min((int)s_count, TOPK_MAX);   // == k by construction
  int p2 = 1;
  while (p2 < cnt) p2 <<= 1;
  for (int i = tid; i < p2; i += 1024) if (i >= cnt) s_cand[i] = 0ull;
  __syncthreads();
  for (int size = 2; size <= p2; size <<= 1) {   // bitonic sort, descending
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < p2; i += 1024) {
        const int j = i ^ stride;
        if (j > i) {
          const unsigned long long a = s_cand[i], b = s_cand[j];
          const bool desc = (i & size) == 0;
          if (desc ? (a < b) : (a > b)) { s_cand[i] = b; s_cand[j] = a; }
        }
      }
      __syncthreads();
    }
  }
  auto value_of = [](unsigned long long w) {
    unsigned u = (unsigned)(w >> 32);
    u = (u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u;
    return __uint_as_float(u);
  };
  const float maxv = value_of(s_cand[0]);
  for (int i = tid; i < cnt; i += 1024) s_p[i] = exp((double)__fsub_rn(value_of(s_cand[i]), maxv));
  __syncthreads();
  if (tid == 0) {
    double sum = 0.0;
    for (int i = 0; i < cnt; i++) sum += s_p[i];
    const double r = u01 * sum;
    double acc = 0.0;
    int pick = cnt - 1;
    for (int i = 0; i < cnt; i++) { acc += s_p[i]; if (r <= acc) { pick = i; break; } }
    *out = (int)(0xFFFFFFFFu - (unsigned)(s_cand[pick] & 0xFFFFFFFFull));
  }
}
int wv_launch_topk_sample(const float* d_logits, int n, int k, float temperature, double u01, int* d_out, cudaStream_t st) {
  topk_sample_kernel<<<1, 1024, 0, st>>>(d_logits, n, k, temperature, u01, d_out);
  return cudaGetLastError() == cudaSuccess ? WV_OK : WV_ECUDA;
}
