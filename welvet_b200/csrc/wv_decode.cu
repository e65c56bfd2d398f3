// The host-ALU steps that sit between the Dense GEMVs of a decoder block in single-token decode,
// on the device, so that activations never leave HBM between projections: RMSNorm, rotary
// position embedding with the KV-cache write, grouped-query attention over the cache, the SwiGLU
// gate product and the residual add. The reference runs all of them in float64 on the host
// (layers/rmsnorm/cpu.go:32-90, layers/mha/rope.go:6-21, layers/mha/cpu.go:184-207,
// layers/mha/attn.go:15-120, simd/silu.go:14-27, model/transformer/scratch.go:33-41); here sums that
// decide a normalisation are kept in float64 and the rest is float32.
#include "wv_common.cuh"
#include <math.h>

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
// One CTA per (query head, split of the positions); the splits' partial results {max, sum, acc[head_dim]}
// are merged by the last split to finish (a counter per head, no waiting). head_dim <= 256, multiple of 4.
#define ATT_THREADS 256
#define ATT_MAX_CHUNK 4096   // positions per split held in shared memory
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const float* __restrict__ q, const float* __restrict__ cache_k,
                                                                  const float* __restrict__ cache_v, float* __restrict__ out,
                                                                  float* __restrict__ part, unsigned* __restrict__ counters,
                                                                  int num_heads, int num_kv_heads, int head_dim, int kv_len, int msl,
                                                                  float scale, int nsplit) {
  __shared__ float s_score[ATT_MAX_CHUNK];
  __shared__ float s_red[ATT_THREADS / 32];
  __shared__ float s_acc[ATT_THREADS / 32][256];
  __shared__ float s_bcast[2];
  __shared__ unsigned s_last;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int h = blockIdx.x, sp = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = ATT_THREADS / 32;
  const int kvh = h / (num_heads / num_kv_heads);
  const int kv_dim = num_kv_heads * head_dim;
  const int per = (kv_len + nsplit - 1) / nsplit;
  const int p0 = sp * per, p1 = min(kv_len, p0 + per);
  const int n = max(0, p1 - p0);
  const int vec = head_dim >> 2;           // float4 per row; lanes beyond it idle
  const float* qh = q + (size_t)h * head_dim;
  float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), qv2 = qv;
  if (lane < vec) qv = reinterpret_cast<const float4*>(qh)[lane];
  if (lane + 32 < vec) qv2 = reinterpret_cast<const float4*>(qh)[lane + 32];
  // scores of this split's positions, one warp per position
  float lmax = -3.0e38f;
  for (int i = warp; i < n; i += nwarp) {
    const float4* kr = reinterpret_cast<const float4*>(cache_k + (size_t)((p0 + i) % msl) * kv_dim + (size_t)kvh * head_dim);
    float d = 0.f;
    if (lane < vec) { const float4 kk = kr[lane]; d = qv.x * kk.x + qv.y * kk.y + qv.z * kk.z + qv.w * kk.w; }
    if (lane + 32 < vec) { const float4 kk = kr[lane + 32]; d += qv2.x * kk.x + qv2.y * kk.y + qv2.z * kk.z + qv2.w * kk.w; }
#pragma unroll
    for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    d *= scale;
    if (lane == 0) s_score[i] = d;
    lmax = fmaxf(lmax, d);
  }
  if (lane == 0) s_red[warp] = lmax;
  __syncthreads();
  if (tid == 0) { float m = s_red[0]; for (int w = 1; w < nwarp; w++) m = fmaxf(m, s_red[w]); s_bcast[0] = m; }
  __syncthreads();
  const float m = s_bcast[0];
  float lsum = 0.f;
  for (int i = tid; i < n; i += ATT_THREADS) { const float e = __expf(s_score[i] - m); s_score[i] = e; lsum += e; }
#pragma unroll
  for (int o = 16; o; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
  if (lane == 0) s_red[warp] = lsum;
  __syncthreads();
  if (tid == 0) { float t = 0.f; for (int w = 0; w < nwarp; w++) t += s_red[w]; s_bcast[1] = t; }
  // weighted sum of the V rows: a warp walks its positions, a lane keeps its 4 (+4) dimensions
  float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
  for (int i = warp; i < n; i += nwarp) {
    const float w = s_score[i];
    const float4* vr = reinterpret_cast<const float4*>(cache_v + (size_t)((p0 + i) % msl) * kv_dim + (size_t)kvh * head_dim);
    if (lane < vec) { const float4 vv = vr[lane]; a0.x += w * vv.x; a0.y += w * vv.y; a0.z += w * vv.z; a0.w += w * vv.w; }
    if (lane + 32 < vec) { const float4 vv = vr[lane + 32]; a1.x += w * vv.x; a1.y += w * vv.y; a1.z += w * vv.z; a1.w += w * vv.w; }
  }
  if (lane < vec) { float* d = &s_acc[warp][lane * 4]; d[0] = a0.x; d[1] = a0.y; d[2] = a0.z; d[3] = a0.w; }
  if (lane + 32 < vec) { float* d = &s_acc[warp][(lane + 32) * 4]; d[0] = a1.x; d[1] = a1.y; d[2] = a1.z; d[3] = a1.w; }
  __syncthreads();
  const float ssum = s_bcast[1];
  // this split's record: [0] max, [1] sum, [2 ..] unnormalised accumulators
  float* rec = part + ((size_t)h * nsplit + sp) * (head_dim + 2);
  if (tid < head_dim) {
    float t = 0.f;
    for (int w = 0; w < nwarp; w++) t += s_acc[w][tid];
    if (nsplit == 1) { out[(size_t)h * head_dim + tid] = n > 0 ? t / ssum : 0.f; }
    else rec[2 + tid] = t;
  }
  if (nsplit == 1) return;
  if (tid == 0) { rec[0] = n > 0 ? m : -3.0e38f; rec[1] = n > 0 ? ssum : 0.f; }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(&counters[h], 1u);
    s_last = (prev == (unsigned)nsplit - 1u);
    if (s_last) counters[h] = 0u;   // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // merge in split order (fixed order: the result does not depend on which split finished last)
  const float* base = part + (size_t)h * nsplit * (head_dim + 2);
  float gm = -3.0e38f;
  for (int s = 0; s < nsplit; s++) gm = fmaxf(gm, __ldcg(base + (size_t)s * (head_dim + 2)));
  if (tid < head_dim) {
    float tot = 0.f, acc = 0.f;
    for (int s = 0; s < nsplit; s++) {
      const float* r = base + (size_t)s * (head_dim + 2);
      const float f = __expf(__ldcg(r) - gm);
      tot += f * __ldcg(r + 1);
      acc += f * __ldcg(r + 2 + tid);
    }
    out[(size_t)h * head_dim + tid] = tot > 0.f ? acc / tot : 0.f;
  }
}

// Scratch of the split merge: nsplit records per head and one counter per head, owned by the library.
static float* g_att_part = nullptr;
static unsigned* g_att_cnt = nullptr;
static size_t g_att_part_floats = 0;
static int g_att_heads = 0;

int wv_launch_attn_decode(const float* dq, const float* dcache_k, const float* dcache_v, float* dout, int num_heads, int num_kv_heads,
                          int head_dim, int kv_len, int msl, float scale, cudaStream_t st) {
  if (head_dim > 256 || (head_dim & 3) || num_heads % num_kv_heads) { wv_set_error("attention: head_dim %d / heads %d:%d not supported", head_dim, num_heads, num_kv_heads); return WV_ESHAPE; }
  // splits: enough CTAs to fill the SMs, each holding at most ATT_MAX_CHUNK positions
  int nsplit = 1;
  while (nsplit < 16 && (num_heads * nsplit < 128 || (kv_len + nsplit - 1) / nsplit > ATT_MAX_CHUNK) && kv_len / (nsplit * 2) >= 64) nsplit *= 2;
  while ((kv_len + nsplit - 1) / nsplit > ATT_MAX_CHUNK) nsplit *= 2;
  if (nsplit > 1024) { wv_set_error("attention: kv_len %d too long", kv_len); return WV_ESHAPE; }
  const size_t need = (size_t)num_heads * nsplit * (head_dim + 2);
  if (need > g_att_part_floats || num_heads > g_att_heads) {
    // grows only when a larger shape arrives (set-up time: not capturable)
    cudaStreamSynchronize(st);
    if (g_att_part) cudaFree(g_att_part);
    if (g_att_cnt) cudaFree(g_att_cnt);
    g_att_part = nullptr; g_att_cnt = nullptr;
    const size_t want = need * 2;
    const int heads = num_heads > 256 ? num_heads : 256;
    if (cudaMalloc(&g_att_part, want * 4) != cudaSuccess || cudaMalloc(&g_att_cnt, (size_t)heads * 4) != cudaSuccess) { cudaGetLastError(); wv_set_error("attention: scratch allocation failed"); return WV_ENOMEM; }
    cudaMemset(g_att_cnt, 0, (size_t)heads * 4);
    g_att_part_floats = want; g_att_heads = heads;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_heads, nsplit); cfg.blockDim = dim3(ATT_THREADS); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, attn_decode_kernel, dq, dcache_k, dcache_v, dout, g_att_part, g_att_cnt, num_heads, num_kv_heads, head_dim,
                            kv_len, msl, scale, nsplit) == cudaSuccess ? WV_OK : WV_ECUDA;
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
