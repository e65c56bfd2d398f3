/*
 * welvet_cuda.h — C ABI of libwelvet_cuda.so, the sm_100a backend for Welvet's Dense MatVec.
 *
 * Plain pointers and sizes only; this is what a cgo package (or ctypes) binds. Each entry
 * names the reference interface it stands in for (paths inside openfluke/welvet). The
 * reference has no plugin registry: a backend is a set of exported functions shaped like
 * the WebGPU resident-weight cache (webgpu/affine_cache.go) plus a dispatch case in
 * layers/dense/dense.go:100-112.
 *
 * Conventions (reference README.md:154 "no fallbacks", webgpu/affine_cache.go:157-203):
 *   - every call returns 0 on success or a negative WV_E* status; wv_last_error() gives the
 *     message for the calling thread. Nothing falls back to the CPU.
 *   - host buffers are copied during the call and never retained (cgo pointer rule).
 *   - a blob is addressed by a caller-chosen 64-bit key; the reference keys its caches by
 *     the address of the *quant.Blob (webgpu/binary_cache.go:198).
 *   - format is a quant.Format value (quant/format.go:9-39); dtype is a core.DType value
 *     (core/dtype.go:15-17) and only matters for FormatNone (1 = f32, 2 = f16, 3 = bf16).
 */
#ifndef WELVET_CUDA_H
#define WELVET_CUDA_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  WV_OK = 0,
  WV_ESHAPE = -1,    /* bad rows/cols/lengths (reference: "size mismatch", quant/helpers.go:94-103) */
  WV_EFORMAT = -2,   /* unknown / unsupported format or dtype (quant.ErrUnsupported, quant/errors.go:17) */
  WV_ENOMEM = -3,    /* device cache budget full (errAffineVRAMFull, webgpu/affine_cache.go:71) */
  WV_ECUDA = -4,     /* CUDA runtime error */
  WV_ETIMEOUT = -5,  /* a bounded device wait ran out */
  WV_ENOTFOUND = -6, /* key not resident */
  WV_EINIT = -7,     /* no usable device (webgpu InitError, webgpu/dense.go:116-125) */
  WV_EARG = -8       /* null pointer / bad argument */
};

/* Session — replaces webgpu.Available / InitError / ensure() (webgpu/dense.go:116-125,177-192). */
int wv_init(int device);           /* bind the library to one CUDA device; idempotent */
int wv_available(void);            /* 1 when a device is bound and usable */
int wv_device_count(void);
const char* wv_last_error(void);   /* thread-local text of the last failure */

/* Resident packed-weight cache — replaces WarmAffineWeight / HasAffineWeight /
 * ClearAffineWeightCache / AffineWeightCacheBytes and their binary / f32 twins
 * (webgpu/affine_cache.go:29-154, webgpu/binary_cache.go, webgpu/f32_cache.go).
 * The arrays are exactly quant.Blob's Raw / Scales / Mins (quant/format.go:110-131);
 * block_weights is Blob.BlockWeights (<= 0: inferred as InferBinaryBlockWeights /
 * InferAffineBlockWeights do, quant/binary_g128.go:79-94, quant/affine_g64.go:95-119).
 * Uploading an existing key is a no-op, as in uploadAffineLocked (affine_cache.go:111-116). */
int wv_blob_upload(uint64_t key, int format, int dtype, int rows, int cols, int block_weights,
                   const void* raw, size_t nraw, const float* scales, size_t ns,
                   const float* mins, size_t nm);
/* Same, from the checkpoint wire form u32 ns | u32 nm | u32 nr | scales | mins | raw
 * (weights.EncodePackedWire / DecodePackedWire, weights/packed_wire.go:30-110; FormatNone
 * wire is the raw element array). */
int wv_blob_upload_wire(uint64_t key, int format, int dtype, int rows, int cols,
                        const void* wire, size_t nwire);
/* Row shard: keeps only rows [rows*rank/world, rows*(rank+1)/world) on this device. The
 * reference shards contiguous row ranges over goroutines the same way
 * (layers/dense/gemv_parallel.go:24-41). The resident blob then has rows_local rows. */
int wv_blob_upload_shard(uint64_t key, int format, int dtype, int rows, int cols, int block_weights,
                         const void* raw, size_t nraw, const float* scales, size_t ns,
                         const float* mins, size_t nm, int rank, int world);
int wv_shard_range(int rows, int rank, int world, int* row_begin, int* row_end);
int wv_blob_has(uint64_t key);     /* 1 / 0 */
int wv_blob_evict(uint64_t key);   /* needed when Store.Pack / Convert replace s.Packed (weights/convert.go:103-124) */
void wv_cache_clear(void);
uint64_t wv_cache_bytes(void);     /* device bytes held by resident blobs */
void wv_cache_set_limit(uint64_t bytes); /* 0 = no limit; beyond it uploads return WV_ENOMEM */
/* rows, cols as resident (local rows for a shard), packed wire bytes, device bytes, and
 * whether the chunked kernels apply (0 = ragged shape path). Any out pointer may be NULL. */
int wv_blob_info(uint64_t key, int* rows, int* cols, uint64_t* wire_bytes, uint64_t* dev_bytes, int* chunked);

/* y[batch, out] = x[batch, in] . W^T — replaces dense.MatVecPackedBlob (layers/dense/simd.go:571-614),
 * dense.MatVecWebGPU (layers/dense/webgpu.go:36-48) and the GEMV inside dense.Forward.
 * Host pointers, synchronous, like the reference's device path (affine_cache.go:370-445).
 * Checks in == cols and out == rows (dense.dims, layers/dense/dense.go:129-143). */
int wv_matvec(uint64_t key, const float* x, float* y, int batch, int in, int out);
/* Device pointers, asynchronous on `stream` (a cudaStream_t; NULL = default stream). For
 * chained decode and for benchmarking with inputs resident in HBM. */
int wv_matvec_dev(uint64_t key, const float* dx, float* dy, int batch, int in, int out, void* stream);

/* Several matrices that share x in one launch — the reference's fused projection groups: Q|K|V
 * (fusedgpu/shaders.go:59-157; on the host mha/cpu.go:48-96 runs three dense forwards on one input) and SwiGLU gate|up
 * (fusedgpu/shaders.go:159-222, swiglu/cpu.go:29-52). y_i[batch, out_i] = x[batch, in] . W_i^T for i < n, n <= 4.
 * Matrices of one format, column count and group run as ONE kernel that waits for its predecessor, brings x in and
 * quantises it once; any other mix runs as n launches with the same results. Device pointers, asynchronous. */
int wv_matvec_dev_multi(const uint64_t* keys, int n, const float* dx, float* const* dy, int batch, int in, const int* out,
                        void* stream);

/* Fused epilogues of the grouped launch (batch 1, device pointers, asynchronous).
 * wv_matvec_dev_swiglu: h[out] = silu(W_gate x) * (W_up x), the SwiGLU gate product of swiglu.forwardHost
 * (layers/swiglu/cpu.go:29-52; arithmetic of simd.SiluMulF32, simd/silu.go:14-27: g / (1 + exp(-g)) * u in
 * float64, rounded to f32) inside the gate|up launch, as the reference's fused shader does
 * (fusedgpu/shaders.go:159-222): gate and up are never written out. Both matrices must have `out` rows.
 * wv_matvec_dev_add: y = W x + residual — the projection followed by residualAddInPlace
 * (model/transformer/forward.go:65,75, scratch.go:33-41; fused precedent fusedgpu/hybrid_shaders.go:82);
 * dy may alias dresidual (h += W x).
 * Shapes the grouped kernel does not take run as separate launches with the same results. */
int wv_matvec_dev_swiglu(uint64_t key_gate, uint64_t key_up, const float* dx, float* dh, int in, int out, void* stream);
int wv_matvec_dev_add(uint64_t key, const float* dx, const float* dresidual, float* dy, int in, int out, void* stream);

/* The steps between the projections of a decoder block in single-token decode, on the device, so that
 * activations stay in HBM from one GEMV to the next (the reference runs them on the host in float64).
 * wv_rmsnorm_dev: y[r, i] = x[r, i] * inv_r * gamma[i], inv_r = 1 / sqrt(mean(x_r^2) + eps)
 *   (rmsnorm.forwardHost, layers/rmsnorm/cpu.go:32-90; sum and scale in float64).
 * wv_rope_cache_dev: applyRoPE (layers/mha/rope.go:6-21; pairs (d, d + head_dim/2), angle pos / theta^(2d/head_dim),
 *   float64 trigonometry) on the token's Q [num_heads * head_dim] in place and on its K [num_kv_heads * head_dim],
 *   then K and V go into row pos % max_seq_len of the caches [max_seq_len, num_kv_heads * head_dim]
 *   (forwardHost, layers/mha/cpu.go:184-207). theta <= 0 leaves Q and K unrotated.
 * wv_attn_decode_dev: attnForward (layers/mha/attn.go:15-120) for one query token under the causal mask: softmax
 *   of q.k * scale over cache positions 0 .. kv_len-1 (position p in row p % max_seq_len), grouped-query heads
 *   (head h reads kv head h / (num_heads / num_kv_heads)), out[num_heads * head_dim] = sum w v. head_dim <= 256
 *   and a multiple of 4; no ALiBi, dropout or sigmoid scores. Uses library-owned scratch for split results:
 *   the first call for a larger shape allocates it (make that call before a stream capture) and calls on
 *   different streams must not overlap.
 * wv_silu_mul_dev: out[i] = silu(gate[i]) * up[i] (simd.SiluMulF32, simd/silu.go:7-27).
 * wv_residual_add_dev: dst[i] += add[i] (residualAddInPlace, model/transformer/scratch.go:33-41). */
int wv_rmsnorm_dev(const float* dx, const float* dgamma, float* dy, int rows, int dim, double eps, void* stream);
int wv_rope_cache_dev(float* dq, const float* dk, const float* dv, float* dcache_k, float* dcache_v, int pos, int max_seq_len,
                      int num_heads, int num_kv_heads, int head_dim, double theta, void* stream);
int wv_attn_decode_dev(const float* dq, const float* dcache_k, const float* dcache_v, float* dout, int num_heads, int num_kv_heads,
                       int head_dim, int kv_len, int max_seq_len, float scale, void* stream);
int wv_silu_mul_dev(const float* dgate, const float* dup, float* dout, int n, void* stream);
int wv_residual_add_dev(float* ddst, const float* dadd, int n, void* stream);

/* Greedy pick on the device — sampling.ArgMax (model/sampling/argmax.go:4-18; the reference's fused path does the same
 * in a shader, fusedgpu/shaders.go:471-510): index of the first strict maximum of n device floats, so that the
 * 128256 logits of an LM head need not be read back. wv_argmax_dev writes the index to device memory on `stream`;
 * wv_argmax synchronises and returns it to the host. */
int wv_argmax_dev(const float* d_logits, int n, int* d_index, void* stream);
int wv_argmax(const float* d_logits, int n, int* index_host, void* stream);
/* Top-K sampling with temperature on the device — sampling.SampleTopK (model/sampling/topk.go:11-50): greedy when
 * top_k == 1, temperature <= 0 or `deterministic`; otherwise the top_k largest of logit / temperature (every logit when
 * top_k <= 0 or top_k >= n; at most 1024 candidates, else WV_EARG), softmax weights in float64, and the draw
 * r = u01 * sum walks them from the largest down. The reference draws u01 from math/rand's global source inside the
 * call; here the caller passes it (0 <= u01 <= 1). Equal values, whose order the reference's unstable sort leaves open,
 * go by rising index. */
int wv_topk_sample_dev(const float* d_logits, int n, int top_k, float temperature, int deterministic, double u01,
                       int* d_index, void* stream);
int wv_topk_sample(const float* d_logits, int n, int top_k, float temperature, int deterministic, double u01,
                   int* index_host, void* stream);

/* Dequantise the resident blob to f32 on the device and copy rows*cols floats out —
 * quant.Unpack (quant/unpack.go:4-34); results are bit-identical to it. */
int wv_unpack(uint64_t key, float* out_host);
int wv_unpack_dev(uint64_t key, float* d_out, void* stream);
/* One output row as f32 — quant.DecodeRow (quant/decode_row.go:7-38): the Cols values Unpack gives for `row`
 * (counted within the rows this device holds); WV_ESHAPE when row is out of range or ndst < Cols, as the reference's
 * shape error. The reference refuses FormatNone here (its weights.DecodeRow covers it); this entry takes it too. */
int wv_decode_row(uint64_t key, int row, float* dst_host, int ndst);
int wv_decode_row_dev(uint64_t key, int row, float* d_dst, void* stream);

/* quant.Pack on the device (quant/pack.go:4-31; dense.Layer.Pack, layers/dense/dense.go:84-89):
 * packs rows x cols f32 weights (host pointer) into caller-allocated Raw / Scales / Mins of
 * the sizes wv_pack_sizes reports. Output bytes are identical to the reference packer's. */
int wv_pack_sizes(int format, int dtype, int block_weights, int rows, int cols,
                  size_t* nraw, size_t* ns, size_t* nm);
int wv_pack(int format, int dtype, int block_weights, const float* w, int rows, int cols,
            void* raw, float* scales, float* mins);
/* Device-side variant: d_w is a device pointer; the packed blob stays on the device and is
 * registered under `key` without a host round trip. */
int wv_pack_upload_dev(uint64_t key, int format, int dtype, int block_weights, const float* d_w,
                       int rows, int cols, void* stream);

/* No counterpart in the reference. wv_matvec_dev for callers that can no longer allocate
 * device memory (a serving process that has committed all of HBM to its own pools, or a decode
 * loop that cannot take the device-wide synchronisation of cudaMalloc): batch-1 y = W x with the
 * activation scratch in a fixed array inside the library instead of the cudaMalloc'ed arena.
 * The call performs no allocation. Limits: packed integer-code formats (not IQ4_NL, not
 * FormatNone), chunk-aligned shapes, in <= 32768 columns (else WV_ESHAPE). The first call on a
 * device resolves the array's address and should come before any stream capture. All calls
 * share the array: calls that overlap on the GPU race — keep them on one stream. */
int wv_matvec_dev_static(uint64_t key, const float* dx, float* dy, int in, int out, void* stream);

/* Row-sharded GEMV whose epilogue is the gather: no counterpart call in the reference, where the
 * goroutines of gemvPackedParallelF32 write disjoint row ranges of one y (layers/dense/gemv_parallel.go:24-41).
 * Here every rank keeps rows [row_offset, row_offset + out_local) of the matrix resident (wv_blob_upload_shard) and
 * the kernel stores each of its output rows into all `world` output vectors — its own and the peers' ones mapped
 * into this process — so that every rank holds the whole y when all ranks' kernels have finished; there is no
 * collective call and no extra launch on the bulk-copy kernels. y_all[r] is rank r's vector as addressable from
 * this process (y_all[rank] is the local one); batch 1. The caller orders "all ranks finished" itself (a
 * barrier between steps, or stream-ordered events), as it would around any collective. */
int wv_matvec_dev_gather(uint64_t key, const float* dx, float* const* y_all, int world, int rank, int row_offset,
                         int in, int out_local, void* stream);
/* The sharded form of the grouped and fused launches: n <= 4 matrices of one format and column count share x; this
 * rank keeps rows [row_offset[i], row_offset[i] + out_local[i]) of matrix i resident, and y_all[i * world + r] is rank
 * r's vector for output i as addressable from this process (world == 1: the local vectors). mode 0: y_i = W_i x
 * (Q|K|V); mode 1: n == 2, gate | up, the one output is h = silu(W_0 x) * (W_1 x) in the vectors of output 1 (those
 * of output 0 may be NULL), so only h crosses NVLink. dresidual (n == 1, may be NULL) is a whole-length
 * vector indexed like the outputs; this rank adds its own rows of it before storing them. Ordering between ranks as for
 * wv_matvec_dev_gather. */
int wv_matvec_dev_group_gather(const uint64_t* keys, int n, const float* dx, float* const* y_all, int world, int rank,
                               const int* row_offset, int in, const int* out_local, int mode, const float* dresidual, void* stream);
/* Everything the grouped launch can fuse, in one descriptor (the entries above are special cases of it): n <= 4
 * matrices of one format and column count on a shared x; optionally x is RMS-normalised on its way in
 * (dnorm_gamma non-NULL: x_j / sqrt(mean(x^2) + norm_eps) * gamma_j in float64, layers/rmsnorm/cpu.go:32-90 — the norm's
 * own launch and its output vector disappear); mode 1 applies the SwiGLU gate product (swiglu/cpu.go:29-52); dresidual adds
 * a residual (model/transformer/forward.go:65,75); world > 1 stores every row into all ranks' vectors. The reference
 * fuses the same steps in its WGSL shaders (fusedgpu/shaders.go:59-222, hybrid_shaders.go:82). Fields as in
 * wv_matvec_dev_group_gather; with world == 1 y_all holds the n local vectors and row_offset may be NULL. */
typedef struct WvFusedCall {
  const uint64_t* keys; int n;
  const float* dx;
  float* const* y_all; int world, rank;
  const int* row_offset; int in; const int* out_local;
  int mode;
  const float* dresidual;
  const float* dnorm_gamma; double norm_eps;
} WvFusedCall;
int wv_matvec_dev_fused(const WvFusedCall* call, void* stream);
/* Plumbing for the vectors above (cudaMalloc + cudaIpcGetMemHandle / cudaIpcOpenMemHandle with lazy peer
 * access): allocate an exportable device buffer and its 64-byte handle; map a peer's handle; unmap; free. */
int wv_gather_alloc(size_t bytes, void** dptr, unsigned char handle[64]);
int wv_gather_open(const unsigned char handle[64], void** dptr);
int wv_gather_close(void* dptr);
int wv_gather_free(void* dptr);
/* Arrival flags for chained steps, so that a step's consumers need no host barrier: each rank owns a flag buffer of
 * world + 2 unsigned words (wv_gather_alloc, zero-filled; mapped by the peers like the output vectors).
 * wv_gather_signal, enqueued after this rank's gather GEMVs of a step, bumps this rank's step counter and stores it
 * into word `rank` of every rank's flags (after a system-scope fence: the rows written before it are visible first).
 * wv_gather_wait, enqueued before the kernels that read y, bumps the local wait counter and holds the stream until all
 * `world` words have reached it. The wait is bounded (a fraction of a second): when it runs out the kernel records a code,
 * returns, and wv_device_status() reports WV_ETIMEOUT; the context stays usable. Both are plain kernels and keep their
 * counters on the device, so a captured graph can be replayed. A rank that has passed the wait of step k may already
 * store rows of step k + 1 while a slower rank still reads step k: alternate two sets of output vectors between steps. */
int wv_gather_signal(unsigned* const* flags_all, int world, int rank, void* stream);
int wv_gather_wait(unsigned* flags_own, int world, void* stream);
/* Both in one launch, for a step whose consumers follow immediately: signal as wv_gather_signal does, then wait as
 * wv_gather_wait does (same counters, same bound on the wait). */
int wv_gather_sync(unsigned* const* flags_all, int world, int rank, void* stream);
/* Copy `bytes` from a gather buffer (own or mapped) to host memory after synchronising `stream`. */
int wv_gather_read(const void* dptr, size_t offset_bytes, void* host, size_t bytes, void* stream);

/* After the caller has synchronised its stream: 0, or WV_ETIMEOUT when a bounded device wait
 * of an asynchronous call (wv_matvec_dev) ran out since the last query. The reference reports
 * device failures through the error of the synchronous call (webgpu/affine_cache.go:439-443). */
int wv_device_status(void);

#ifdef __cplusplus
}
#endif
#endif
