// C ABI of libwelvet_cuda.so (see include/welvet_cuda.h): session, resident packed-weight
// cache and the MatVec / Unpack / Pack entry points. Modelled on the reference's WebGPU
// resident caches (webgpu/affine_cache.go): one mutex around the key -> entry map, uploads
// idempotent per key, dispatch outside the lock, hard errors and no host fallback.
#include "wv_common.cuh"
#include "wv_gemv_common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <unordered_map>
#include <vector>

// ---------------------------------------------------------------- errors
static thread_local char t_err[512] = "";
void wv_set_error(const char* fmt, ...) {
  va_list ap; va_start(ap, fmt); vsnprintf(t_err, sizeof t_err, fmt, ap); va_end(ap);
}
extern "C" const char* wv_last_error(void) { return t_err; }

#define CUDA_TRY(expr)                                                                     \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess) {                                                              \
      wv_set_error("%s: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__);  \
      return WV_ECUDA;                                                                     \
    }                                                                                      \
  } while (0)

// ---------------------------------------------------------------- session
int wv_gemv_scratch_init(size_t bytes);  // wv_gemv.cu
int wv_tma_init();                       // wv_gemv_tma.cu
int wv_tma_take_error();
struct Entry {
  WvDevBlob blob;
  void* mem = nullptr;
  size_t dev_bytes = 0, wire_bytes = 0;
  uint64_t gen = 0;       // upload generation: tells a re-uploaded key from the blob a cached launch graph was built for
};
static std::atomic<uint64_t> g_upload_gen{0};
static std::mutex g_mu;                // guards the map and the byte counters
static std::unordered_map<uint64_t, Entry> g_cache;
static uint64_t g_cache_bytes = 0, g_cache_limit = 0;
static int g_device = -1;
static cudaStream_t g_stream = nullptr;

extern "C" int wv_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

extern "C" int wv_init(int device) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_device >= 0) {
    if (device == g_device || device < 0) return WV_OK;
    wv_set_error("wv_init: already bound to device %d", g_device);
    return WV_EINIT;
  }
  int n = wv_device_count();
  if (n <= 0) { wv_set_error("wv_init: no CUDA device"); return WV_EINIT; }
  if (device < 0) device = 0;
  if (device >= n) { wv_set_error("wv_init: device %d of %d", device, n); return WV_EINIT; }
  cudaDeviceProp prop;
  CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    wv_set_error("wv_init: device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major, prop.minor);
    return WV_EINIT;
  }
  CUDA_TRY(cudaSetDevice(device));
  CUDA_TRY(cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking));
  {
    size_t mb = 32;
    if (const char* e = getenv("WELVET_CUDA_SCRATCH_MB")) { long v = atol(e); if (v > 0) mb = (size_t)v; }
    if (wv_gemv_scratch_init(mb << 20) != WV_OK) { wv_set_error("wv_init: cannot allocate %zu MB of activation scratch", mb); return WV_ENOMEM; }
  }
  if (wv_tma_init() != WV_OK) { wv_set_error("wv_init: cannot allocate the device status word"); return WV_ENOMEM; }
  g_device = device;
  return WV_OK;
}
extern "C" int wv_available(void) { return g_device >= 0 ? 1 : 0; }

static int ensure_init() {
  if (g_device < 0) { wv_set_error("welvet_cuda: wv_init has not bound a device"); return WV_EINIT; }
  cudaSetDevice(g_device);
  return WV_OK;
}

// For entry points implemented in other files: the library's device becomes current on the calling
// thread; returns its index, or WV_EINIT.
int wv_api_bind_device() {
  const int rc = ensure_init();
  return rc ? rc : g_device;
}

// ---------------------------------------------------------------- sizes
struct Sizes { size_t nraw, ns, nm; int group; long long npad; };

// Lengths the reference packers produce (quant/*.go) and the padded weight count.
static int expected_sizes(int format, int dtype, int bw, int rows, int cols, Sizes* s) {
  if (rows <= 0 || cols <= 0) { wv_set_error("bad shape rows=%d cols=%d", rows, cols); return WV_ESHAPE; }
  const long long n = (long long)rows * cols;
  const WvFmtInfo fi = wv_fmt_info(format);
  s->nraw = s->ns = s->nm = 0; s->group = fi.pgroup; s->npad = n;
  switch (fi.kind) {
  case WK_NONE:
    if (format != WV_NONE) { wv_set_error("unknown format %d", format); return WV_EFORMAT; }
    if (dtype != WV_DT_F32 && dtype != WV_DT_F16 && dtype != WV_DT_BF16) {
      wv_set_error("FormatNone dtype %d not supported (f32, f16, bf16 only)", dtype);
      return WV_EFORMAT;
    }
    s->nraw = (size_t)n * (dtype == WV_DT_F32 ? 4 : 2); s->group = 1;
    return WV_OK;
  case WK_CLASSIC: { long long nb = (n + 31) / 32; s->nraw = (size_t)nb * fi.wire_block; s->npad = nb * 32; return WV_OK; }
  case WK_KQUANT: { long long nsb = (n + 255) / 256; s->nraw = (size_t)nsb * fi.wire_block; s->npad = nsb * 256; return WV_OK; }
  case WK_IQ: {
    long long padn = (n + fi.pgroup - 1) / fi.pgroup * fi.pgroup;
    s->ns = (size_t)(padn / fi.pgroup); s->nraw = (size_t)((padn * (fi.bits_lo + fi.bits_hi) + 7) / 8); s->npad = padn;
    return WV_OK;
  }
  case WK_TERNARY: { long long ng = (n + 15) / 16; s->ns = (size_t)ng; s->nraw = (size_t)ng * 4; s->npad = ng * 16; return WV_OK; }
  case WK_BINARY:
    if (bw == 128) {
      if (cols % 128) { wv_set_error("binary g128 needs cols %% 128 == 0 (cols=%d)", cols); return WV_ESHAPE; }
      s->group = 128; s->ns = (size_t)rows * (cols / 128); s->nraw = (size_t)rows * (cols / 32) * 4;
    } else {
      long long ng = (n + 31) / 32; s->group = 32; s->ns = (size_t)ng; s->nraw = (size_t)ng * 4; s->npad = ng * 32;
    }
    return WV_OK;
  case WK_AFFINE: {
    int g = bw > 0 ? bw : 64;
    if (cols % 8 || cols % g || g % 8) { wv_set_error("affine needs cols %% 8 == 0 and cols %% group == 0 (cols=%d group=%d)", cols, g); return WV_ESHAPE; }
    s->group = g; s->ns = s->nm = (size_t)rows * (cols / g); s->nraw = (size_t)rows * (cols / 8) * 4;
    return WV_OK;
  }
  }
  return WV_EFORMAT;
}

extern "C" int wv_pack_sizes(int format, int dtype, int block_weights, int rows, int cols, size_t* nraw, size_t* ns, size_t* nm) {
  Sizes s;
  int rc = expected_sizes(format, dtype, block_weights, rows, cols, &s);
  if (rc) return rc;
  if (nraw) *nraw = s.nraw;
  if (ns) *ns = s.ns;
  if (nm) *nm = s.nm;
  return WV_OK;
}

// BlockWeights re-inference for blobs that lost it on the wire (DecodePackedWire drops it).
static int infer_block_weights(int format, int rows, int cols, int bw, size_t ns) {
  if (format == WV_BINARY) {  // quant/binary_g128.go:79-94
    if (bw == 128 || bw == 32) return bw;
    if (cols > 0 && cols % 128 == 0 && ns == (size_t)rows * (cols / 128)) return 128;
    return 32;
  }
  if (format == WV_AFFINE) {  // quant/affine_g64.go:95-119
    if (bw > 0 && cols % bw == 0 && ns == (size_t)rows * (cols / bw)) return bw;
    if (cols % 64 == 0 && ns == (size_t)rows * (cols / 64)) return 64;
    if (rows > 0 && ns % rows == 0) { size_t gpr = ns / rows; if (gpr > 0 && cols % gpr == 0) return (int)(cols / gpr); }
    return bw > 0 ? bw : 64;
  }
  return bw;
}

// ---------------------------------------------------------------- upload
static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Plan { size_t lo, hi, p0, p1, km, total; };
static Plan plan_layout(const WvFmtInfo& fi, int dtype, const Sizes& s, long long nchunks) {
  Plan p{};
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align256(off + bytes); return o; };
  if (fi.kind == WK_NONE) { p.lo = take(s.nraw + 16); p.total = off; return p; }
  p.lo = take((size_t)nchunks * fi.bits_lo * 4);
  p.hi = fi.bits_hi ? take((size_t)nchunks * fi.bits_hi * 4) : 0;
  if (fi.kind == WK_CLASSIC) { p.p0 = take((size_t)nchunks * 4); p.p1 = fi.has_min ? take((size_t)nchunks * 4) : 0; }
  else if (fi.kind == WK_KQUANT) { p.p0 = take((size_t)((nchunks + 7) / 8) * 8); p.km = take((size_t)nchunks * (fi.has_min ? 4 : 2)); }
  else { p.p0 = take((s.ns + 2) * 4); p.p1 = s.nm ? take((s.nm + 2) * 4) : 0; }
  p.total = off;
  return p;
}

static int upload_locked_free(uint64_t key, int format, int dtype, int rows, int cols, int bw,
                              const void* raw, size_t nraw, const float* scales, size_t ns,
                              const float* mins, size_t nm) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!raw) { wv_set_error("wv_blob_upload: null raw"); return WV_EARG; }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_cache.count(key)) return WV_OK;  // idempotent per key
  }
  const WvFmtInfo fi = wv_fmt_info(format);
  bw = infer_block_weights(format, rows, cols, bw, ns);
  Sizes s;
  rc = expected_sizes(format, dtype, bw, rows, cols, &s);
  if (rc) return rc;
  const bool side_arrays = fi.kind == WK_IQ || fi.kind == WK_TERNARY || fi.kind == WK_BINARY || fi.kind == WK_AFFINE;
  if (nraw < s.nraw || (side_arrays && (ns < s.ns || nm < s.nm || (s.ns && !scales) || (s.nm && !mins)))) {
    wv_set_error("wv_blob_upload: short buffers for format %d %dx%d: raw %zu/%zu scales %zu/%zu mins %zu/%zu",
                 format, rows, cols, nraw, s.nraw, ns, s.ns, nm, s.nm);
    return WV_ESHAPE;
  }
  const long long nchunks = fi.kind == WK_NONE ? 0 : (s.npad + 31) / 32;
  const Plan p = plan_layout(fi, dtype, s, nchunks);
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_cache_limit && g_cache_bytes + p.total > g_cache_limit) {
      wv_set_error("wv_blob_upload: device weight budget full (%llu + %zu > %llu bytes)",
                   (unsigned long long)g_cache_bytes, p.total, (unsigned long long)g_cache_limit);
      return WV_ENOMEM;
    }
  }
  unsigned char* mem = nullptr;
  cudaError_t ce = cudaMalloc(&mem, p.total);
  if (ce != cudaSuccess) {
    cudaGetLastError();
    wv_set_error("wv_blob_upload: cudaMalloc(%zu): %s", p.total, cudaGetErrorString(ce));
    return WV_ENOMEM;
  }
  Entry e;
  e.mem = mem; e.dev_bytes = p.total; e.wire_bytes = s.nraw + 4 * s.ns + 4 * s.nm;
  WvDevBlob& b = e.blob;
  b.format = format; b.dtype = dtype; b.rows = rows; b.cols = cols; b.group = s.group > 0 ? s.group : 1;
  b.n = (long long)rows * cols; b.nchunks = nchunks;
  b.lo = reinterpret_cast<uint32_t*>(mem + p.lo);
  b.hi = fi.bits_hi ? reinterpret_cast<uint32_t*>(mem + p.hi) : nullptr;
  b.p0 = fi.kind != WK_NONE ? reinterpret_cast<float*>(mem + p.p0) : nullptr;
  b.p1 = p.p1 ? reinterpret_cast<float*>(mem + p.p1) : nullptr;
  b.km = p.km ? reinterpret_cast<uint32_t*>(mem + p.km) : nullptr;
  if (fi.kind == WK_NONE) b.fast = (cols % 8 == 0);
  else if (fi.kind == WK_AFFINE || fi.kind == WK_BINARY) b.fast = (cols % 32 == 0) && (s.group % 32 == 0);
  else b.fast = (cols % 32 == 0);

  auto fail = [&](int code) { cudaFree(mem); return code; };
  if (fi.kind == WK_NONE) {
    if (cudaMemcpyAsync(mem + p.lo, raw, s.nraw, cudaMemcpyHostToDevice, g_stream) != cudaSuccess) { wv_set_error("upload copy failed"); return fail(WV_ECUDA); }
  } else {
    unsigned char* tmp = nullptr;
    if (cudaMalloc(&tmp, s.nraw + 16) != cudaSuccess) { cudaGetLastError(); wv_set_error("wv_blob_upload: staging cudaMalloc(%zu) failed", s.nraw); return fail(WV_ENOMEM); }
    bool ok = cudaMemcpyAsync(tmp, raw, s.nraw, cudaMemcpyHostToDevice, g_stream) == cudaSuccess;
    if (ok && side_arrays) {
      ok = cudaMemsetAsync(mem + p.p0, 0, (s.ns + 2) * 4, g_stream) == cudaSuccess &&
           cudaMemcpyAsync(mem + p.p0, scales, s.ns * 4, cudaMemcpyHostToDevice, g_stream) == cudaSuccess;
      if (ok && s.nm) ok = cudaMemcpyAsync(mem + p.p1, mins, s.nm * 4, cudaMemcpyHostToDevice, g_stream) == cudaSuccess;
    }
    if (ok) ok = wv_launch_relayout(b, tmp, s.nraw, g_stream) == WV_OK;
    cudaError_t se = cudaStreamSynchronize(g_stream);
    cudaFree(tmp);
    if (!ok || se != cudaSuccess) { wv_set_error("wv_blob_upload: device re-layout failed: %s", cudaGetErrorString(se)); return fail(WV_ECUDA); }
  }
  if (cudaStreamSynchronize(g_stream) != cudaSuccess) { wv_set_error("upload sync failed"); return fail(WV_ECUDA); }
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_cache.count(key)) { cudaFree(mem); return WV_OK; }
  e.gen = ++g_upload_gen;
  g_cache[key] = e;
  g_cache_bytes += p.total;
  return WV_OK;
}

extern "C" int wv_blob_upload(uint64_t key, int format, int dtype, int rows, int cols, int block_weights,
                              const void* raw, size_t nraw, const float* scales, size_t ns,
                              const float* mins, size_t nm) {
  return upload_locked_free(key, format, dtype, rows, cols, block_weights, raw, nraw, scales, ns, mins, nm);
}

extern "C" int wv_blob_upload_wire(uint64_t key, int format, int dtype, int rows, int cols, const void* wire, size_t n) {
  if (!wire) { wv_set_error("wv_blob_upload_wire: null wire"); return WV_EARG; }
  const unsigned char* w = static_cast<const unsigned char*>(wire);
  if (format == WV_NONE) return upload_locked_free(key, format, dtype, rows, cols, 1, w, n, nullptr, 0, nullptr, 0);
  if (n < 12) { wv_set_error("packed wire too short (%zu bytes)", n); return WV_ESHAPE; }
  uint32_t ns, nm, nr;
  memcpy(&ns, w, 4); memcpy(&nm, w + 4, 4); memcpy(&nr, w + 8, 4);
  size_t need = 12 + (size_t)ns * 4 + (size_t)nm * 4 + nr;
  if (n < need) { wv_set_error("packed wire truncated (need %zu, have %zu)", need, n); return WV_ESHAPE; }
  // float arrays sit at offset 12: 4-byte aligned when the wire buffer is; copy if not.
  std::vector<float> sc(ns), mn(nm);
  if (ns) memcpy(sc.data(), w + 12, (size_t)ns * 4);
  if (nm) memcpy(mn.data(), w + 12 + (size_t)ns * 4, (size_t)nm * 4);
  return upload_locked_free(key, format, dtype, rows, cols, 0, w + 12 + (size_t)ns * 4 + (size_t)nm * 4, nr,
                            sc.data(), ns, mn.data(), nm);
}

extern "C" int wv_shard_range(int rows, int rank, int world, int* row_begin, int* row_end) {
  if (world <= 0 || rank < 0 || rank >= world || rows < 0) { wv_set_error("wv_shard_range: rank %d of %d", rank, world); return WV_EARG; }
  if (row_begin) *row_begin = (int)((long long)rows * rank / world);
  if (row_end) *row_end = (int)((long long)rows * (rank + 1) / world);
  return WV_OK;
}

extern "C" int wv_blob_upload_shard(uint64_t key, int format, int dtype, int rows, int cols, int bw,
                                    const void* raw, size_t nraw, const float* scales, size_t ns,
                                    const float* mins, size_t nm, int rank, int world) {
  int r0, r1;
  int rc = wv_shard_range(rows, rank, world, &r0, &r1);
  if (rc) return rc;
  if (r1 <= r0) { wv_set_error("wv_blob_upload_shard: empty shard for rank %d of %d (rows=%d)", rank, world, rows); return WV_ESHAPE; }
  const WvFmtInfo fi = wv_fmt_info(format);
  bw = infer_block_weights(format, rows, cols, bw, ns);
  Sizes full;
  rc = expected_sizes(format, dtype, bw, rows, cols, &full);
  if (rc) return rc;
  if (nraw < full.nraw || ns < full.ns || nm < full.nm) { wv_set_error("wv_blob_upload_shard: short buffers"); return WV_ESHAPE; }
  const long long f0 = (long long)r0 * cols, f1 = (long long)r1 * cols;
  const int bits = fi.bits_lo + fi.bits_hi;
  const unsigned char* rp = static_cast<const unsigned char*>(raw);
  long long unit = 1;
  size_t roff = 0, soff = 0;
  switch (fi.kind) {
  case WK_NONE: roff = (size_t)f0 * (dtype == WV_DT_F32 ? 4 : 2); break;
  case WK_CLASSIC: unit = 32; roff = (size_t)(f0 / 32) * fi.wire_block; break;
  case WK_KQUANT: unit = 256; roff = (size_t)(f0 / 256) * fi.wire_block; break;
  case WK_IQ: unit = fi.pgroup; while ((unit * bits) % 8) unit *= 2; roff = (size_t)(f0 * bits / 8); soff = (size_t)(f0 / fi.pgroup); break;
  case WK_TERNARY: unit = 16; roff = (size_t)(f0 / 16) * 4; soff = (size_t)(f0 / 16); break;
  case WK_BINARY: unit = full.group; roff = (size_t)(f0 / 32) * 4; soff = (size_t)(f0 / full.group); break;
  case WK_AFFINE: unit = full.group; roff = (size_t)(f0 / 8) * 4; soff = (size_t)(f0 / full.group); break;
  }
  if (f0 % unit || (f1 % unit && r1 != rows)) {
    wv_set_error("wv_blob_upload_shard: row range [%d,%d) of %dx%d splits a %lld-weight block", r0, r1, rows, cols, unit);
    return WV_ESHAPE;
  }
  Sizes part;
  rc = expected_sizes(format, dtype, bw, r1 - r0, cols, &part);
  if (rc) return rc;
  return upload_locked_free(key, format, dtype, r1 - r0, cols, bw, rp + roff, part.nraw,
                            part.ns ? scales + soff : nullptr, part.ns,
                            part.nm ? mins + soff : nullptr, part.nm);
}

extern "C" int wv_blob_has(uint64_t key) {
  std::lock_guard<std::mutex> lk(g_mu);
  return g_cache.count(key) ? 1 : 0;
}
// Eviction takes the entry out of the map under the lock and frees it outside: the device-wide
// synchronisation (kernels still reading the blob) and cudaFree must not stall concurrent lookups.
extern "C" int wv_blob_evict(uint64_t key) {
  void* mem = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_cache.find(key);
    if (it == g_cache.end()) { wv_set_error("wv_blob_evict: key %llu not resident", (unsigned long long)key); return WV_ENOTFOUND; }
    mem = it->second.mem;
    g_cache_bytes -= it->second.dev_bytes;
    g_cache.erase(it);
  }
  if (g_device >= 0) { cudaSetDevice(g_device); cudaDeviceSynchronize(); cudaFree(mem); }
  return WV_OK;
}
extern "C" void wv_cache_clear(void) {
  std::vector<void*> mems;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto& kv : g_cache) mems.push_back(kv.second.mem);
    g_cache.clear();
    g_cache_bytes = 0;
  }
  if (g_device >= 0) { cudaSetDevice(g_device); cudaDeviceSynchronize(); }
  for (void* m : mems) cudaFree(m);
}
extern "C" uint64_t wv_cache_bytes(void) { std::lock_guard<std::mutex> lk(g_mu); return g_cache_bytes; }
extern "C" void wv_cache_set_limit(uint64_t bytes) { std::lock_guard<std::mutex> lk(g_mu); g_cache_limit = bytes; }

static int lookup(uint64_t key, Entry* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_cache.find(key);
  if (it == g_cache.end()) { wv_set_error("key %llu not resident", (unsigned long long)key); return WV_ENOTFOUND; }
  *out = it->second;
  return WV_OK;
}

// Copy of a resident blob's descriptor for entry points implemented in other files.
int wv_api_get_blob(uint64_t key, WvDevBlob* out) {
  if (g_device < 0) { wv_set_error("welvet_cuda: wv_init has not bound a device"); return WV_EINIT; }
  Entry e;
  int rc = lookup(key, &e);
  if (rc) return rc;
  *out = e.blob;
  return WV_OK;
}

extern "C" int wv_blob_info(uint64_t key, int* rows, int* cols, uint64_t* wire_bytes, uint64_t* dev_bytes, int* chunked) {
  Entry e;
  int rc = lookup(key, &e);
  if (rc) return rc;
  if (rows) *rows = e.blob.rows;
  if (cols) *cols = e.blob.cols;
  if (wire_bytes) *wire_bytes = e.wire_bytes;
  if (dev_bytes) *dev_bytes = e.dev_bytes;
  if (chunked) *chunked = e.blob.fast;
  return WV_OK;
}

// ---------------------------------------------------------------- matvec
static int check_dims(const Entry& e, int batch, int in, int out) {
  if (batch <= 0 || in != e.blob.cols || out != e.blob.rows) {  // dense.dims, layers/dense/dense.go:129-143
    wv_set_error("matvec: size mismatch rows=%d cols=%d batch=%d in=%d out=%d", e.blob.rows, e.blob.cols, batch, in, out);
    return WV_ESHAPE;
  }
  return WV_OK;
}

extern "C" int wv_matvec_dev(uint64_t key, const float* dx, float* dy, int batch, int in, int out, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dx || !dy) { wv_set_error("wv_matvec_dev: null pointer"); return WV_EARG; }
  Entry e;
  if ((rc = lookup(key, &e))) return rc;
  if ((rc = check_dims(e, batch, in, out))) return rc;
  rc = wv_launch_gemv(e.blob, dx, dy, batch, 0, e.blob.rows, static_cast<cudaStream_t>(stream));
  if (rc) wv_set_error("wv_matvec_dev: launch failed (%d): %s", rc, cudaGetErrorString(cudaGetLastError()));
  return rc;
}

int wv_launch_argmax(const float* d_logits, int n, int* d_out, cudaStream_t st);   // wv_gemv.cu

extern "C" int wv_argmax_dev(const float* d_logits, int n, int* d_index, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!d_logits || !d_index || n < 0) { wv_set_error("wv_argmax_dev: bad argument"); return WV_EARG; }
  return wv_launch_argmax(d_logits, n, d_index, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_argmax(const float* d_logits, int n, int* index_host, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!d_logits || !index_host || n < 0) { wv_set_error("wv_argmax: bad argument"); return WV_EARG; }
  static int* h_idx = nullptr;     // mapped pinned word: the kernel writes the index straight to the host
  static int* d_idx = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  if (!h_idx) {
    if (cudaHostAlloc(&h_idx, sizeof(int), cudaHostAllocMapped) != cudaSuccess || cudaHostGetDevicePointer(&d_idx, h_idx, 0) != cudaSuccess) {
      cudaGetLastError(); h_idx = nullptr; wv_set_error("wv_argmax: no pinned word"); return WV_ENOMEM;
    }
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((rc = wv_launch_argmax(d_logits, n, d_idx, st))) return rc;
  CUDA_TRY(cudaStreamSynchronize(st));
  *index_host = *h_idx;
  return WV_OK;
}

int wv_launch_topk_sample(const float* d_logits, int n, int k, float temperature, double u01, int* d_out, cudaStream_t st);   // wv_decode.cu

// sampling.SampleTopK (model/sampling/topk.go:11-50). Greedy (top_k == 1, temperature <= 0 or `deterministic`)
// is ArgMax; otherwise K = top_k, or every logit when top_k <= 0 or top_k >= n, and K must not exceed 1024.
static int topk_launch(const char* who, const float* d_logits, int n, int top_k, float temperature, int deterministic, double u01,
                       int* d_index, cudaStream_t st) {
  if (n <= 0 || top_k == 1 || !(temperature > 0.0f) || deterministic) return wv_launch_argmax(d_logits, n, d_index, st);
  if (!(u01 >= 0.0 && u01 <= 1.0)) { wv_set_error("%s: the uniform draw must lie in [0, 1]", who); return WV_EARG; }
  const int k = (top_k > 0 && top_k < n) ? top_k : n;
  if (k > 1024) { wv_set_error("%s: %d candidates (top_k = %d over %d logits); the device sampler takes at most 1024", who, k, top_k, n); return WV_EARG; }
  return wv_launch_topk_sample(d_logits, n, k, temperature, u01, d_index, st);
}
extern "C" int wv_topk_sample_dev(const float* d_logits, int n, int top_k, float temperature, int deterministic, double u01,
                                  int* d_index, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!d_logits || !d_index || n < 0) { wv_set_error("wv_topk_sample_dev: bad argument"); return WV_EARG; }
  return topk_launch("wv_topk_sample_dev", d_logits, n, top_k, temperature, deterministic, u01, d_index, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_topk_sample(const float* d_logits, int n, int top_k, float temperature, int deterministic, double u01,
                              int* index_host, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!d_logits || !index_host || n < 0) { wv_set_error("wv_topk_sample: bad argument"); return WV_EARG; }
  static int* h_idx = nullptr;     // mapped pinned word, as in wv_argmax
  static int* d_idx = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  if (!h_idx) {
    if (cudaHostAlloc(&h_idx, sizeof(int), cudaHostAllocMapped) != cudaSuccess || cudaHostGetDevicePointer(&d_idx, h_idx, 0) != cudaSuccess) {
      cudaGetLastError(); h_idx = nullptr; wv_set_error("wv_topk_sample: no pinned word"); return WV_ENOMEM;
    }
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((rc = topk_launch("wv_topk_sample", d_logits, n, top_k, temperature, deterministic, u01, d_idx, st))) return rc;
  CUDA_TRY(cudaStreamSynchronize(st));
  *index_host = *h_idx;
  return WV_OK;
}

extern "C" int wv_matvec_dev_multi(const uint64_t* keys, int n, const float* dx, float* const* dy, int batch, int in, const int* out,
                                   void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!keys || !dx || !dy || !out || n < 1 || n > 4) { wv_set_error("wv_matvec_dev_multi: bad argument (1..4 matrices)"); return WV_EARG; }
  WvDevBlob blobs[4];
  for (int i = 0; i < n; i++) {
    if (!dy[i]) { wv_set_error("wv_matvec_dev_multi: dy[%d] is null", i); return WV_EARG; }
    Entry e;
    if ((rc = lookup(keys[i], &e))) return rc;
    if ((rc = check_dims(e, batch, in, out[i]))) return rc;
    blobs[i] = e.blob;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n > 1 && blobs[0].fast && blobs[0].format != WV_NONE) {
    rc = wv_launch_gemv_tma_group(blobs, n, dx, dy, batch, 0, 0, st);
    if (rc != 1) {
      if (rc) wv_set_error("wv_matvec_dev_multi: launch failed (%d): %s", rc, cudaGetErrorString(cudaGetLastError()));
      return rc;
    }
  }
  for (int i = 0; i < n; i++) {
    rc = wv_launch_gemv(blobs[i], dx, dy[i], batch, 0, blobs[i].rows, st);
    if (rc) { wv_set_error("wv_matvec_dev_multi: launch %d failed (%d): %s", i, rc, cudaGetErrorString(cudaGetLastError())); return rc; }
  }
  return WV_OK;
}

extern "C" int wv_matvec_dev_gather(uint64_t key, const float* dx, float* const* y_all, int world, int rank, int row_offset,
                                    int in, int out_local, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dx || !y_all) { wv_set_error("wv_matvec_dev_gather: null pointer"); return WV_EARG; }
  if (world < 1 || world > WV_MAX_PEERS || rank < 0 || rank >= world || row_offset < 0) {
    wv_set_error("wv_matvec_dev_gather: world=%d rank=%d row_offset=%d (at most %d ranks)", world, rank, row_offset, WV_MAX_PEERS);
    return WV_EARG;
  }
  Entry e;
  if ((rc = lookup(key, &e))) return rc;
  if ((rc = check_dims(e, 1, in, out_local))) return rc;
  WvPeers peers{};
  peers.n = world; peers.self = rank;
  for (int q = 0; q < world; q++) {
    if (!y_all[q]) { wv_set_error("wv_matvec_dev_gather: y_all[%d] is null", q); return WV_EARG; }
    peers.y[q] = y_all[q] + row_offset;
  }
  wv_cur_peers = &peers;
  rc = wv_launch_gemv(e.blob, dx, peers.y[rank], 1, 0, e.blob.rows, static_cast<cudaStream_t>(stream));
  wv_cur_peers = nullptr;
  if (rc) wv_set_error("wv_matvec_dev_gather: launch failed (%d): %s", rc, cudaGetErrorString(cudaGetLastError()));
  return rc;
}

// ---------------------------------------------------------------- fused projection epilogues and decode steps
int wv_launch_rmsnorm(const float* dx, const float* dgamma, float* dy, int rows, int dim, double eps, cudaStream_t st);   // wv_decode.cu
int wv_launch_rope_cache(float* dq, const float* dk, const float* dv, float* dcache_k, float* dcache_v, int pos, int msl,
                         int num_heads, int num_kv_heads, int head_dim, double theta, cudaStream_t st);
int wv_launch_attn_decode(const float* dq, const float* dcache_k, const float* dcache_v, float* dout, int num_heads, int num_kv_heads,
                          int head_dim, int kv_len, int msl, float scale, cudaStream_t st);
int wv_launch_silu_mul(const float* dgate, const float* dup, float* dout, int n, cudaStream_t st);
int wv_launch_residual_add(float* ddst, const float* dadd, int n, cudaStream_t st);

// Sharded or local group launch with fused epilogues. keys[n]; y_all[n * world] lists, matrix by matrix, every
// rank's output vector (world == 1: just the local ones); row_offset[n] is where this rank's rows start in them.
static int fused_launch(const char* who, const uint64_t* keys, int n, const float* dx, float* const* y_all, int world, int rank,
                        const int* row_offset, int in, const int* out_local, int mode, const float* dres, cudaStream_t st,
                        const float* dgamma = nullptr, double eps = 0.0) {
  if (!keys || !dx || !y_all || !out_local || n < 1 || n > 4) { wv_set_error("%s: bad argument (1..4 matrices)", who); return WV_EARG; }
  if (world < 1 || world > WV_MAX_PEERS || rank < 0 || rank >= world) { wv_set_error("%s: world=%d rank=%d (at most %d ranks)", who, world, rank, WV_MAX_PEERS); return WV_EARG; }
  if (mode == 1 && n != 2) { wv_set_error("%s: the gate product takes exactly two matrices", who); return WV_EARG; }
  if (dres && n != 1) { wv_set_error("%s: a residual goes with one matrix", who); return WV_EARG; }
  WvDevBlob blobs[4];
  int rc;
  for (int i = 0; i < n; i++) {
    Entry e;
    if ((rc = lookup(keys[i], &e))) return rc;
    if ((rc = check_dims(e, 1, in, out_local[i]))) return rc;
    blobs[i] = e.blob;
    for (int q = 0; q < world; q++)
      if (!y_all[i * world + q] && !(mode == 1 && i == 0)) { wv_set_error("%s: output %d of rank %d is null", who, i, q); return WV_EARG; }
  }
  if (mode == 1 && blobs[0].rows != blobs[1].rows) { wv_set_error("%s: gate and up differ in rows", who); return WV_ESHAPE; }
  WvFuse fuse{};
  fuse.mode = mode;
  fuse.residual = dres ? dres + (row_offset ? row_offset[0] : 0) : nullptr;   // indexed like the output vectors
  fuse.npeers = world > 1 ? world : 0;
  fuse.norm_gamma = dgamma;
  fuse.norm_eps = eps;
  float* local[4];
  for (int i = 0; i < n; i++) {
    const int off = row_offset ? row_offset[i] : 0;
    float* own = y_all[i * world + rank];
    local[i] = own ? own + off : nullptr;
    for (int q = 0; q < world; q++) fuse.py[i][q] = y_all[i * world + q] ? y_all[i * world + q] + off : nullptr;
  }
  const bool need_fuse = mode != 0 || dres || world > 1 || dgamma;
  if (blobs[0].fast && blobs[0].format != WV_NONE) {
    wv_cur_fuse = need_fuse ? &fuse : nullptr;
    rc = wv_launch_gemv_tma_group(blobs, n, dx, local, 1, 0, n == 1 ? blobs[0].rows : 0, st);   // a single matrix carries its row range
    wv_cur_fuse = nullptr;
    if (rc != 1) {
      if (rc) wv_set_error("%s: launch failed (%d): %s", who, rc, cudaGetErrorString(cudaGetLastError()));
      return rc;
    }
  }
  // Shapes or mixes the grouped kernel does not take: the same results from separate launches.
  if (dgamma) {   // the norm as its own launch into a scratch vector
    float* xn = reinterpret_cast<float*>(wv_scratch_take((size_t)in * 4));
    if (!xn) { wv_set_error("%s: activation scratch too small", who); return WV_ENOMEM; }
    if ((rc = wv_launch_rmsnorm(dx, dgamma, xn, 1, in, eps, st))) return rc;
    dx = xn;
  }
  if (world > 1) {
    if (mode != 0 || dres) { wv_set_error("%s: this shape has no sharded fused path", who); return WV_ESHAPE; }
    for (int i = 0; i < n; i++) {
      WvPeers peers{};
      peers.n = world; peers.self = rank;
      for (int q = 0; q < world; q++) peers.y[q] = fuse.py[i][q];
      wv_cur_peers = &peers;
      rc = wv_launch_gemv(blobs[i], dx, peers.y[rank], 1, 0, blobs[i].rows, st);
      wv_cur_peers = nullptr;
      if (rc) return rc;
    }
    return WV_OK;
  }
  if (mode == 1) {
    // gate into the output vector, up into a scratch slot, then the product in place
    float* up = reinterpret_cast<float*>(wv_scratch_take((size_t)blobs[1].rows * 4));
    if (!up) { wv_set_error("%s: activation scratch too small", who); return WV_ENOMEM; }
    if ((rc = wv_launch_gemv(blobs[0], dx, local[1], 1, 0, blobs[0].rows, st))) return rc;
    if ((rc = wv_launch_gemv(blobs[1], dx, up, 1, 0, blobs[1].rows, st))) return rc;
    return wv_launch_silu_mul(local[1], up, local[1], blobs[1].rows, st);
  }
  for (int i = 0; i < n; i++) {
    if (dres && dres == local[i]) {   // in place: W x into scratch, then added
      float* tmp = reinterpret_cast<float*>(wv_scratch_take((size_t)blobs[i].rows * 4));
      if (!tmp) { wv_set_error("%s: activation scratch too small", who); return WV_ENOMEM; }
      if ((rc = wv_launch_gemv(blobs[i], dx, tmp, 1, 0, blobs[i].rows, st))) return rc;
      if ((rc = wv_launch_residual_add(local[i], tmp, blobs[i].rows, st))) return rc;
    } else {
      if ((rc = wv_launch_gemv(blobs[i], dx, local[i], 1, 0, blobs[i].rows, st))) return rc;
      if (dres && (rc = wv_launch_residual_add(local[i], dres, blobs[i].rows, st))) return rc;
    }
  }
  return WV_OK;
}

extern "C" int wv_matvec_dev_swiglu(uint64_t key_gate, uint64_t key_up, const float* dx, float* dh, int in, int out, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dh) { wv_set_error("wv_matvec_dev_swiglu: null output"); return WV_EARG; }
  const uint64_t keys[2] = {key_gate, key_up};
  float* ys[2] = {nullptr, dh};
  const int outs[2] = {out, out};
  return fused_launch("wv_matvec_dev_swiglu", keys, 2, dx, ys, 1, 0, nullptr, in, outs, 1, nullptr, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_matvec_dev_add(uint64_t key, const float* dx, const float* dresidual, float* dy, int in, int out, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dy || !dresidual) { wv_set_error("wv_matvec_dev_add: null pointer"); return WV_EARG; }
  float* ys[1] = {dy};
  return fused_launch("wv_matvec_dev_add", &key, 1, dx, ys, 1, 0, nullptr, in, &out, 0, dresidual, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_matvec_dev_group_gather(const uint64_t* keys, int n, const float* dx, float* const* y_all, int world, int rank,
                                          const int* row_offset, int in, const int* out_local, int mode, const float* dresidual, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  return fused_launch("wv_matvec_dev_group_gather", keys, n, dx, y_all, world, rank, row_offset, in, out_local, mode, dresidual,
                      static_cast<cudaStream_t>(stream));
}

extern "C" int wv_matvec_dev_fused(const WvFusedCall* c, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!c) { wv_set_error("wv_matvec_dev_fused: null call"); return WV_EARG; }
  if (c->dnorm_gamma && !(c->norm_eps >= 0.0)) { wv_set_error("wv_matvec_dev_fused: negative eps"); return WV_EARG; }
  return fused_launch("wv_matvec_dev_fused", c->keys, c->n, c->dx, c->y_all, c->world, c->rank, c->row_offset, c->in, c->out_local, c->mode,
                      c->dresidual, static_cast<cudaStream_t>(stream), c->dnorm_gamma, c->norm_eps);
}

extern "C" int wv_rmsnorm_dev(const float* dx, const float* dgamma, float* dy, int rows, int dim, double eps, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dx || !dgamma || !dy || rows < 1 || dim < 1) { wv_set_error("wv_rmsnorm_dev: bad argument"); return WV_EARG; }
  return wv_launch_rmsnorm(dx, dgamma, dy, rows, dim, eps, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_rope_cache_dev(float* dq, const float* dk, const float* dv, float* dcache_k, float* dcache_v, int pos, int max_seq_len,
                                 int num_heads, int num_kv_heads, int head_dim, double theta, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dq || !dk || !dv || !dcache_k || !dcache_v || pos < 0 || max_seq_len < 1 || num_heads < 1 || num_kv_heads < 1 || head_dim < 2 || (head_dim & 1)) {
    wv_set_error("wv_rope_cache_dev: bad argument"); return WV_EARG;
  }
  return wv_launch_rope_cache(dq, dk, dv, dcache_k, dcache_v, pos, max_seq_len, num_heads, num_kv_heads, head_dim, theta, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_attn_decode_dev(const float* dq, const float* dcache_k, const float* dcache_v, float* dout, int num_heads, int num_kv_heads,
                                  int head_dim, int kv_len, int max_seq_len, float scale, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dq || !dcache_k || !dcache_v || !dout || num_heads < 1 || num_kv_heads < 1 || kv_len < 1 || max_seq_len < 1 || kv_len > max_seq_len) {
    wv_set_error("wv_attn_decode_dev: bad argument"); return WV_EARG;
  }
  return wv_launch_attn_decode(dq, dcache_k, dcache_v, dout, num_heads, num_kv_heads, head_dim, kv_len, max_seq_len, scale, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_silu_mul_dev(const float* dgate, const float* dup, float* dout, int n, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dgate || !dup || !dout || n < 0) { wv_set_error("wv_silu_mul_dev: bad argument"); return WV_EARG; }
  return wv_launch_silu_mul(dgate, dup, dout, n, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_residual_add_dev(float* ddst, const float* dadd, int n, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!ddst || !dadd || n < 0) { wv_set_error("wv_residual_add_dev: bad argument"); return WV_EARG; }
  return wv_launch_residual_add(ddst, dadd, n, static_cast<cudaStream_t>(stream));
}

int wv_launch_gather_signal(unsigned* const* flags_all, int world, int rank, cudaStream_t st);   // wv_gemv.cu
int wv_launch_gather_wait(unsigned* flags_own, int world, cudaStream_t st);

extern "C" int wv_gather_signal(unsigned* const* flags_all, int world, int rank, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!flags_all || world < 1 || world > WV_MAX_PEERS || rank < 0 || rank >= world) { wv_set_error("wv_gather_signal: bad argument"); return WV_EARG; }
  for (int q = 0; q < world; q++) if (!flags_all[q]) { wv_set_error("wv_gather_signal: flags_all[%d] is null", q); return WV_EARG; }
  return wv_launch_gather_signal(flags_all, world, rank, static_cast<cudaStream_t>(stream));
}
int wv_launch_gather_sync(unsigned* const* flags_all, int world, int rank, cudaStream_t st);
extern "C" int wv_gather_sync(unsigned* const* flags_all, int world, int rank, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!flags_all || world < 1 || world > WV_MAX_PEERS || rank < 0 || rank >= world) { wv_set_error("wv_gather_sync: bad argument"); return WV_EARG; }
  for (int q = 0; q < world; q++) if (!flags_all[q]) { wv_set_error("wv_gather_sync: flags_all[%d] is null", q); return WV_EARG; }
  return wv_launch_gather_sync(flags_all, world, rank, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_gather_wait(unsigned* flags_own, int world, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!flags_own || world < 1 || world > WV_MAX_PEERS) { wv_set_error("wv_gather_wait: bad argument"); return WV_EARG; }
  return wv_launch_gather_wait(flags_own, world, static_cast<cudaStream_t>(stream));
}

extern "C" int wv_gather_alloc(size_t bytes, void** dptr, unsigned char handle[64]) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dptr || !handle || !bytes) { wv_set_error("wv_gather_alloc: bad argument"); return WV_EARG; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); wv_set_error("wv_gather_alloc: %zu bytes", bytes); return WV_ENOMEM; }
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); wv_set_error("wv_gather_alloc: %s", cudaGetErrorString(e)); cudaGetLastError(); return WV_ECUDA; }
  memcpy(handle, &h, 64);
  CUDA_TRY(cudaMemset(p, 0, bytes));
  *dptr = p;
  return WV_OK;
}
extern "C" int wv_gather_open(const unsigned char handle[64], void** dptr) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dptr || !handle) { wv_set_error("wv_gather_open: bad argument"); return WV_EARG; }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  cudaError_t e = cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { wv_set_error("wv_gather_open: %s", cudaGetErrorString(e)); cudaGetLastError(); return WV_ECUDA; }
  return WV_OK;
}
extern "C" int wv_gather_close(void* dptr) {
  if (!dptr) return WV_OK;
  cudaError_t e = cudaIpcCloseMemHandle(dptr);
  if (e != cudaSuccess) { wv_set_error("wv_gather_close: %s", cudaGetErrorString(e)); cudaGetLastError(); return WV_ECUDA; }
  return WV_OK;
}
extern "C" int wv_gather_free(void* dptr) {
  if (dptr && cudaFree(dptr) != cudaSuccess) { cudaGetLastError(); return WV_ECUDA; }
  return WV_OK;
}

extern "C" int wv_gather_read(const void* dptr, size_t offset_bytes, void* host, size_t bytes, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dptr || !host) { wv_set_error("wv_gather_read: null pointer"); return WV_EARG; }
  CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  CUDA_TRY(cudaMemcpy(host, static_cast<const unsigned char*>(dptr) + offset_bytes, bytes, cudaMemcpyDeviceToHost));
  return WV_OK;
}

static int grow(float** p, size_t* cap, size_t n, bool pinned) {
  if (*cap >= n) return WV_OK;
  if (*p) { if (pinned) cudaFreeHost(*p); else cudaFree(*p); *p = nullptr; *cap = 0; }
  size_t want = n + n / 2 + 1024;
  cudaError_t e = pinned ? cudaMallocHost(p, want * 4) : cudaMalloc(p, want * 4);
  if (e != cudaSuccess) { cudaGetLastError(); wv_set_error("staging allocation of %zu floats failed: %s", want, cudaGetErrorString(e)); return WV_ENOMEM; }
  *cap = want;
  return WV_OK;
}

// ---------------------------------------------------------------- host-pointer call
// A small pool of staging slots, each with its own stream: concurrent callers (the reference calls Dense from several
// goroutines, layers/dense/cpu.go forwardTiledMC) overlap instead of queueing on one lock. x is copied into mapped pinned
// memory and brought to the device by a one-CTA kernel (a copy-engine transfer of a few kilobytes costs more in start-up
// than in transfer); the GEMV behind it is launched with programmatic stream serialisation, so its prologue overlaps
// that kernel; y is stored by the GEMV straight into mapped pinned memory. Calls with a batch share slot 0: the
// batched kernel's split scratch belongs to the library and takes one launch at a time.
// A slot also keeps one instantiated CUDA graph per matrix it has served (copy-in kernel + GEMV with the slot's fixed
// buffers): launches from several host threads are serialised by the driver, so a call that costs one graph launch instead
// of two kernel launches leaves more of the GPU to the other callers. A graph is built on the second call for a matrix
// (the first one may still set kernel attributes), only for the batch-1 kernels that use no scratch from the shared
// arena, and is dropped when the key is re-uploaded or the slot's buffers move.
struct SlotGraph { uint64_t gen = 0; cudaGraphExec_t exec = nullptr; int seen = 0; };
struct StageSlot {
  std::mutex mu;
  cudaStream_t st = nullptr;
  float *hx = nullptr, *hx_dev = nullptr, *dx = nullptr, *hy = nullptr, *hy_dev = nullptr;
  size_t hx_n = 0, dx_n = 0, hy_n = 0;
  std::unordered_map<uint64_t, SlotGraph> graphs;
  void drop_graphs() {
    for (auto& kv : graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    graphs.clear();
  }
};
#define WV_STAGE_SLOTS 8
static StageSlot g_slots[WV_STAGE_SLOTS];
static std::atomic<unsigned> g_slot_rr{0};

__global__ void __launch_bounds__(256) stage_in_kernel(const float4* __restrict__ src, float4* __restrict__ dst, int n4, const float* __restrict__ src1,
                                                       float* __restrict__ dst1, int tail) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) dst[i] = src[i];
  if (blockIdx.x == 0 && (int)threadIdx.x < tail) dst1[threadIdx.x] = src1[threadIdx.x];
}

static int grow_mapped(float** h, float** d, size_t* cap, size_t n) {
  if (*cap >= n) return WV_OK;
  if (*h) { cudaFreeHost(*h); *h = nullptr; *cap = 0; }
  const size_t want = n + n / 2 + 1024;
  if (cudaHostAlloc(h, want * 4, cudaHostAllocMapped) != cudaSuccess) { cudaGetLastError(); wv_set_error("staging allocation of %zu floats failed", want); return WV_ENOMEM; }
  if (cudaHostGetDevicePointer(d, *h, 0) != cudaSuccess) { cudaGetLastError(); cudaFreeHost(*h); *h = nullptr; wv_set_error("no device alias for a staging buffer"); return WV_ECUDA; }
  *cap = want;
  return WV_OK;
}

extern "C" int wv_matvec(uint64_t key, const float* x, float* y, int batch, int in, int out) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!x || !y) { wv_set_error("wv_matvec: null pointer"); return WV_EARG; }
  Entry e;
  if ((rc = lookup(key, &e))) return rc;
  if ((rc = check_dims(e, batch, in, out))) return rc;
  const size_t nx = (size_t)batch * in, ny = (size_t)batch * out;
  StageSlot* slot = nullptr;
  if (batch == 1) {
    // a caller thread keeps coming back to the slot it took first, so that slot's buffers and launch graphs serve it again
    static thread_local int t_first = -1;
    if (t_first < 0) t_first = (int)(g_slot_rr.fetch_add(1) % WV_STAGE_SLOTS);
    const unsigned first = (unsigned)t_first;
    for (unsigned i = 0; i < WV_STAGE_SLOTS && !slot; i++) {
      StageSlot& c = g_slots[(first + i) % WV_STAGE_SLOTS];
      if (c.mu.try_lock()) slot = &c;
    }
    if (!slot) { slot = &g_slots[first % WV_STAGE_SLOTS]; slot->mu.lock(); }
  } else {
    slot = &g_slots[0];
    slot->mu.lock();
  }
  std::lock_guard<std::mutex> lk(slot->mu, std::adopt_lock);
  if (!slot->st) {
    if (slot == &g_slots[0]) slot->st = g_stream;
    else CUDA_TRY(cudaStreamCreateWithFlags(&slot->st, cudaStreamNonBlocking));
  }
  if (slot->hx_n < nx || slot->dx_n < nx || slot->hy_n < ny) slot->drop_graphs();   // the buffers are about to move
  if ((rc = grow_mapped(&slot->hx, &slot->hx_dev, &slot->hx_n, nx)) || (rc = grow(&slot->dx, &slot->dx_n, nx, false)) ||
      (rc = grow_mapped(&slot->hy, &slot->hy_dev, &slot->hy_n, ny))) return rc;
  memcpy(slot->hx, x, nx * 4);
  auto enqueue = [&]() -> int {
    const int n4 = (int)(nx / 4), tail = (int)(nx % 4);
    int blocks = (n4 + 255) / 256;
    if (blocks > 16) blocks = 16;
    if (blocks < 1) blocks = 1;
    stage_in_kernel<<<blocks, 256, 0, slot->st>>>(reinterpret_cast<const float4*>(slot->hx_dev), reinterpret_cast<float4*>(slot->dx), n4,
                                                 slot->hx_dev + (size_t)n4 * 4, slot->dx + (size_t)n4 * 4, tail);
    if (cudaGetLastError() != cudaSuccess) return WV_ECUDA;
    return wv_launch_gemv(e.blob, slot->dx, slot->hy_dev, batch, 0, e.blob.rows, slot->st);
  };
  const bool graphable = batch == 1 && e.blob.fast && e.blob.format != WV_NONE && e.blob.cols <= 16384;
  bool launched = false;
  if (graphable) {
    if (slot->graphs.size() >= 512 && !slot->graphs.count(key)) slot->drop_graphs();   // bound what a slot keeps
    SlotGraph& sg = slot->graphs[key];
    if (sg.gen != e.gen) { if (sg.exec) cudaGraphExecDestroy(sg.exec); sg = SlotGraph{}; sg.gen = e.gen; }
    if (!sg.exec && sg.seen == 1) {
      cudaGraph_t graph = nullptr;
      if (cudaStreamBeginCapture(slot->st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        const int crc = enqueue();
        const cudaError_t ce = cudaStreamEndCapture(slot->st, &graph);
        if (crc == WV_OK && ce == cudaSuccess && graph && cudaGraphInstantiate(&sg.exec, graph, 0) != cudaSuccess) sg.exec = nullptr;
        if (graph) cudaGraphDestroy(graph);
      }
      cudaGetLastError();
      if (!sg.exec) sg.seen = 2;      // could not be captured: this matrix stays on plain launches
    }
    if (sg.exec) {
      if (cudaGraphLaunch(sg.exec, slot->st) == cudaSuccess) launched = true;
      else { cudaGetLastError(); cudaGraphExecDestroy(sg.exec); sg.exec = nullptr; sg.seen = 2; }
    } else if (sg.seen == 0) sg.seen = 1;
  }
  if (!launched) {
    rc = enqueue();
    if (rc) { wv_set_error("wv_matvec: launch failed (%d): %s", rc, cudaGetErrorString(cudaGetLastError())); return rc; }
  }
  CUDA_TRY(cudaStreamSynchronize(slot->st));
  if (int te = wv_tma_take_error()) { wv_set_error("wv_matvec: a bounded device wait ran out (code %d)", te); return WV_ETIMEOUT; }
  memcpy(y, slot->hy, ny * 4);
  return WV_OK;
}

extern "C" int wv_device_status(void) {
  if (int te = wv_tma_take_error()) { wv_set_error("a bounded device wait ran out (code %d)", te); return WV_ETIMEOUT; }
  return WV_OK;
}

// ---------------------------------------------------------------- unpack
extern "C" int wv_unpack_dev(uint64_t key, float* d_out, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!d_out) { wv_set_error("wv_unpack_dev: null pointer"); return WV_EARG; }
  Entry e;
  if ((rc = lookup(key, &e))) return rc;
  return wv_launch_unpack(e.blob, d_out, static_cast<cudaStream_t>(stream));
}

extern "C" int wv_unpack(uint64_t key, float* out_host) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!out_host) { wv_set_error("wv_unpack: null pointer"); return WV_EARG; }
  Entry e;
  if ((rc = lookup(key, &e))) return rc;
  float* d = nullptr;
  cudaError_t ce = cudaMalloc(&d, (size_t)e.blob.n * 4);
  if (ce != cudaSuccess) { cudaGetLastError(); wv_set_error("wv_unpack: cudaMalloc(%lld floats): %s", e.blob.n, cudaGetErrorString(ce)); return WV_ENOMEM; }
  rc = wv_launch_unpack(e.blob, d, g_stream);
  cudaError_t c2 = cudaMemcpyAsync(out_host, d, (size_t)e.blob.n * 4, cudaMemcpyDeviceToHost, g_stream);
  cudaError_t c3 = cudaStreamSynchronize(g_stream);
  cudaFree(d);
  if (rc || c2 != cudaSuccess || c3 != cudaSuccess) { wv_set_error("wv_unpack failed: %s", cudaGetErrorString(c3 != cudaSuccess ? c3 : c2)); return rc ? rc : WV_ECUDA; }
  return WV_OK;
}

// quant.DecodeRow (quant/decode_row.go:7-38): row `row` of the rows this device holds, Cols floats.
extern "C" int wv_decode_row_dev(uint64_t key, int row, float* d_dst, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!d_dst) { wv_set_error("wv_decode_row_dev: null pointer"); return WV_EARG; }
  Entry e;
  if ((rc = lookup(key, &e))) return rc;
  if (row < 0 || row >= e.blob.rows) { wv_set_error("wv_decode_row_dev: shape row=%d rows=%d cols=%d", row, e.blob.rows, e.blob.cols); return WV_ESHAPE; }
  return wv_launch_unpack_rows(e.blob, row, 1, d_dst, static_cast<cudaStream_t>(stream));
}
extern "C" int wv_decode_row(uint64_t key, int row, float* dst_host, int ndst) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!dst_host) { wv_set_error("wv_decode_row: null pointer"); return WV_EARG; }
  Entry e;
  if ((rc = lookup(key, &e))) return rc;
  if (row < 0 || row >= e.blob.rows || ndst < e.blob.cols) {
    wv_set_error("wv_decode_row: shape row=%d cols=%d dst=%d", row, e.blob.cols, ndst); return WV_ESHAPE;
  }
  float* d = nullptr;
  if (cudaMalloc(&d, (size_t)e.blob.cols * 4) != cudaSuccess) { cudaGetLastError(); wv_set_error("wv_decode_row: cudaMalloc failed"); return WV_ENOMEM; }
  rc = wv_launch_unpack_rows(e.blob, row, 1, d, g_stream);
  cudaError_t c2 = cudaMemcpyAsync(dst_host, d, (size_t)e.blob.cols * 4, cudaMemcpyDeviceToHost, g_stream);
  cudaError_t c3 = cudaStreamSynchronize(g_stream);
  cudaFree(d);
  if (rc || c2 != cudaSuccess || c3 != cudaSuccess) { wv_set_error("wv_decode_row failed: %s", cudaGetErrorString(c3 != cudaSuccess ? c3 : c2)); return rc ? rc : WV_ECUDA; }
  return WV_OK;
}

// ---------------------------------------------------------------- pack
extern "C" int wv_pack(int format, int dtype, int bw, const float* w, int rows, int cols, void* raw, float* scales, float* mins) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!w || !raw) { wv_set_error("wv_pack: null pointer"); return WV_EARG; }
  Sizes s;
  if ((rc = expected_sizes(format, dtype, bw, rows, cols, &s))) return rc;
  if ((s.ns && !scales) || (s.nm && !mins)) { wv_set_error("wv_pack: format %d needs scales/mins buffers", format); return WV_EARG; }
  const size_t n = (size_t)rows * cols;
  float* dw = nullptr; unsigned char* dr = nullptr; float *ds = nullptr, *dm = nullptr;
  auto cleanup = [&]() { cudaFree(dw); cudaFree(dr); cudaFree(ds); cudaFree(dm); };
  if (cudaMalloc(&dw, n * 4) != cudaSuccess || cudaMalloc(&dr, s.nraw + 16) != cudaSuccess ||
      cudaMalloc(&ds, (s.ns + 1) * 4) != cudaSuccess || cudaMalloc(&dm, (s.nm + 1) * 4) != cudaSuccess) {
    cudaGetLastError(); cleanup(); wv_set_error("wv_pack: device allocation failed"); return WV_ENOMEM;
  }
  bool ok = cudaMemcpyAsync(dw, w, n * 4, cudaMemcpyHostToDevice, g_stream) == cudaSuccess &&
            cudaMemsetAsync(dr, 0, s.nraw, g_stream) == cudaSuccess;
  if (ok) rc = wv_launch_pack(format, dtype, s.group, dw, rows, cols, dr, ds, dm, g_stream);
  if (ok && !rc) {
    ok = cudaMemcpyAsync(raw, dr, s.nraw, cudaMemcpyDeviceToHost, g_stream) == cudaSuccess;
    if (ok && s.ns) ok = cudaMemcpyAsync(scales, ds, s.ns * 4, cudaMemcpyDeviceToHost, g_stream) == cudaSuccess;
    if (ok && s.nm) ok = cudaMemcpyAsync(mins, dm, s.nm * 4, cudaMemcpyDeviceToHost, g_stream) == cudaSuccess;
  }
  cudaError_t se = cudaStreamSynchronize(g_stream);
  cleanup();
  if (rc) return rc;
  if (!ok || se != cudaSuccess) { wv_set_error("wv_pack failed: %s", cudaGetErrorString(se)); return WV_ECUDA; }
  return WV_OK;
}

extern "C" int wv_pack_upload_dev(uint64_t key, int format, int dtype, int bw, const float* d_w, int rows, int cols, void* stream) {
  int rc = ensure_init();
  if (rc) return rc;
  if (!d_w) { wv_set_error("wv_pack_upload_dev: null pointer"); return WV_EARG; }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_cache.count(key)) return WV_OK;
  }
  Sizes s;
  if ((rc = expected_sizes(format, dtype, bw, rows, cols, &s))) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* dr = nullptr; float *ds = nullptr, *dm = nullptr;
  auto cleanup = [&]() { cudaFree(dr); cudaFree(ds); cudaFree(dm); };
  if (cudaMalloc(&dr, s.nraw + 16) != cudaSuccess || cudaMalloc(&ds, (s.ns + 1) * 4) != cudaSuccess || cudaMalloc(&dm, (s.nm + 1) * 4) != cudaSuccess) {
    cudaGetLastError(); cleanup(); wv_set_error("wv_pack_upload_dev: device allocation failed"); return WV_ENOMEM;
  }
  cudaMemsetAsync(dr, 0, s.nraw, st);
  rc = wv_launch_pack(format, dtype, s.group, d_w, rows, cols, dr, ds, dm, st);
  if (cudaStreamSynchronize(st) != cudaSuccess) rc = rc ? rc : WV_ECUDA;
  if (rc) { cleanup(); wv_set_error("wv_pack_upload_dev: pack failed (%d)", rc); return rc; }
  // Reuse the normal upload path from a host bounce of the packed arrays: packed blobs are
  // 4-25x smaller than the f32 source, and upload is a one-time cost per blob.
  std::vector<unsigned char> hr(s.nraw);
  std::vector<float> hs(s.ns), hm(s.nm);
  cudaMemcpy(hr.data(), dr, s.nraw, cudaMemcpyDeviceToHost);
  if (s.ns) cudaMemcpy(hs.data(), ds, s.ns * 4, cudaMemcpyDeviceToHost);
  if (s.nm) cudaMemcpy(hm.data(), dm, s.nm * 4, cudaMemcpyDeviceToHost);
  cleanup();
  return upload_locked_free(key, format, dtype, rows, cols, s.group, hr.data(), s.nraw, hs.data(), s.ns, hm.data(), s.nm);
}
