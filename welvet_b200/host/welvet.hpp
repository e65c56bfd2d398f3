// welvet.hpp — C++17 host side of the CUDA Dense MatVec backend, above the C ABI of
// libwelvet_cuda.so (include/welvet_cuda.h). Header only.
//
// The reference is a Go module; this mirror keeps its package / function names and argument
// meaning for the Dense MatVec path so that code written against the reference reads the same:
//
//   Go (reference)                                   C++ (here)
//   b, err := quant.Pack(f, w, rows, cols)           auto [b, err] = quant::Pack(f, w, rows, cols);
//   err := quant.MatVec(b, x, y)                     Error err = quant::MatVec(b.get(), x, y);
//   pre, post, err := dense.Forward(l, in)           auto [pre, post, err] = dense::Forward(l.get(), &in);
//
// Go's `error` is welvet::Error (falsy = nil). Nothing here computes on the host: Pack, Unpack
// and every GEMV run in the library; without a usable device every call returns the library's
// error (no fallback, reference README.md:154).
//
// Reference interfaces mirrored (paths inside openfluke/welvet):
//   core.Backend / DType / Tensor / ActivationType  core/layer.go:125-153, core/dtype.go:15-17, core/tensor.go
//   quant.Format, Blob, Pack, Unpack, MatVec          quant/format.go:9-144, pack.go:4-31, unpack.go:4-34, matvec.go:5-35
//   weights.Store, New, FromBlob, packed wire         weights/store.go:14-66, from_blob.go:11-32, packed_wire.go:30-110
//   dense.Layer, NewConfigured, Forward, MatVec*      layers/dense/dense.go:12-167, simd.go:571-614, webgpu.go:17-48
//   resident-weight cache (Warm / Has / Clear / Bytes) webgpu/affine_cache.go:29-203
//   sampling.ArgMax                                    model/sampling/argmax.go:4-18
//   fused projection groups (Q|K|V, gate|up)           fusedgpu/shaders.go:59-222, mha/cpu.go:48-96, swiglu/cpu.go:29-52
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "welvet_cuda.h"

namespace welvet {

// Go's error value: falsy when nil.
struct Error {
  int code = 0;  // WV_E* status of the C ABI, 0 = nil
  std::string msg;
  explicit operator bool() const { return code != 0; }
  const std::string& String() const { return msg; }
};
inline Error errorf(int code, std::string msg) { return Error{code, std::move(msg)}; }
inline Error fromStatus(const char* op, int rc) {
  if (rc == 0) return {};
  return Error{rc, std::string("cuda ") + op + ": " + wv_last_error()};
}

namespace core {
enum Backend : int { BackendCPUTiled = 0, BackendSIMD = 1, BackendWebGPU = 2, BackendCUDA = 3 };  // core/layer.go:127-131 + CUDA
inline const char* BackendString(Backend b) {
  switch (b) { case BackendCPUTiled: return "cpu_tiled"; case BackendSIMD: return "simd"; case BackendWebGPU: return "webgpu"; case BackendCUDA: return "cuda"; }
  return "unknown";
}
enum DType : int { DTypeFloat32 = 1, DTypeFloat16 = 2, DTypeBFloat16 = 3 };  // the three FormatNone dtypes the backend streams
// core.ActivationType (core/layer.go:91-98): the integer values are part of the call surface.
enum ActivationType : int {
  ActivationLinear = -1, ActivationReLU = 0, ActivationSilu = 1, ActivationGELU = 2, ActivationTanh = 3,
  ActivationSigmoid = 4, ActivationLeakyReLU = 5, ActivationReLU2 = 6
};
// core.Activate (core/activate.go:6-38) in f64. `ok` turns false for a value outside the enum: the
// reference hands such a value back unchanged, this mirror reports it (dense::ForwardCUDA).
inline double Activate(double x, ActivationType act, bool* ok = nullptr) {
  switch (act) {
  case ActivationLinear: return x;
  case ActivationReLU: return x < 0 ? 0.0 : x;
  case ActivationReLU2: return x < 0 ? 0.0 : x * x;
  case ActivationLeakyReLU: return x < 0 ? 0.01 * x : x;
  case ActivationSilu: return x / (1 + std::exp(-x));
  case ActivationGELU: return 0.5 * x * (1 + std::tanh(std::sqrt(2 / 3.14159265358979323846) * (x + 0.044715 * x * x * x)));
  case ActivationTanh: return std::tanh(x);
  case ActivationSigmoid: return 1 / (1 + std::exp(-x));
  }
  if (ok) *ok = false;
  return x;
}
struct ExecConfig { Backend Backend_ = BackendCUDA; bool MultiCore = true; int TileSize = 32; };  // core/layer.go:147-153

template <typename T> struct Tensor {  // core.Tensor[T]: flat data + shape
  std::vector<T> Data;
  std::vector<int> Shape;
};
template <typename T> std::unique_ptr<Tensor<T>> NewTensor(int d0, int d1) {
  auto t = std::make_unique<Tensor<T>>();
  t->Shape = {d0, d1};
  t->Data.assign((size_t)d0 * d1, T(0));
  return t;
}
}  // namespace core

namespace cuda {
// Session and resident-weight cache: twins of webgpu.Available / ensure and of the Warm*/Has*/
// Clear*/*CacheBytes family.
inline Error Init(int device = 0) { return fromStatus("init", wv_init(device)); }
inline bool Available() { return wv_available() == 1; }
inline int DeviceCount() { return wv_device_count(); }
inline void Clear() { wv_cache_clear(); }
inline uint64_t CacheBytes() { return wv_cache_bytes(); }
inline void SetCacheLimit(uint64_t bytes) { wv_cache_set_limit(bytes); }
inline bool IsVRAMFull(const Error& e) { return e.code == WV_ENOMEM; }  // IsAffineVRAMFull, webgpu/affine_cache.go:71-83
}  // namespace cuda

namespace quant {
enum Format : int {  // quant/format.go:9-39
  FormatNone = 0, FormatQ8_0, FormatQ4_0, FormatQ4_1, FormatQ5_0, FormatQ5_1, FormatQ2_K, FormatQ3_K, FormatQ4_K, FormatQ5_K,
  FormatQ6_K, FormatIQ1_S, FormatIQ2_XXS, FormatIQ2_XS, FormatIQ3_XXS, FormatIQ3_S, FormatIQ4_NL, FormatIQ4_XS,
  FormatTernaryPacked, FormatBinaryPacked, FormatAffinePacked, formatCount
};
inline const char* FormatString(Format f) {  // Format.String(), the ENTITY header names (quant/format.go:50-97)
  static const char* n[] = {"none", "Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ1_S", "IQ2_XXS",
                            "IQ2_XS", "IQ3_XXS", "IQ3_S", "IQ4_NL", "IQ4_XS", "TernaryPacked", "BinaryPacked", "AffinePacked"};
  return (f >= 0 && f < formatCount) ? n[f] : "unknown";
}
inline Format ParseFormatName(const std::string& s) {  // quant/format.go:134-144: unknown names read as FormatNone
  for (int f = 1; f < formatCount; f++) if (s == FormatString((Format)f)) return (Format)f;
  return FormatNone;
}
inline bool IsKQuant(Format f) { return f >= FormatQ2_K && f <= FormatQ6_K; }
constexpr int BinaryG128Group = 128, AffineG64Group = 64;

// quant.Blob (quant/format.go:110-131). The cache key is the Blob's address, as in the
// reference (webgpu/binary_cache.go:198); destroying a Blob evicts its device copy so that a
// reused address can never alias a stale entry.
struct Blob {
  Format Format_ = FormatNone;
  int Rows = 0, Cols = 0;
  std::vector<uint8_t> Raw;
  std::vector<float> Scales, Mins;
  std::vector<uint8_t> Meta;
  int BlockWeights = 0;
  core::DType DType_ = core::DTypeFloat32;  // FormatNone only
  Blob() = default;
  Blob(const Blob&) = delete;
  Blob& operator=(const Blob&) = delete;
  ~Blob() { if (wv_available() == 1 && wv_blob_has(Key()) == 1) wv_blob_evict(Key()); }
  uint64_t Key() const { return (uint64_t)(uintptr_t)this; }
  size_t PackedBytes() const { return Raw.size() + 4 * Scales.size() + 4 * Mins.size(); }
};
using BlobPtr = std::unique_ptr<Blob>;

// Upload once per Blob; with world > 1 only this rank's contiguous row range stays resident
// (the reference shards rows over goroutines the same way, layers/dense/gemv_parallel.go:24-41).
inline Error EnsureResident(const Blob* b, int rank = 0, int world = 1) {
  if (!b || b->Raw.empty()) return errorf(WV_EARG, "cuda: nil blob");
  if (wv_blob_has(b->Key()) == 1) return {};
  const float* sc = b->Scales.empty() ? nullptr : b->Scales.data();
  const float* mn = b->Mins.empty() ? nullptr : b->Mins.data();
  int rc = world > 1 ? wv_blob_upload_shard(b->Key(), b->Format_, b->DType_, b->Rows, b->Cols, b->BlockWeights, b->Raw.data(), b->Raw.size(),
                                           sc, b->Scales.size(), mn, b->Mins.size(), rank, world)
                     : wv_blob_upload(b->Key(), b->Format_, b->DType_, b->Rows, b->Cols, b->BlockWeights, b->Raw.data(), b->Raw.size(), sc,
                                      b->Scales.size(), mn, b->Mins.size());
  return fromStatus("upload", rc);
}

// quant.Pack on the device: output bytes identical to the reference packer's. blockWeights = 128
// with FormatBinaryPacked builds the row-aligned g128 layout; FormatNone encodes dt.
inline std::pair<BlobPtr, Error> Pack(Format format, const std::vector<float>& weights, int rows, int cols, int blockWeights = 0,
                                      core::DType dt = core::DTypeFloat32) {
  if (rows <= 0 || cols <= 0 || weights.size() < (size_t)rows * cols)
    return {nullptr, errorf(WV_ESHAPE, "quant: Pack: bad shape")};
  size_t nraw = 0, ns = 0, nm = 0;
  if (int rc = wv_pack_sizes(format, dt, blockWeights, rows, cols, &nraw, &ns, &nm)) return {nullptr, fromStatus("pack_sizes", rc)};
  auto b = std::make_unique<Blob>();
  b->Format_ = format; b->Rows = rows; b->Cols = cols; b->DType_ = dt;
  b->Raw.assign(nraw, 0); b->Scales.assign(ns, 0.f); b->Mins.assign(nm, 0.f);
  if (int rc = wv_pack(format, dt, blockWeights, weights.data(), rows, cols, b->Raw.data(), ns ? b->Scales.data() : nullptr,
                       nm ? b->Mins.data() : nullptr))
    return {nullptr, fromStatus("pack", rc)};
  switch (format) {
  case FormatNone: b->BlockWeights = 1; break;
  case FormatTernaryPacked: b->BlockWeights = 16; break;
  case FormatBinaryPacked: b->BlockWeights = blockWeights == BinaryG128Group ? BinaryG128Group : 32; break;
  case FormatAffinePacked: b->BlockWeights = blockWeights ? blockWeights : AffineG64Group; break;
  default: b->BlockWeights = IsKQuant(format) ? 256 : 32;
  }
  return {std::move(b), Error{}};
}

// quant.Unpack: the dequantised f32 weights, bit-identical to the reference's.
inline std::pair<std::vector<float>, Error> Unpack(const Blob* b) {
  if (Error e = EnsureResident(b)) return {{}, e};
  std::vector<float> out((size_t)b->Rows * b->Cols);
  if (int rc = wv_unpack(b->Key(), out.data())) return {{}, fromStatus("unpack", rc)};
  return {std::move(out), Error{}};
}

// quant.MatVec: y = W x with the reference's length rule (quant/helpers.go:94-103).
inline Error MatVec(const Blob* b, const std::vector<float>& x, std::vector<float>& y) {
  if (!b) return errorf(WV_EARG, "quant: MatVec: nil blob");
  if (x.size() < (size_t)b->Cols || y.size() < (size_t)b->Rows) return errorf(WV_ESHAPE, "quant: MatVec: size mismatch");
  if (Error e = EnsureResident(b)) return e;
  return fromStatus("matvec", wv_matvec(b->Key(), x.data(), y.data(), 1, b->Cols, b->Rows));
}

// quant.DecodeRow (quant/decode_row.go:7-38): one output row of a packed Blob into dst (len >= Cols); FormatNone is
// refused as in the reference ("use weights.DecodeRow").
inline Error DecodeRow(const Blob* b, int row, std::vector<float>& dst) {
  if (!b) return errorf(WV_EFORMAT, "quant: DecodeRow: nil blob");
  if (row < 0 || row >= b->Rows || dst.size() < (size_t)b->Cols)
    return errorf(WV_ESHAPE, "quant: DecodeRow shape row=" + std::to_string(row) + " cols=" + std::to_string(b->Cols) + " dst=" + std::to_string(dst.size()));
  if (b->Format_ == FormatNone) return errorf(WV_EFORMAT, "quant: DecodeRow FormatNone - use weights.DecodeRow");
  if (Error e = EnsureResident(b)) return e;
  return fromStatus("decode_row", wv_decode_row(b->Key(), row, dst.data(), (int)dst.size()));
}
}  // namespace quant

namespace weights {
// weights.Store (weights/store.go:14-32): storage truth for one matrix.
struct Store {
  core::DType DType_ = core::DTypeFloat32;
  quant::Format Format_ = quant::FormatNone;
  int Rows = 0, Cols = 0;
  quant::BlobPtr Packed;
  std::vector<double> Bias;  // applied after the GEMV (dense.applyBiasAct)

  // Store.Pack (weights/store.go:86-103, weights/convert.go:103-124): re-encode as `format`;
  // the old blob's device copy goes with it.
  Error Pack(quant::Format format, int blockWeights = 0) {
    if (!Packed) return errorf(WV_EARG, "weights: nil packed blob");
    auto [w, e1] = quant::Unpack(Packed.get());
    if (e1) return e1;
    auto [b, e2] = quant::Pack(format, w, Rows, Cols, blockWeights, DType_);
    if (e2) return e2;
    Packed = std::move(b);
    Format_ = format;
    return {};
  }
};
using StorePtr = std::unique_ptr<Store>;

// weights.New (weights/store.go:35-66): nil data means zeros.
inline std::pair<StorePtr, Error> New(int rows, int cols, const std::vector<float>* data, core::DType dt, quant::Format format,
                                      int blockWeights = 0) {
  if (rows <= 0 || cols <= 0) return {nullptr, errorf(WV_ESHAPE, "weights: bad shape")};
  const size_t n = (size_t)rows * cols;
  std::vector<float> zeros;
  if (!data) { zeros.assign(n, 0.f); data = &zeros; }
  if (data->size() < n) return {nullptr, errorf(WV_ESHAPE, "weights: not enough values")};
  auto [b, e] = quant::Pack(format, *data, rows, cols, blockWeights, dt);
  if (e) return {nullptr, e};
  auto s = std::make_unique<Store>();
  s->DType_ = dt; s->Format_ = format; s->Rows = rows; s->Cols = cols; s->Packed = std::move(b);
  return {std::move(s), Error{}};
}

// weights.FromBlob (weights/from_blob.go:11-32): the Store takes the blob over.
inline std::pair<StorePtr, Error> FromBlob(quant::BlobPtr b) {
  if (!b) return {nullptr, errorf(WV_EARG, "weights: nil blob")};
  auto s = std::make_unique<Store>();
  s->DType_ = b->DType_; s->Format_ = b->Format_; s->Rows = b->Rows; s->Cols = b->Cols; s->Packed = std::move(b);
  return {std::move(s), Error{}};
}

// weights.EncodePackedWire (weights/packed_wire.go:30-53): u32 ns | u32 nm | u32 nr | scales |
// mins | raw, little-endian; FormatNone is the raw element array.
inline std::pair<std::vector<uint8_t>, Error> EncodePackedWire(const quant::Blob* b) {
  if (!b) return {{}, errorf(WV_EARG, "weights: nil blob")};
  if (b->Format_ == quant::FormatNone) return {b->Raw, Error{}};
  const uint32_t hdr[3] = {(uint32_t)b->Scales.size(), (uint32_t)b->Mins.size(), (uint32_t)b->Raw.size()};
  std::vector<uint8_t> out(12 + 4 * b->Scales.size() + 4 * b->Mins.size() + b->Raw.size());
  uint8_t* p = out.data();
  std::memcpy(p, hdr, 12); p += 12;
  if (!b->Scales.empty()) std::memcpy(p, b->Scales.data(), 4 * b->Scales.size());
  p += 4 * b->Scales.size();
  if (!b->Mins.empty()) std::memcpy(p, b->Mins.data(), 4 * b->Mins.size());
  p += 4 * b->Mins.size();
  if (!b->Raw.empty()) std::memcpy(p, b->Raw.data(), b->Raw.size());
  return {std::move(out), Error{}};
}

// weights.DecodePackedWire (weights/packed_wire.go:55-110): Meta / BlockWeights are not on the
// wire; binary blobs re-infer theirs (quant/binary_g128.go:79-94).
inline std::pair<quant::BlobPtr, Error> DecodePackedWire(quant::Format format, int rows, int cols, const std::vector<uint8_t>& wire,
                                                        core::DType dt = core::DTypeFloat32) {
  auto b = std::make_unique<quant::Blob>();
  b->Format_ = format; b->Rows = rows; b->Cols = cols; b->DType_ = dt;
  if (format == quant::FormatNone) {
    const size_t need = (size_t)rows * cols * (dt == core::DTypeFloat32 ? 4 : 2);
    if (wire.size() < need) return {nullptr, errorf(WV_ESHAPE, "weights: FormatNone wire short")};
    b->Raw.assign(wire.begin(), wire.begin() + need);
    b->BlockWeights = 1;
    return {std::move(b), Error{}};
  }
  if (wire.size() < 12) return {nullptr, errorf(WV_ESHAPE, "weights: packed wire too short")};
  uint32_t hdr[3];
  std::memcpy(hdr, wire.data(), 12);
  const size_t ns = hdr[0], nm = hdr[1], nr = hdr[2], need = 12 + 4 * ns + 4 * nm + nr;
  if (wire.size() < need) return {nullptr, errorf(WV_ESHAPE, "weights: packed wire truncated")};
  b->Scales.resize(ns); b->Mins.resize(nm); b->Raw.resize(nr);
  const uint8_t* p = wire.data() + 12;
  if (ns) std::memcpy(b->Scales.data(), p, 4 * ns);
  p += 4 * ns;
  if (nm) std::memcpy(b->Mins.data(), p, 4 * nm);
  p += 4 * nm;
  if (nr) std::memcpy(b->Raw.data(), p, nr);
  if (format == quant::FormatBinaryPacked)
    b->BlockWeights = (cols % 128 == 0 && ns == (size_t)rows * (cols / 128)) ? 128 : 32;
  return {std::move(b), Error{}};
}

// weights.MatVec for the packed path (weights/store.go:135-181).
inline Error MatVec(const Store* s, const std::vector<float>& x, std::vector<float>& y) {
  if (!s || !s->Packed) return errorf(WV_EARG, "weights: nil store");
  return quant::MatVec(s->Packed.get(), x, y);
}
}  // namespace weights

namespace dense {
// dense.Layer (layers/dense/dense.go:12-19)
struct Layer {
  int InputHeight = 0, OutputHeight = 0;
  core::ActivationType Activation = core::ActivationLinear;
  weights::StorePtr Weights;
  core::ExecConfig Exec;
};
using LayerPtr = std::unique_ptr<Layer>;

// dense.NewConfigured (layers/dense/dense.go:47-69)
inline std::pair<LayerPtr, Error> NewConfigured(int in, int out, core::ActivationType act, core::DType dt, quant::Format format,
                                                const std::vector<float>* init, int blockWeights = 0) {
  auto [ws, e] = weights::New(out, in, init, dt, format, blockWeights);
  if (e) return {nullptr, e};
  auto l = std::make_unique<Layer>();
  l->InputHeight = in; l->OutputHeight = out; l->Activation = act; l->Weights = std::move(ws);
  return {std::move(l), Error{}};
}

// Twin of dense.MatVecWebGPU (layers/dense/webgpu.go:36-48): y[batch,out] = x[batch,in] W^T.
inline Error MatVecCUDA(const weights::Store* s, const std::vector<float>& x, std::vector<float>& y, int batch, int in, int out) {
  if (!s || !s->Packed) return errorf(WV_EARG, "dense: nil weights");
  if (x.size() < (size_t)batch * in || y.size() < (size_t)batch * out) return errorf(WV_ESHAPE, "dense: matvec shape");
  if (Error e = quant::EnsureResident(s->Packed.get())) return e;
  return fromStatus("matvec", wv_matvec(s->Packed->Key(), x.data(), y.data(), batch, in, out));
}

// Projection group on one shared x (Q|K|V of mha, gate|up of swiglu): device pointers, asynchronous on `stream`;
// stores of one format and column count run as one launch, any other mix as separate launches.
inline Error MatVecGroupCUDA(const std::vector<const weights::Store*>& stores, const float* dx, const std::vector<float*>& dy,
                             int batch, int in, void* stream = nullptr) {
  const int n = (int)stores.size();
  if (n < 1 || n > 4 || dy.size() != stores.size()) return errorf(WV_EARG, "dense: group of 1..4 stores with one output each");
  uint64_t keys[4]; int outs[4]; float* ys[4];
  for (int i = 0; i < n; i++) {
    if (!stores[i] || !stores[i]->Packed) return errorf(WV_EARG, "dense: nil weights");
    if (Error e = quant::EnsureResident(stores[i]->Packed.get())) return e;
    keys[i] = stores[i]->Packed->Key(); outs[i] = stores[i]->Rows; ys[i] = dy[i];
  }
  return fromStatus("matvec_multi", wv_matvec_dev_multi(keys, n, dx, ys, batch, in, outs, stream));
}

// dense.MatVecPackedBlob (layers/dense/simd.go:571-614)
inline Error MatVecPackedBlob(const quant::Blob* b, const std::vector<float>& x, std::vector<float>& y) {
  if (!b) return errorf(WV_EARG, "dense: nil packed blob");
  if (x.size() < (size_t)b->Cols || y.size() < (size_t)b->Rows) return errorf(WV_ESHAPE, "dense: packed matvec shape");
  return quant::MatVec(b, x, y);
}

template <typename T> using TensorPtr = std::unique_ptr<core::Tensor<T>>;

// Shaped like dense.ForwardWebGPU (layers/dense/webgpu.go:17-33): x staged as f32, GEMV on the
// device, then bias + activation in f64 (applyBiasAct, dense.go:145-167). For a linear layer
// without bias the reference returns post aliased to pre; here post is a copy of pre.
template <typename T>
std::tuple<TensorPtr<T>, TensorPtr<T>, Error> ForwardCUDA(const Layer* l, const core::Tensor<T>* input) {
  if (input->Shape.size() < 2) return {nullptr, nullptr, errorf(WV_ESHAPE, "dense: input shape need [batch,in]")};
  const int batch = input->Shape[0], in = l->InputHeight, out = l->OutputHeight;
  if (input->Shape[1] != in) return {nullptr, nullptr, errorf(WV_ESHAPE, "dense: input width != layer in")};
  if (l->Weights->Rows != out || l->Weights->Cols != in) return {nullptr, nullptr, errorf(WV_ESHAPE, "dense: weight shape != out x in")};
  if (input->Data.size() < (size_t)batch * in) return {nullptr, nullptr, errorf(WV_ESHAPE, "dense: input data short")};
  {
    bool known = true;
    core::Activate(0.0, l->Activation, &known);
    if (!known) return {nullptr, nullptr, errorf(WV_EARG, "dense: unknown activation " + std::to_string((int)l->Activation))};
  }
  std::vector<float> xf(input->Data.begin(), input->Data.begin() + (size_t)batch * in), yf((size_t)batch * out);
  if (Error e = MatVecCUDA(l->Weights.get(), xf, yf, batch, in, out)) return {nullptr, nullptr, e};
  auto pre = core::NewTensor<T>(batch, out), post = core::NewTensor<T>(batch, out);
  const auto& bias = l->Weights->Bias;
  for (int bi = 0; bi < batch; bi++) {
    for (int o = 0; o < out; o++) {
      double v = (double)yf[(size_t)bi * out + o];
      if ((size_t)o < bias.size()) v += bias[o];
      pre->Data[(size_t)bi * out + o] = (T)v;
      post->Data[(size_t)bi * out + o] = (T)core::Activate((double)(T)v, l->Activation);
    }
  }
  return {std::move(pre), std::move(post), Error{}};
}

// dense.Forward (layers/dense/dense.go:100-112): dispatch on Exec.Backend. Backends this
// library does not provide are an error, not a silent host route.
template <typename T>
std::tuple<TensorPtr<T>, TensorPtr<T>, Error> Forward(const Layer* l, const core::Tensor<T>* input) {
  if (!l || !l->Weights || !input) return {nullptr, nullptr, errorf(WV_EARG, "dense: nil layer/input")};
  if (l->Exec.Backend_ == core::BackendCUDA) return ForwardCUDA<T>(l, input);
  return {nullptr, nullptr, errorf(WV_EFORMAT, std::string("dense: backend ") + core::BackendString(l->Exec.Backend_) + " is not provided by this library (cuda only)")};
}
}  // namespace dense

namespace sampling {
// sampling.ArgMax (model/sampling/argmax.go:4-18) over n device floats: first strict maximum, NaN never wins.
inline std::pair<int, Error> ArgMax(const float* d_logits, int n, void* stream = nullptr) {
  int idx = 0;
  if (int rc = wv_argmax(d_logits, n, &idx, stream)) return {0, fromStatus("argmax", rc)};
  return {idx, Error{}};
}
// sampling.SampleTopK (model/sampling/topk.go:11-50) over n device floats. `u` is the uniform draw the reference takes
// from math/rand inside the call (0 <= u <= 1); at most 1024 candidates on the device.
inline std::pair<int, Error> SampleTopK(const float* d_logits, int n, int topK, float temperature, bool deterministic, double u,
                                        void* stream = nullptr) {
  int idx = 0;
  if (int rc = wv_topk_sample(d_logits, n, topK, temperature, deterministic ? 1 : 0, u, &idx, stream)) return {0, fromStatus("topk_sample", rc)};
  return {idx, Error{}};
}
}  // namespace sampling
}  // namespace welvet
