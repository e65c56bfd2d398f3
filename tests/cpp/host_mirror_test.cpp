// Test program for the C++ host mirror (welvet_b200/host/welvet.hpp), written the way the
// reference's Go tests for this path read: build a blob, run it, compare with the CPU
// restatement (the oracle library; test infrastructure only).
//
//   host_mirror_test host   checks that need no device: names, wire codec, argument errors,
//                           the error of a device call without a device
//   host_mirror_test gpu    Pack / Unpack / MatVec / dense.Forward on cuda:0 against the oracle
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "welvet.hpp"

using namespace welvet;

extern "C" {
typedef struct {
  int32_t format, dtype, rows, cols, block_weights, _pad;
  uint8_t* raw; uint64_t nraw;
  float* scales; uint64_t ns;
  float* mins; uint64_t nm;
} wvo_blob;
int wvo_sizes(int format, int dtype, int block_weights, int rows, int cols, uint64_t* nraw, uint64_t* ns, uint64_t* nm);
int wvo_pack(const float* w, wvo_blob* out);
int wvo_unpack(const wvo_blob* b, float* out);
int wvo_matvec(const wvo_blob* b, const float* x, float* y);
int wvo_sum_abs_wx(const wvo_blob* b, const float* x, double* out);
}

static int failures = 0;
#define CHECK(cond, ...) do { if (!(cond)) { failures++; std::printf("FAIL %s:%d: ", __FILE__, __LINE__); std::printf(__VA_ARGS__); std::printf("\n"); } } while (0)

// Deterministic N(0, sigma) without a library generator: the same arrays feed device and oracle.
static std::vector<float> normal(size_t n, float sigma, uint64_t seed) {
  std::vector<float> v(n);
  uint64_t s = seed * 6364136223846793005ull + 1442695040888963407ull;
  auto u01 = [&]() { s = s * 6364136223846793005ull + 1442695040888963407ull; return ((s >> 11) + 0.5) / 9007199254740992.0; };
  for (size_t i = 0; i < n; i += 2) {
    const double r = std::sqrt(-2.0 * std::log(u01())), t = 6.283185307179586 * u01();
    v[i] = (float)(sigma * r * std::cos(t));
    if (i + 1 < n) v[i + 1] = (float)(sigma * r * std::sin(t));
  }
  return v;
}

struct OracleBlob {
  wvo_blob b{};
  std::vector<uint8_t> raw; std::vector<float> scales, mins;
};
static bool oracle_pack(OracleBlob& o, int format, int dtype, int bw, int rows, int cols, const std::vector<float>& w) {
  uint64_t nraw, ns, nm;
  if (wvo_sizes(format, dtype, bw, rows, cols, &nraw, &ns, &nm)) return false;
  o.raw.assign(nraw, 0); o.scales.assign(ns, 0.f); o.mins.assign(nm, 0.f);
  o.b.format = format; o.b.dtype = dtype; o.b.rows = rows; o.b.cols = cols; o.b.block_weights = bw;
  o.b.raw = o.raw.data(); o.b.nraw = nraw; o.b.scales = o.scales.data(); o.b.ns = ns; o.b.mins = o.mins.data(); o.b.nm = nm;
  return wvo_pack(w.data(), &o.b) == 0;
}

static void host_checks() {
  // Format names are the ENTITY header strings and round-trip through ParseFormatName
  for (int f = 0; f < quant::formatCount; f++)
    CHECK(quant::ParseFormatName(quant::FormatString((quant::Format)f)) == f, "format name %d", f);
  CHECK(std::string(quant::FormatString(quant::FormatQ4_K)) == "Q4_K", "Q4_K name");
  CHECK(quant::ParseFormatName("no-such-format") == quant::FormatNone, "unknown name reads as none");
  CHECK(std::string(core::BackendString(core::BackendCUDA)) == "cuda", "backend name");

  // packed wire: encode -> decode gives the same arrays; truncation is an error
  quant::Blob b;
  b.Format_ = quant::FormatQ4_1; b.Rows = 2; b.Cols = 32;
  b.Raw = {1, 2, 3, 4, 5, 6, 7, 8}; b.Scales = {0.5f, 0.25f}; b.Mins = {-1.f};
  auto [wire, e1] = weights::EncodePackedWire(&b);
  CHECK(!e1 && wire.size() == 12 + 8 + 4 + 8, "wire size %zu", wire.size());
  auto [d, e2] = weights::DecodePackedWire(quant::FormatQ4_1, 2, 32, wire);
  CHECK(!e2 && d && d->Raw == b.Raw && d->Scales == b.Scales && d->Mins == b.Mins, "wire round trip");
  wire.resize(wire.size() - 1);
  auto [d2, e3] = weights::DecodePackedWire(quant::FormatQ4_1, 2, 32, wire);
  CHECK(e3.code == WV_ESHAPE && !d2, "truncated wire must fail");
  // binary blobs re-infer the group from the scale count
  quant::Blob bb;
  bb.Format_ = quant::FormatBinaryPacked; bb.Rows = 1; bb.Cols = 128; bb.Raw.assign(16, 0xff); bb.Scales = {1.f};
  auto [w2, e4] = weights::EncodePackedWire(&bb);
  auto [d3, e5] = weights::DecodePackedWire(quant::FormatBinaryPacked, 1, 128, w2);
  CHECK(!e4 && !e5 && d3->BlockWeights == 128, "g128 inference");

  // argument errors come before any device work
  std::vector<float> x(8), y(1);
  CHECK(quant::MatVec(nullptr, x, y).code == WV_EARG, "nil blob");
  CHECK(quant::MatVec(&b, x, y).code == WV_ESHAPE, "short x");
  CHECK(dense::MatVecPackedBlob(&b, x, y).code == WV_ESHAPE, "short x (dense)");
  auto [p, e6] = quant::Pack(quant::FormatQ4_0, x, 4, 4);
  CHECK(e6.code == WV_ESHAPE && !p, "Pack with too few weights");
  auto [pre, post, e7] = dense::Forward<float>(nullptr, nullptr);
  CHECK(e7.code == WV_EARG, "nil layer");

  // no device: the call fails with the library's error, nothing falls back to the host
  if (cuda::DeviceCount() == 0) {
    Error e = cuda::Init(0);
    CHECK(e.code == WV_EINIT && !e.msg.empty(), "Init without a device -> WV_EINIT (%d)", e.code);
    CHECK(!cuda::Available(), "not available");
    std::vector<float> w(64 * 32, 0.1f);
    auto [q, e8] = quant::Pack(quant::FormatQ8_0, w, 64, 32);
    CHECK(e8.code != 0 && !q, "Pack without a device must fail");
  }
}

static void gpu_checks() {
  Error e = cuda::Init(0);
  if (e) { std::printf("FAIL init: %s\n", e.msg.c_str()); failures++; return; }
  const int rows = 96, cols = 1024;
  const auto w = normal((size_t)rows * cols, 0.02f, 3);
  const auto x = normal(cols, 1.0f, 4);
  struct Case { quant::Format f; int bw; core::DType dt; };
  std::vector<Case> cases;
  for (int f = 1; f < quant::formatCount; f++) cases.push_back({(quant::Format)f, f == quant::FormatAffinePacked ? 64 : 0, core::DTypeFloat32});
  cases.push_back({quant::FormatBinaryPacked, 128, core::DTypeFloat32});
  cases.push_back({quant::FormatNone, 0, core::DTypeFloat32});
  cases.push_back({quant::FormatNone, 0, core::DTypeFloat16});
  cases.push_back({quant::FormatNone, 0, core::DTypeBFloat16});
  for (const Case& c : cases) {
    const char* name = quant::FormatString(c.f);
    auto [b, ep] = quant::Pack(c.f, w, rows, cols, c.bw, c.dt);
    CHECK(!ep && b, "%s: Pack: %s", name, ep.msg.c_str());
    if (!b) continue;
    OracleBlob o;
    CHECK(oracle_pack(o, c.f, c.dt, c.bw, rows, cols, w), "%s: oracle pack", name);
    o.b.block_weights = b->BlockWeights;
    CHECK(b->Raw == o.raw && b->Scales == o.scales && b->Mins == o.mins, "%s bw=%d dt=%d: packed bytes differ from the reference packer's", name, c.bw, c.dt);
    auto [u, eu] = quant::Unpack(b.get());
    std::vector<float> uo((size_t)rows * cols);
    CHECK(!eu && wvo_unpack(&o.b, uo.data()) == 0 && std::memcmp(u.data(), uo.data(), uo.size() * 4) == 0, "%s: Unpack not bit-identical", name);
    std::vector<float> y(rows, -1.f), yo(rows);
    Error em = quant::MatVec(b.get(), x, y);
    std::vector<double> den(rows);
    CHECK(!em && wvo_matvec(&o.b, x.data(), yo.data()) == 0 && wvo_sum_abs_wx(&o.b, x.data(), den.data()) == 0, "%s: MatVec: %s", name, em.msg.c_str());
    double worst = 0;
    for (int r = 0; r < rows; r++) worst = std::fmax(worst, std::fabs((double)y[r] - yo[r]) / std::fmax(den[r], 1e-30));
    CHECK(worst <= 1e-3, "%s: |y - y_ref| / sum|w x| = %.3e", name, worst);  // the reference's stated bound
    // the wire form reaches the same device result
    auto [wire, ew] = weights::EncodePackedWire(b.get());
    auto [b2, ed] = weights::DecodePackedWire(c.f, rows, cols, wire, c.dt);
    CHECK(!ew && !ed && b2, "%s: wire", name);
    if (b2) {
      if (c.f == quant::FormatAffinePacked) b2->BlockWeights = b->BlockWeights;   // not on the wire (Meta is dropped)
      std::vector<float> y2(rows);
      CHECK(!quant::MatVec(b2.get(), x, y2) && y2 == y, "%s: wire blob gives a different y", name);
    }
  }
  // dense.Forward: batch 3, bias + ReLU, Q4_K weights
  {
    auto [l, el] = dense::NewConfigured(cols, rows, core::ActivationReLU, core::DTypeFloat32, quant::FormatQ4_K, &w);
    CHECK(!el && l, "NewConfigured: %s", el.msg.c_str());
    l->Weights->Bias.assign(rows, 0.01);
    auto in = core::NewTensor<float>(3, cols);
    const auto xin = normal((size_t)3 * cols, 1.0f, 9);
    in->Data = xin;
    auto [pre, post, ef] = dense::Forward<float>(l.get(), in.get());
    CHECK(!ef && pre && post && pre->Shape == std::vector<int>({3, rows}), "Forward: %s", ef.msg.c_str());
    OracleBlob o;
    oracle_pack(o, quant::FormatQ4_K, 1, 0, rows, cols, w);
    o.b.block_weights = 256;
    for (int bi = 0; bi < 3 && pre; bi++) {
      std::vector<float> yo(rows); std::vector<double> den(rows);
      wvo_matvec(&o.b, xin.data() + (size_t)bi * cols, yo.data());
      wvo_sum_abs_wx(&o.b, xin.data() + (size_t)bi * cols, den.data());
      for (int r = 0; r < rows; r++) {
        const double want = (double)yo[r] + 0.01;
        CHECK(std::fabs(pre->Data[(size_t)bi * rows + r] - want) <= 1e-3 * den[r] + 1e-6, "Forward pre[%d,%d]", bi, r);
        CHECK(post->Data[(size_t)bi * rows + r] == (pre->Data[(size_t)bi * rows + r] > 0 ? pre->Data[(size_t)bi * rows + r] : 0.f), "Forward post[%d,%d]", bi, r);
      }
    }
    l->Exec.Backend_ = core::BackendSIMD;
    auto [p2, q2, e2] = dense::Forward<float>(l.get(), in.get());
    CHECK(e2.code == WV_EFORMAT && !p2, "a backend this library does not provide must be an error");
    // Store.Pack re-encodes and drops the old device copy
    const uint64_t before = cuda::CacheBytes();
    CHECK(!l->Weights->Pack(quant::FormatQ8_0) && l->Weights->Format_ == quant::FormatQ8_0, "Store.Pack");
    CHECK(cuda::CacheBytes() <= before, "old blob evicted (%llu -> %llu)", (unsigned long long)before, (unsigned long long)cuda::CacheBytes());
  }
  // quant.DecodeRow: a row equals the same row of Unpack; shape and FormatNone errors as in the reference
  {
    auto [b, ep] = quant::Pack(quant::FormatQ4_K, w, rows, cols);
    CHECK(!ep && b, "Pack for DecodeRow");
    if (b) {
      auto [all, eu] = quant::Unpack(b.get());
      std::vector<float> row(cols + 2, -1.f);
      CHECK(!eu && !quant::DecodeRow(b.get(), 3, row), "DecodeRow");
      bool same = !eu;
      for (int c = 0; c < cols && same; c++) same = std::memcmp(&row[c], &all[(size_t)3 * cols + c], 4) == 0;
      CHECK(same && row[cols] == -1.f, "DecodeRow row 3 equals Unpack row 3");
      std::vector<float> small(cols - 1);
      CHECK(quant::DecodeRow(b.get(), 0, small).code == WV_ESHAPE, "short dst");
      CHECK(quant::DecodeRow(b.get(), rows, row).code == WV_ESHAPE, "row out of range");
      CHECK(quant::DecodeRow(nullptr, 0, row).code == WV_EFORMAT, "nil blob");
    }
    auto [bn, en] = quant::Pack(quant::FormatNone, w, rows, cols);
    std::vector<float> row(cols);
    CHECK(!en && bn && quant::DecodeRow(bn.get(), 0, row).code == WV_EFORMAT, "FormatNone is refused");
  }
  // cache budget: beyond the limit an upload is WV_ENOMEM, the reference's VRAM-full sentinel
  {
    cuda::Clear();
    cuda::SetCacheLimit(1024);
    auto [b, ep] = quant::Pack(quant::FormatQ8_0, w, rows, cols);
    std::vector<float> y(rows);
    Error em = b ? quant::MatVec(b.get(), x, y) : ep;
    CHECK(cuda::IsVRAMFull(em), "cache limit -> WV_ENOMEM (got %d)", em.code);
    cuda::SetCacheLimit(0);
    CHECK(b && !quant::MatVec(b.get(), x, y), "works again without the limit");
  }
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "host";
  host_checks();
  if (mode == "gpu") gpu_checks();
  std::printf("%s: %d failure(s)\n", mode.c_str(), failures);
  return failures ? 1 : 0;
}
