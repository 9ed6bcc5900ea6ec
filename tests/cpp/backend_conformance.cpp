// Drives the C++ CudaBackend through the reference's own interfaces: the
// Backend class (include/tessera/backend.hpp), the launch helpers of
// src/core/decode_internal.hpp (GemmFor, ProjectDevice, ProjectTiledDevice,
// GemmVecSplit, GemmRowsKernelName, CachedKernel) and the cross-device helpers
// of src/core/buffer.cpp (CopyAcrossDevices, AllReduceSum), and checks every
// result against the reference's host functions (src/core/numerics).
//
// Built by tessera_b200/backend/Makefile where the reference checkout is
// present; tests/test_backend_conformance.py runs the binary on a GPU.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <span>
#include <string>
#include <vector>

#include "core/decode_internal.hpp"
#include "core/numerics/gemm.hpp"
#include "core/numerics/quant.hpp"
#include "tessera/backend.hpp"

using namespace tessera;
namespace cd = tessera::core::detail;

namespace {

int g_failures = 0;

void Report(const std::string& name, bool ok, double value = 0.0) {
  std::printf("%s %s %.3e\n", ok ? "PASS" : "FAIL", name.c_str(), value);
  if (!ok) ++g_failures;
}

double RelErr(const std::vector<float>& y, const std::vector<float>& r) {
  double num = 0, den = 1e-30;
  for (std::size_t i = 0; i < y.size(); ++i) {
    num = std::max(num, std::fabs(static_cast<double>(y[i]) - r[i]));
    den = std::max(den, std::fabs(static_cast<double>(r[i])));
  }
  return num / den;
}

template <typename T>
std::span<const std::byte> Bytes(const std::vector<T>& v) {
  return {reinterpret_cast<const std::byte*>(v.data()), v.size() * sizeof(T)};
}

template <typename T>
std::unique_ptr<Buffer> Upload(Backend& b, const std::vector<T>& v) {
  auto buf = b.AllocateBuffer(v.size() * sizeof(T), MemoryKind::Device);
  if (!buf || !b.CopyH2D(**buf, Bytes(v))) return nullptr;
  return std::move(*buf);
}

std::vector<float> Download(Backend& b, const Buffer& buf, std::size_t count) {
  std::vector<float> out(count);
  if (!b.CopyD2H(buf, reinterpret_cast<std::byte*>(out.data()), count * 4)) out.clear();
  return out;
}

std::vector<float> Normal(std::size_t n, unsigned seed, float scale = 1.0f) {
  std::mt19937 g(seed);
  std::normal_distribution<float> d(0.0f, scale);
  std::vector<float> v(n);
  for (auto& x : v) x = d(g);
  return v;
}

// Q4_K weights through the reference's own fixture quantiser.
std::vector<std::byte> MakeQ4K(std::size_t n, std::size_t k, unsigned seed) {
  const auto w = Normal(n * k, seed, 0.05f);
  std::vector<std::byte> out(n * (k / 256) * 144);
  for (std::size_t b = 0; b < n * (k / 256); ++b)
    core::QuantizeQ4K(std::span<const float>(w.data() + b * 256, 256), out.data() + b * 144);
  return out;
}

std::vector<std::byte> MakeQ6K(std::size_t n, std::size_t k, unsigned seed) {
  std::mt19937 g(seed);
  std::vector<std::byte> out(n * (k / 256) * 210);
  for (std::size_t b = 0; b < n * (k / 256); ++b) {
    std::byte* blk = out.data() + b * 210;
    for (int i = 0; i < 192; ++i) blk[i] = static_cast<std::byte>(g() & 0xFF);
    for (int i = 192; i < 208; ++i) blk[i] = static_cast<std::byte>(static_cast<int>(g() % 96) - 48);
    const std::uint16_t d = core::Fp16FromFloat(1.0e-4f * (1 + g() % 4));
    blk[208] = static_cast<std::byte>(d & 0xFF);
    blk[209] = static_cast<std::byte>(d >> 8);
  }
  return out;
}

std::vector<std::byte> MakeMxFp4(std::size_t n, std::size_t k, unsigned seed) {
  std::mt19937 g(seed);
  std::vector<std::byte> out(n * k / 2 + n * k / 32);
  for (std::size_t i = 0; i < n * k / 2; ++i) out[i] = static_cast<std::byte>(g() & 0xFF);
  for (std::size_t i = 0; i < n * k / 32; ++i) out[n * k / 2 + i] = static_cast<std::byte>(127 - g() % 9);
  return out;
}

// The split-K sequence of ProjectGemvDevice (src/models/qwen3_5/internal.hpp:104-145).
bool ProjectGemv(Backend& b, core::KernelCache& cache, const Kernel& gemm, const Buffer& a,
                 const Buffer& w, Buffer& out, std::size_t m, std::size_t n, std::size_t k) {
  const std::size_t total = m * n;
  const std::size_t split = cd::GemmVecSplit(total, k);
  if (split <= 1) return cd::ProjectDevice(b, gemm, a, w, out, m, n, k).has_value();
  auto part = b.AllocateBuffer(split * total * 4, MemoryKind::Device);
  auto reduce = cd::CachedKernel(b, cache, 0x7001, "gemm_vec_reduce");
  if (!part || !reduce) return false;
  KernelLaunch launch;
  launch.grid_x = static_cast<std::uint32_t>((total + 7) / 8);
  launch.grid_y = static_cast<std::uint32_t>(split);
  launch.buffers = {&a, &w, part->get()};
  launch.scalars = {m, n, k, split};
  if (!b.LaunchKernel(gemm, launch)) return false;
  KernelLaunch red;
  red.grid_x = static_cast<std::uint32_t>((total + 255) / 256);
  red.buffers = {part->get(), &out};
  red.scalars = {total, split};
  const bool ok = b.LaunchKernel(**reduce, red).has_value();
  b.Synchronize();
  return ok;
}

void BlockFormat(Backend& b, DType dtype, const char* tag, const std::vector<std::byte>& w,
                 std::size_t n, std::size_t k) {
  // the reference keeps the GEMV ids and the tiled ids in separate caches
  // (Qwen35State::gemms and ::gemm_tiled); the keys overlap by design
  core::KernelCache cache, tiled_cache;
  auto wb = Upload(b, w);
  for (std::size_t m : {1, 3, 4, 5, 17, 32, 64}) {
    const auto a = Normal(m * k, 100 + static_cast<unsigned>(m));
    std::vector<float> ref(m * n);
    if (dtype == DType::Q4K) {
      (void)core::GemmQ4KRef(a, w, ref, m, n, k);
    } else {
      (void)core::GemmQ6KRef(a, w, ref, m, n, k);
    }
    auto ab = Upload(b, a);
    auto out = b.AllocateBuffer(m * n * 4, MemoryKind::Device);
    bool ok = false;
    std::string id;
    const auto rows_name = cd::GemmRowsKernelName(dtype, m);
    if (m >= 2 && m <= 5 && !rows_name.empty()) {
      auto rows = cd::CachedKernel(b, cache, 0x1000 + static_cast<int>(m), rows_name);
      if (rows) {
        id = std::string((*rows)->Id());
        KernelLaunch launch;
        launch.grid_x = static_cast<std::uint32_t>((n + 7) / 8);
        launch.buffers = {ab.get(), wb.get(), out->get()};
        launch.scalars = {m, n, k, 1};
        ok = b.LaunchKernel(**rows, launch).has_value();
      }
    } else if (m >= cd::kGemmWmmaMinRows) {
      auto wmma = cd::GemmWmmaFor(b, tiled_cache, dtype);
      if (wmma) {
        id = std::string((*wmma)->Id());
        ok = cd::ProjectTiledDevice(b, **wmma, *ab, *wb, **out, m, n, k).has_value();
      }
    } else if (m >= 16) {
      auto tiled = cd::GemmTiledFor(b, tiled_cache, dtype);
      if (tiled) {
        id = std::string((*tiled)->Id());
        ok = cd::ProjectTiledDevice(b, **tiled, *ab, *wb, **out, m, n, k).has_value();
      }
    } else {
      auto gemm = cd::GemmFor(b, cache, dtype);
      if (gemm) {
        id = std::string((*gemm)->Id());
        ok = ProjectGemv(b, cache, **gemm, *ab, *wb, **out, m, n, k);
      }
    }
    const auto got = Download(b, **out, m * n);
    const double err = ok && !got.empty() ? RelErr(got, ref) : 1.0;
    Report(std::string(tag) + " m=" + std::to_string(m) + " " + id, ok && err < 2e-3, err);
  }
}

}  // namespace

int main() {
  auto names = ListGpuNames();
  Report("ListGpuNames", names.has_value() && !names->empty());
  if (!names) return 1;
  std::printf("device 0: %s\n", (*names)[0].c_str());
  auto backend = CreateBackend();
  Report("CreateBackend", backend != nullptr && backend->Name() == "cuda");
  log::Diagnostics diag;
  backend->SetDiagnostics(&diag);
  backend->SetDeviceIndex(static_cast<int>(names->size()) + 3);
  auto bad = backend->Init();
  Report("Init rejects an out-of-range device", !bad && bad.error() == StatusCode::InvalidArgument);
  backend->SetDeviceIndex(0);
  Report("Init", backend->Init().has_value() && backend->Init().has_value());
  Backend& b = *backend;
  Report("MemoryInfo", b.MemoryInfo().total_bytes > 0);

  auto zero = b.AllocateBuffer(0, MemoryKind::Device);
  Report("AllocateBuffer(0) is InvalidArgument", !zero && zero.error() == StatusCode::InvalidArgument);
  auto miss = b.LoadKernel("layernorm", {});
  Report("unknown id is UnsupportedFeature", !miss && miss.error() == StatusCode::UnsupportedFeature);
  const std::byte code[1] = {std::byte{1}};
  auto module = b.LoadKernel("gemm_q4k_vec", code);
  Report("kernel modules are UnsupportedFeature", !module && module.error() == StatusCode::UnsupportedFeature);

  const std::size_t n = 200, k = 1024;
  BlockFormat(b, DType::Q4K, "q4k", MakeQ4K(n, k, 1), n, k);
  BlockFormat(b, DType::Q6K, "q6k", MakeQ6K(n, k, 2), n, k);

  {  // MXFP4: plain and W4A8 tensor-core contract
    core::KernelCache cache;
    const auto w = MakeMxFp4(n, k, 3);
    const std::span<const std::byte> blob(w.data(), n * k / 2), scales(w.data() + n * k / 2, n * k / 32);
    auto wb = Upload(b, w);
    for (std::size_t m : {1, 7, 16}) {
      const auto a = Normal(m * k, 200 + static_cast<unsigned>(m));
      std::vector<float> ref(m * n);
      (void)core::GemmMxFp4Ref(a, blob, scales, ref, m, n, k);
      auto ab = Upload(b, a);
      auto out = b.AllocateBuffer(m * n * 4, MemoryKind::Device);
      auto gemm = m == 1 ? cd::GemmFor(b, cache, DType::F4E2M1)
                         : cd::CachedKernel(b, cache, 0x2000, "gemm_mxfp4_rows");
      bool ok = gemm && cd::ProjectDevice(b, **gemm, *ab, *wb, **out, m, n, k).has_value();
      const auto got = Download(b, **out, m * n);
      const double err = ok ? RelErr(got, ref) : 1.0;
      Report("mxfp4 m=" + std::to_string(m), ok && err < 2e-3, err);

      // quantize_fp8_pack_rows + mxfp4_row_ref + gemm_mxfp4_wmma (project.cpp:92-231)
      std::vector<std::byte> a8(m * k), fold(n * k), wref(n);
      std::vector<float> as(m), ref8(m * n);
      (void)core::QuantizeFp8PackRef(a, a8, as, m, k);
      (void)core::FoldMxFp4ToFp8(blob, scales, fold, wref, n, k);
      (void)core::GemmMxFp4Fp8Ref(a8, as, fold, wref, ref8, m, n, k);
      auto k_pack = b.LoadKernel("quantize_fp8_pack_rows", {});
      auto k_ref = b.LoadKernel("mxfp4_row_ref", {});
      auto k_mma = b.LoadKernel("gemm_mxfp4_wmma", {});
      auto d_a8 = b.AllocateBuffer(m * k, MemoryKind::Device);
      auto d_as = b.AllocateBuffer(m * 4, MemoryKind::Device);
      auto d_wref = b.AllocateBuffer(n, MemoryKind::Device);
      ok = k_pack && k_ref && k_mma;
      if (ok) {
        KernelLaunch l1;
        l1.grid_x = static_cast<std::uint32_t>(m);
        l1.block_x = 1024;
        l1.buffers = {ab.get(), d_a8->get(), d_as->get()};
        l1.scalars = {m, k};
        KernelLaunch l2;
        l2.grid_x = static_cast<std::uint32_t>((n + 255) / 256);
        l2.buffers = {wb.get(), d_wref->get()};
        l2.scalars = {n, k};
        KernelLaunch l3;
        l3.grid_x = static_cast<std::uint32_t>((n + 63) / 64);
        l3.block_x = 128;
        l3.buffers = {d_a8->get(), wb.get(), d_as->get(), d_wref->get(), out->get()};
        l3.scalars = {m, n, k, 1, 0};
        ok = b.LaunchKernel(**k_pack, l1) && b.LaunchKernel(**k_ref, l2) && b.LaunchKernel(**k_mma, l3);
      }
      const auto got8 = Download(b, **out, m * n);
      const double err8 = ok ? RelErr(got8, ref8) : 1.0;
      Report("w4a8 m=" + std::to_string(m), ok && err8 < 2e-3, err8);
    }
  }

  {  // per-token FP8 quantise-dequantise and bf16 rounding, bit exact
    const std::size_t rows = 5, cols = 1536;
    auto x = Normal(rows * cols, 7, 3.0f);
    for (std::size_t c = 0; c < cols; ++c) x[cols + c] = 0.0f;
    std::vector<float> ref = x, scale_ref(rows);
    (void)core::QuantizeFp8Ref(ref, scale_ref, rows, cols);
    auto d = Upload(b, x);
    auto s = b.AllocateBuffer(rows * 4, MemoryKind::Device);
    auto kq = b.LoadKernel("quantize_fp8", {});
    KernelLaunch l;
    l.grid_x = static_cast<std::uint32_t>(rows);
    l.buffers = {d.get(), s->get()};
    l.scalars = {rows, cols};
    bool ok = kq && b.LaunchKernel(**kq, l).has_value();
    const auto got = Download(b, *d, rows * cols), gs = Download(b, **s, rows);
    ok = ok && std::memcmp(got.data(), ref.data(), ref.size() * 4) == 0 &&
         std::memcmp(gs.data(), scale_ref.data(), rows * 4) == 0;
    Report("quantize_fp8 bit exact", ok);
    std::vector<float> r2 = x;
    (void)core::RoundBf16Ref(r2);
    auto d2 = Upload(b, x);
    auto kr = b.LoadKernel("round_bf16", {});
    ok = kr && cd::RoundBf16Device(b, **kr, *d2, rows * cols).has_value();
    const auto got2 = Download(b, *d2, rows * cols);
    Report("round_bf16 bit exact", ok && std::memcmp(got2.data(), r2.data(), r2.size() * 4) == 0);
  }

  {  // two backends: CopyAcrossDevices, AllReduceSum and the rank-0 reduce of TpReduce
    auto second = CreateBackend();
    second->SetDeviceIndex(names->size() > 1 ? 1 : 0);
    bool ok = second->Init().has_value();
    const std::size_t hidden = 5120;
    const auto p0 = Normal(hidden, 11), p1 = Normal(hidden, 12);
    auto b0 = Upload(b, p0);
    auto b1 = Upload(*second, p1);
    auto scratch = b.AllocateBuffer(hidden * 4, MemoryKind::Device);
    auto add = b.LoadKernel("add", {});
    ok = ok && add && CopyAcrossDevices(*b1, 0, **scratch, 0, hidden * 4).has_value();
    KernelLaunch l;
    l.grid_x = static_cast<std::uint32_t>((hidden + 255) / 256);
    l.buffers = {b0.get(), scratch->get(), b0.get()};
    l.scalars = {hidden};
    ok = ok && b.LaunchKernel(**add, l).has_value();
    ok = ok && CopyAcrossDevices(*b0, 0, *b1, 0, hidden * 4).has_value();
    const auto r0 = Download(b, *b0, hidden), r1 = Download(*second, *b1, hidden);
    bool same = ok && r0 == r1;
    for (std::size_t i = 0; same && i < hidden; ++i) same = r0[i] == p0[i] + p1[i];
    Report("TpReduce sequence (peer copy, add, broadcast)", same);
    auto c0 = Upload(b, p0);
    auto c1 = Upload(*second, p1);
    Buffer* both[2] = {c0.get(), c1.get()};
    ok = AllReduceSum(both, hidden * 4).has_value();
    const auto s0 = Download(b, *c0, hidden), s1 = Download(*second, *c1, hidden);
    same = ok && s0 == s1;
    for (std::size_t i = 0; same && i < hidden; ++i) same = s0[i] == p0[i] + p1[i];
    Report("AllReduceSum", same);
  }
  b.Synchronize();
  std::printf("%s (%d failures)\n", g_failures == 0 ? "ALL PASS" : "FAILED", g_failures);
  return g_failures == 0 ? 0 : 1;
}
