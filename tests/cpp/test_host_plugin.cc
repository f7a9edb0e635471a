// Drives the C++ host side of the plugin (spoc_b200/host/sarek_b200.hpp) the way the reference's
// own tests and benchmarks drive a backend: kernels as IR, vectors, run_vectors, then verification
// against a host baseline with the reference's tolerances.
//
//   test_host_plugin cpu <dir-with-ir-files>     no GPU needed: recognition, fusion, error behaviour
//   test_host_plugin gpu <dir-with-ir-files>     runs the kernels on device 0
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../spoc_b200/host/sarek_b200.hpp"

using namespace sarek_b200;

static int failures = 0;
#define EXPECT(cond)                                                        \
  do {                                                                      \
    if (!(cond)) {                                                          \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);         \
      ++failures;                                                           \
    }                                                                       \
  } while (0)

static std::string slurp(const std::string& path) {
  std::ifstream f(path);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

static int run_cpu(const std::string& dir) {
  Backend b;
  const Backend::DeviceT fake{0, "none", 0, 10, 0, 148};
  // recognition needs no device
  auto k = b.Kernel.compile(fake, "sarek_kern", slurp(dir + "/vector_add.ir"));
  EXPECT(b.Kernel.kind(k) == SB200_KIND_MAP);
  EXPECT(b.Kernel.describe(k).find("vector_add") != std::string::npos);
  k = b.Kernel.compile(fake, "sarek_kern", slurp(dir + "/matmul_tiled.ir"));
  EXPECT(b.Kernel.kind(k) == SB200_KIND_GEMM_TILED);
  k = b.Kernel.compile(fake, "sarek_kern", slurp(dir + "/matmul_naive.ir"));
  EXPECT(b.Kernel.kind(k) == SB200_KIND_GEMM_NAIVE);
  k = b.Kernel.compile(fake, "sarek_kern", slurp(dir + "/dot_product.ir"));
  EXPECT(b.Kernel.kind(k) == SB200_KIND_BLOCK_REDUCE);
  // unrecognised IR is Unsupported_construct, malformed IR a plain backend error
  bool unsupported = false, parse_error = false;
  try {
    b.Kernel.compile(fake, "k", "(kernel k (params (vec a 1 f32)) (body (while (const bool true) (empty))))");
  } catch (const UnsupportedConstruct& e) {
    unsupported = e.code == SB200_ERR_UNSUPPORTED;
  }
  try {
    b.Kernel.compile(fake, "k", "(kernel");
  } catch (const UnsupportedConstruct&) {
  } catch (const BackendError& e) {
    parse_error = e.code == SB200_ERR_PARSE;
  }
  EXPECT(unsupported);
  EXPECT(parse_error);
  // fusion of the a = b + 3c ; d = a*a + b chain, as sarek/tests/e2e/test_fusion_api.ml drives the pass
  const std::string prod = slurp(dir + "/triad_producer.ir"), cons = slurp(dir + "/square_add_consumer.ir");
  EXPECT(!fusion::can_fuse(prod, cons, "a"));  // two reads of `a`: a stencil for the reference
  std::string fused;
  EXPECT(fusion::try_fuse_all(prod, cons, "a", &fused));
  EXPECT(fused.find("(read a") == std::string::npos);
  EXPECT(fusion::fuse(prod, cons, "a").find("square_add_fused") != std::string::npos);
  // the guarded kernel form of the benchmarks: the reference's pass gives the consumer back, the backend's fuses it
  const std::string gprod = slurp(dir + "/stream_triad.ir"), gcons = slurp(dir + "/square_add_guarded.ir");
  EXPECT(fusion::fuse(gprod, gcons, "a").find("(read a") != std::string::npos);
  std::string gfused;
  EXPECT(fusion::fuse_guarded(gprod, gcons, "a", &gfused));
  EXPECT(gfused.find("(read a") == std::string::npos && gfused.find("(kernel square_add_fused") == 0);
  EXPECT(!fusion::fuse_guarded(gprod, cons, "a", &gfused));  // unguarded consumer behind a guarded producer
  // argument binding errors come before any device work
  bool args_error = false;
  try {
    auto kt = b.Kernel.compile_cached(fake, "sarek_kern", slurp(dir + "/stream_triad.ir"));
    auto ka = b.Kernel.create_args();
    b.Kernel.set_arg_int32(ka, 0, 3);
    b.Kernel.launch(kt, ka, dims1d(1), dims1d(32), 0);
  } catch (const BackendError& e) {
    args_error = e.code == SB200_ERR_ARGS;
  }
  EXPECT(args_error);
  if (!b.is_available()) {
    bool no_device = false;
    try {
      b.Device.init();
    } catch (const BackendError& e) {
      no_device = e.code == SB200_ERR_NO_DEVICE;
    }
    EXPECT(no_device);  // no CPU fallback: the absence of a GPU is an error
  }
  return failures;
}

static int run_gpu(const std::string& dir) {
  Backend b;
  b.Device.init();
  EXPECT(b.Device.count() > 0);
  const Backend::DeviceT dev = b.Device.get(0);
  b.Device.set_current(dev);

  {  // stream_triad: benchmarks/bench_stream_triad.ml:44-49,122-140 (tolerance 1e-5)
    const int n = 100000;
    std::vector<float> hb(n), hc(n);
    std::vector<double> expected(n);
    for (int i = 0; i < n; ++i) {
      const double bv = (i % 100) / 100.0, cv = ((i + 1) % 100) / 100.0;
      hb[i] = static_cast<float>(bv);
      hc[i] = static_cast<float>(cv);
      expected[i] = bv + cv * 3.0;
    }
    Vector va(b, n), vb(b, hb), vc(b, hc);
    run_vectors(b, dev, slurp(dir + "/stream_triad.ir"),
                {&va, &vb, &vc, ScalarArg::float32(3.0f), ScalarArg::int32(n)}, dims1d(256), dims1d((n + 255) / 256));
    b.Device.synchronize(dev);
    EXPECT(va.location() == Vector::Stale_CPU && vb.location() == Vector::Stale_CPU);
    const auto& got = va.to_array();
    double worst = 0;
    for (int i = 0; i < n; ++i) worst = std::fmax(worst, std::fabs(got[i] - expected[i]));
    EXPECT(worst <= 1e-5);
  }
  {  // the reference's timing protocol at its small benchmark size: 5 warm-ups, 20 x (launch + synchronise), median
    const int n = 1000000;
    Vector va(b, size_t(n)), vb(b, std::vector<float>(n, 0.5f)), vc(b, std::vector<float>(n, 0.25f));
    const std::string ir = slurp(dir + "/stream_triad.ir");
    std::vector<double> us;
    for (int it = 0; it < 25; ++it) {
      const auto t0 = std::chrono::steady_clock::now();
      run_vectors(b, dev, ir, {&va, &vb, &vc, ScalarArg::float32(3.0f), ScalarArg::int32(n)}, dims1d(256), dims1d((n + 255) / 256));
      b.Device.synchronize(dev);
      const auto t1 = std::chrono::steady_clock::now();
      if (it >= 5) us.push_back(std::chrono::duration<double, std::micro>(t1 - t0).count());
    }
    std::sort(us.begin(), us.end());
    std::printf("stream_triad n=1000000 launch+synchronise through run_vectors (C++ host): median %.1f us, min %.1f us\n",
                us[us.size() / 2], us.front());
    EXPECT(va.to_array()[n - 1] == 0.5f + 0.25f * 3.0f);
  }
  for (const char* file : {"/matmul_naive.ir", "/matmul_tiled.ir"}) {
    // benchmarks/bench_matrix_mul_tiled.ml:41-52,109-112,194-212 (tolerance 1e-3)
    const int m = 64, n = 48, k = 80;
    std::vector<double> a(m * k), bb(k * n), expected(m * n, 0.0);
    for (int i = 0; i < m * k; ++i) a[i] = (i % 10) / 10.0;
    for (int i = 0; i < k * n; ++i) bb[i] = ((i + 1) % 10) / 10.0;
    for (int row = 0; row < m; ++row)
      for (int col = 0; col < n; ++col) {
        double sum = 0.0;
        for (int i = 0; i < k; ++i) sum += a[row * k + i] * bb[i * n + col];
        expected[row * n + col] = sum;
      }
    Vector va(b, std::vector<float>(a.begin(), a.end())), vb(b, std::vector<float>(bb.begin(), bb.end())), vc(b, size_t(m) * n);
    const bool tiled = std::string(file).find("tiled") != std::string::npos;
    run_vectors(b, dev, slurp(dir + file), {&va, &vb, &vc, ScalarArg::int32(m), ScalarArg::int32(n), ScalarArg::int32(k)},
                tiled ? dims2d(16, 16) : dims1d(256), tiled ? dims2d((n + 15) / 16, (m + 15) / 16) : dims1d((m * n + 255) / 256),
                tiled ? 2 * 16 * 16 * 4 : 0);
    const auto& got = vc.to_array();
    double worst = 0;
    for (int i = 0; i < m * n; ++i) worst = std::fmax(worst, std::fabs(got[i] - expected[i]));
    EXPECT(worst <= 1e-3);
  }
  {  // vectors of 16 MiB: pageable on the first launch, pinned in place from the second transfer on, after which the
     // launch call pipelines the uploads with the GEMM and sends the result back behind it; same bits every time
    const int m = 2048, n = 2048, k = 2048;
    std::vector<float> a(size_t(m) * k), bb(size_t(k) * n);
    for (size_t i = 0; i < a.size(); ++i) a[i] = static_cast<float>((i * 7 % 13) / 13.0 - 0.4);
    for (size_t i = 0; i < bb.size(); ++i) bb[i] = static_cast<float>((i * 5 % 11) / 11.0 - 0.5);
    Vector va(b, a), vb(b, bb), vc(b, size_t(m) * n);
    const std::string ir = slurp(dir + "/matmul_naive.ir");
    std::vector<float> first;
    for (int rep = 0; rep < 4; ++rep) {
      va.set(0, a[0]);  // the host copies are the valid ones again: the next launch uploads them
      vb.set(0, bb[0]);
      run_vectors(b, dev, ir, {&va, &vb, &vc, ScalarArg::int32(m), ScalarArg::int32(n), ScalarArg::int32(k)}, dims1d(256),
                  dims1d((m * n + 255) / 256));
      const auto& got = vc.to_array();
      if (rep == 0) first = got;
      EXPECT(std::memcmp(first.data(), got.data(), first.size() * sizeof(float)) == 0);
    }
    double worst = 0;
    for (int row = 0; row < m; row += 191)
      for (int col = 0; col < n; col += 53) {
        double sum = 0.0;
        for (int i = 0; i < k; ++i) sum += double(a[size_t(row) * k + i]) * double(bb[size_t(i) * n + col]);
        worst = std::fmax(worst, std::fabs(first[size_t(row) * n + col] - sum));
      }
    EXPECT(worst <= 1e-3);
  }
  {  // a group of one GPU: the sharded product on host operands against the reference's host baseline
    const int m = 300, n = 48, k = 80;
    std::vector<float> a(m * k), bb(k * n), d(size_t(m) * n, -1.0f);
    for (int i = 0; i < m * k; ++i) a[i] = static_cast<float>((i % 10) / 10.0);
    for (int i = 0; i < k * n; ++i) bb[i] = static_cast<float>(((i + 1) % 10) / 10.0);
    DeviceGroup grp({dev.id});
    EXPECT(grp.size() == 1 && grp.row_block(m, 0).second == m);
    grp.gemm_host(SB200_MODE_3XTF32, m, n, k, a.data(), bb.data(), d.data());
    double worst = 0;
    for (int row = 0; row < m; row += 37)
      for (int col = 0; col < n; ++col) {
        double sum = 0.0;
        for (int i = 0; i < k; ++i) sum += double(a[row * k + i]) * double(bb[i * n + col]);
        worst = std::fmax(worst, std::fabs(d[size_t(row) * n + col] - sum));
      }
    EXPECT(worst <= 1e-3);
    bool threw = false;
    try {
      DeviceGroup bad({dev.id, dev.id});
    } catch (const BackendError& e) {
      threw = e.code == SB200_ERR_INVALID_VALUE;
    }
    EXPECT(threw);
  }
  {  // event timing and an explicit stream, as Spoc_core.Profiling uses them
    auto e0 = b.Event.create(), e1 = b.Event.create();
    auto s = b.Stream.default_stream(dev);
    b.Event.record(e0, s);
    b.Event.record(e1, s);
    b.Event.synchronize(e1);
    EXPECT(b.Event.elapsed(e0, e1) >= 0.0f);
    b.Event.destroy(e0);
    b.Event.destroy(e1);
  }
  return failures;
}

int main(int argc, char** argv) {
  if (argc < 3) {
    std::printf("usage: %s cpu|gpu <ir-dir>\n", argv[0]);
    return 2;
  }
  int rc = 1;
  try {
    rc = std::string(argv[1]) == "gpu" ? run_gpu(argv[2]) : run_cpu(argv[2]);
  } catch (const std::exception& e) {
    std::printf("EXCEPTION: %s\n", e.what());
    return 1;
  }
  std::printf(rc == 0 ? "ALL PASSED\n" : "%d FAILURE(S)\n", rc);
  return rc == 0 ? 0 : 1;
}
