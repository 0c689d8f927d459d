// The C++ host layer (anode_b200/host/anode_ops.hpp) on a GPU, checked against the CPU oracle
// (oracle/bn_oracle.c).  Written the way the reference tests its operators (tests/test_gpu.rs:
// build the op, run it, read the value back, compare): one function per behaviour, exit code 0
// when all pass.  Tolerance: |got - want| <= 1e-5 + 1e-4*|want|; elements whose pre-activation is
// within 1e-5 of zero are skipped in y / dx (the ReLU mask there depends on the last bit of the
// statistics).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <string>
#include <vector>

#include "../../anode_b200/host/anode_ops.hpp"

extern "C" {
void oracle_bn_relu_fwd_bwd_f32(uint32_t dim0, uint32_t dim1, uint32_t dim2, float epsilon, float avg_rate, const float *x,
                                const float *dy, const float *gamma, const float *beta, float *run_mean, float *run_var, float *y,
                                float *dx, float *mean, float *var, float *dgamma, float *dbeta, float *xhat, float *dz,
                                uint32_t block_sz);
void oracle_bn_relu_fwd_bwd_f64(uint32_t dim0, uint32_t dim1, uint32_t dim2, double epsilon, double avg_rate, const float *x,
                                const float *dy, const float *gamma, const float *beta, double *run_mean, double *run_var, double *y,
                                double *dx, double *mean, double *var, double *dgamma, double *dbeta);
}

using namespace anode;

static int g_checks = 0;
struct Failure { std::string what; };
#define EXPECT(cond, msg) do { ++g_checks; if (!(cond)) throw Failure{std::string(msg) + " [" #cond "]"}; } while (0)

// seeded N(loc, scale) by Box-Muller over a 64-bit LCG; U(lo, hi) from the same stream
struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 6364136223846793005ull + 1442695040888963407ull) {}
  double uni() { s = s * 6364136223846793005ull + 1442695040888963407ull; return ((s >> 11) + 0.5) / 9007199254740992.0; }
  double normal() { const double u = uni(), v = uni(); return std::sqrt(-2.0 * std::log(u)) * std::cos(6.283185307179586 * v); }
};
static std::vector<float> normals(size_t n, Rng &r, double loc, double scale)
{
  std::vector<float> v(n);
  for (auto &e : v) e = (float)(loc + scale * r.normal());
  return v;
}
static std::vector<float> uniforms(size_t n, Rng &r, double lo, double hi)
{
  std::vector<float> v(n);
  for (auto &e : v) e = (float)(lo + (hi - lo) * r.uni());
  return v;
}

template <typename T>
static void expect_close(const std::vector<float> &got, const std::vector<T> &want, const char *what, const std::vector<char> *skip = nullptr,
                         double rtol = 1e-4, double atol = 1e-5)
{
  EXPECT(got.size() == want.size(), what);
  for (size_t i = 0; i < got.size(); ++i) {
    if (skip && (*skip)[i]) continue;
    const double w = (double)want[i], g = (double)got[i];
    if (!(std::fabs(g - w) <= atol + rtol * std::fabs(w))) {
      char buf[256];
      snprintf(buf, sizeof(buf), "%s: element %zu got %.9g want %.9g", what, i, g, w);
      throw Failure{buf};
    }
  }
  ++g_checks;
}
static void expect_sum_close(const std::vector<float> &got, const std::vector<double> &want, const char *what)
{
  double ms = 0.0;
  for (double w : want) ms += w * w;
  const double rms = want.empty() ? 0.0 : std::sqrt(ms / want.size());
  expect_close(got, want, what, nullptr, 1e-4, 1e-5 + 1e-4 * rms);
}

struct Problem {
  std::vector<uint32_t> size;        // [spatial..., C, N]
  uint32_t dim0, c, n;
  std::vector<float> x, dy, gamma, beta;
  std::vector<int> axes;
};
static Problem make_problem(std::vector<uint32_t> size, uint64_t seed, double loc, double scale)
{
  Problem p;
  p.size = size;
  p.dim0 = 1;
  for (size_t i = 0; i + 2 < size.size(); ++i) { p.dim0 *= size[i]; p.axes.push_back((int)i); }
  p.c = size[size.size() - 2]; p.n = size[size.size() - 1];
  Rng r(seed);
  const size_t len = (size_t)p.dim0 * p.c * p.n;
  p.x = normals(len, r, loc, scale);
  p.dy = normals(len, r, 0.0, 1.0);
  p.gamma = uniforms(p.c, r, 0.5, 1.5);
  p.beta = uniforms(p.c, r, -0.1, 0.1);
  return p;
}

struct Truth { std::vector<double> y, dx, mean, var, run_mean, run_var, dgamma, dbeta; std::vector<char> borderline; };
static Truth truth_f64(const Problem &p, bool affine)
{
  const size_t len = p.x.size();
  Truth t;
  t.y.resize(len); t.dx.resize(len); t.mean.resize(p.c); t.var.resize(p.c); t.dgamma.resize(p.c); t.dbeta.resize(p.c);
  t.run_mean.assign(p.c, 0.0); t.run_var.assign(p.c, 1.0);
  oracle_bn_relu_fwd_bwd_f64(p.dim0, p.c, p.n, 1e-5, 0.1, p.x.data(), p.dy.data(), affine ? p.gamma.data() : nullptr,
                             affine ? p.beta.data() : nullptr, t.run_mean.data(), t.run_var.data(), t.y.data(), t.dx.data(), t.mean.data(),
                             t.var.data(), t.dgamma.data(), t.dbeta.data());
  t.borderline.resize(len);
  for (uint32_t n = 0; n < p.n; ++n)
    for (uint32_t c = 0; c < p.c; ++c)
      for (uint32_t i = 0; i < p.dim0; ++i) {
        const size_t at = i + (size_t)p.dim0 * (c + (size_t)p.c * n);
        const double g = affine ? p.gamma[c] : 1.0, b = affine ? p.beta[c] : 0.0;
        const double pre = g * ((double)p.x[at] - t.mean[c]) / std::sqrt(t.var[c]) + b;
        t.borderline[at] = std::fabs(pre) < 1e-5;
      }
  return t;
}

// ---- tests -----------------------------------------------------------------------------------

// tests/test_gpu.rs:561-593: a running average that starts at zero and sees ones with rate 0.25
// reads 0.25, then 0.4375.
static void test_online_average_rule()
{
  DeviceArray x = DeviceArray::filled({8}, 1.0f), y = DeviceArray::zeros({8});
  OnlineAverageOp::apply(0.25f, x, y);
  for (float v : y.to_host()) EXPECT(v == 0.25f, "first update");
  OnlineAverageOp::apply(0.25f, x, y);
  for (float v : y.to_host()) EXPECT(v == 0.4375f, "second update");
}

// The reference's own route: batch_normalize_2d (five launches), positive_clip, then the adjoint
// chain, against the literal f32 restatement of the same kernels.
static void test_reference_composition_matches_literal_oracle()
{
  const Problem p = make_problem({12, 10, 6, 9}, 11, 0.5, 2.0);
  const size_t len = p.x.size();
  std::vector<float> y(len), dx(len), mean(p.c), var(p.c), rm(p.c, 0.f), rv(p.c, 0.f), xhat(len), dz(len);
  oracle_bn_relu_fwd_bwd_f32(p.dim0, p.c, p.n, 1e-5f, 0.1f, p.x.data(), p.dy.data(), nullptr, nullptr, rm.data(), rv.data(), y.data(),
                             dx.data(), mean.data(), var.data(), nullptr, nullptr, xhat.data(), dz.data(), 1024);
  DeviceArray x = DeviceArray::from_host(p.size, p.x.data()), dy = DeviceArray::from_host(p.size, p.dy.data());
  DeviceArray avg_mean, avg_var;                       // empty: start from zeros, as zeros_like in the reference
  BatchNormalizeOut o = batch_normalize_2d(x, p.axes, true, 0.1f, 1e-5f, avg_mean, avg_var);
  DeviceArray act(p.size), dzd(p.size);
  PositiveClipOp::apply(o.y, act);
  PositiveClipBwdOp::apply(dy, act, dzd);
  DeviceArray dxd = batch_normalize_adjoint(p.axes, dzd, x, o.mean, o.var);
  expect_close(o.mean.to_host(), mean, "mean");
  expect_close(o.var.to_host(), var, "var");
  expect_close(avg_mean.to_host(), rm, "avg_mean");
  expect_close(avg_var.to_host(), rv, "avg_var");
  const Truth t = truth_f64(p, false);
  expect_close(act.to_host(), y, "y", &t.borderline);
  expect_close(dxd.to_host(), dx, "dx", &t.borderline);
}

static void check_fused(const std::vector<uint32_t> &size, uint64_t seed, double loc, double scale)
{
  const Problem p = make_problem(size, seed, loc, scale);
  const Truth t = truth_f64(p, true);
  FusedBatchNormRelu layer(p.c);
  layer.gamma.copy_from_host(p.gamma.data()); layer.beta.copy_from_host(p.beta.data());
  DeviceArray x = DeviceArray::from_host(p.size, p.x.data()), dy = DeviceArray::from_host(p.size, p.dy.data());
  DeviceArray y(p.size), dx(p.size);
  layer.forward(x, y);
  layer.backward(dy, dx);
  EXPECT(layer.status() == 0, "status word");
  expect_close(y.to_host(), t.y, "fused y", &t.borderline);
  expect_close(dx.to_host(), t.dx, "fused dx", &t.borderline);
  expect_close(layer.mean.to_host(), t.mean, "fused mean");
  expect_close(layer.var.to_host(), t.var, "fused var");
  expect_close(layer.avg_mean.to_host(), t.run_mean, "fused avg_mean");
  expect_close(layer.avg_var.to_host(), t.run_var, "fused avg_var");
  expect_sum_close(layer.dgamma.to_host(), t.dgamma, "fused dgamma");
  expect_sum_close(layer.dbeta.to_host(), t.dbeta, "fused dbeta");
}
static void test_fused_layer_matches_float64_oracle()
{
  check_fused({28, 28, 16, 8}, 21, 0.0, 1.0);          // rows, 128-bit path
  check_fused({7, 7, 48, 32}, 22, 0.5, 2.0);           // short rows: cluster kernel
  check_fused({5, 3, 3, 5}, 23, 0.5, 2.0);             // odd sizes: scalar path
  check_fused({8, 8, 4, 6, 3}, 24, 0.0, 1.0);          // [W,H,D,C,N]
}

// online = false normalizes with the running averages (src/ops.rs:1010-1011); the fused inference
// operator without activation computes the same thing.
static void test_inference_branch()
{
  const Problem p = make_problem({10, 10, 6, 4}, 31, 0.5, 2.0);
  DeviceArray x = DeviceArray::from_host(p.size, p.x.data());
  Rng r5(5), r6(6);
  std::vector<float> am = uniforms(p.c, r5, -0.2, 0.2), av = uniforms(p.c, r6, 0.8, 1.6);
  DeviceArray avg_mean = DeviceArray::from_host({p.c}, am.data()), avg_var = DeviceArray::from_host({p.c}, av.data());
  BatchNormalizeOut o = batch_normalize_2d(x, p.axes, false, 0.0f, 1e-5f, avg_mean, avg_var);     // rate 0: averages stay
  DeviceArray y(p.size);
  BatchNormalize2dActInferOp::apply(p.axes, x, avg_mean, avg_var, y, nullptr, nullptr, 1.0f);
  std::vector<double> want(p.x.size());
  for (uint32_t n = 0; n < p.n; ++n)
    for (uint32_t c = 0; c < p.c; ++c)
      for (uint32_t i = 0; i < p.dim0; ++i) {
        const size_t at = i + (size_t)p.dim0 * (c + (size_t)p.c * n);
        want[at] = ((double)p.x[at] - am[c]) / std::sqrt((double)av[c]);
      }
  expect_close(o.y.to_host(), want, "legacy normalize with running averages");
  expect_close(y.to_host(), want, "fused inference, no activation");
}

static void test_host_step_equals_resident_calls()
{
  const Problem p = make_problem({14, 14, 12, 8}, 41, 0.0, 1.0);
  const size_t len = p.x.size();
  float *hx, *hdy, *hy, *hdx;
  cuda_check(cudaMallocHost(&hx, len * 4), "cudaMallocHost"); cuda_check(cudaMallocHost(&hdy, len * 4), "cudaMallocHost");
  cuda_check(cudaMallocHost(&hy, len * 4), "cudaMallocHost"); cuda_check(cudaMallocHost(&hdx, len * 4), "cudaMallocHost");
  for (size_t i = 0; i < len; ++i) { hx[i] = p.x[i]; hdy[i] = p.dy[i]; hy[i] = hdx[i] = NAN; }
  FusedBatchNormRelu a(p.c), b(p.c);
  for (FusedBatchNormRelu *l : {&a, &b}) { l->gamma.copy_from_host(p.gamma.data()); l->beta.copy_from_host(p.beta.data()); }
  a.step_from_host(p.size, hx, hdy, hy, hdx, 4);
  cuda_check(cudaStreamSynchronize(0), "cudaStreamSynchronize");
  const Truth t = truth_f64(p, true);
  expect_close(std::vector<float>(hy, hy + len), t.y, "host step y", &t.borderline);
  expect_close(std::vector<float>(hdx, hdx + len), t.dx, "host step dx", &t.borderline);
  expect_sum_close(a.dgamma.to_host(), t.dgamma, "host step dgamma");
  DeviceArray x = DeviceArray::from_host(p.size, p.x.data()), dy = DeviceArray::from_host(p.size, p.dy.data()), y(p.size), dx(p.size);
  b.forward(x, y); b.backward(dy, dx);
  expect_close(a.mean.to_host(), b.mean.to_host(), "host step mean vs resident", nullptr, 1e-6, 1e-7);
  cudaFreeHost(hx); cudaFreeHost(hdy); cudaFreeHost(hy); cudaFreeHost(hdx);
}

static void test_error_behaviour()
{
  DeviceArray x = DeviceArray::zeros({4, 4, 3, 2}), mean = DeviceArray::zeros({3});
  bool threw = false;
  try { BatchMean2dOp::apply({1, 0}, x, mean); } catch (const Error &e) { threw = e.code == ANODE_E_DIMS; }
  EXPECT(threw, "axes other than the leading ones are rejected");
  threw = false;
  try { DeviceArray wrong = DeviceArray::zeros({5}); BatchMean2dOp::apply({0, 1}, x, wrong); } catch (const Error &) { threw = true; }
  EXPECT(threw, "a statistics vector of the wrong length is rejected");
  DeviceArray y(x.size()), var = DeviceArray::zeros({3});
  void *ws = nullptr;
  cuda_check(cudaMalloc(&ws, 256), "cudaMalloc");
  const int rc = anode_gpu_batch_norm_relu_fused_fwd_3d1_packed_f32(16, 3, 2, 1e-5f, 0.1f, 1, x.ptr(), nullptr, nullptr, y.ptr(), mean.ptr(),
                                                                    var.ptr(), nullptr, nullptr, ws, 256, kernel_config(), nullptr);
  EXPECT(rc == ANODE_E_WORKSPACE, "a workspace that is too small is refused before anything is enqueued");
  cudaFree(ws);
}

// The synchronized layer with a communicator of one rank gives what the one-GPU layer gives; the handle
// without NCCL refuses what it cannot do (several ranks need several GPUs: tests/test_gpu_sync.py).
static void test_sync_layer_world_one()
{
  const Problem p = make_problem({28, 28, 12, 6}, 41, 0.5, 2.0);
  const Truth t = truth_f64(p, true);
  SyncComm comm = SyncComm::exchange_only(0, 1);
  SyncBatchNormRelu layer(comm, p.c);
  layer.gamma.copy_from_host(p.gamma.data()); layer.beta.copy_from_host(p.beta.data());
  DeviceArray x = DeviceArray::from_host(p.size, p.x.data()), dy = DeviceArray::from_host(p.size, p.dy.data());
  DeviceArray y(p.size), dx(p.size);
  for (int rep = 0; rep < 2; ++rep) {          // twice on one workspace
    layer.avg_mean = DeviceArray::zeros({p.c}); layer.avg_var = DeviceArray::filled({p.c}, 1.0f);
    layer.forward(x, y);
    layer.backward(dy, dx);
  }
  EXPECT(layer.status() == 0, "status word");
  expect_close(y.to_host(), t.y, "sync y", &t.borderline);
  expect_close(dx.to_host(), t.dx, "sync dx", &t.borderline);
  expect_close(layer.mean.to_host(), t.mean, "sync mean");
  expect_close(layer.var.to_host(), t.var, "sync var");
  expect_close(layer.avg_mean.to_host(), t.run_mean, "sync avg_mean");
  expect_close(layer.avg_var.to_host(), t.run_var, "sync avg_var");
  expect_sum_close(layer.dgamma.to_host(), t.dgamma, "sync dgamma");
  expect_sum_close(layer.dbeta.to_host(), t.dbeta, "sync dbeta");
  // two claimed ranks, no exchange attached, no NCCL: refused before anything is enqueued
  SyncComm two = SyncComm::exchange_only(0, 2);
  SyncBatchNormRelu orphan(two, p.c);
  bool refused = false;
  try { orphan.forward(x, y); } catch (const Error &e) { refused = e.code == ANODE_E_COMM; }
  EXPECT(refused, "a communicator without NCCL and without an exchange buffer refuses the call");
}

int main()
{
  int devs = 0;
  if (cudaGetDeviceCount(&devs) != cudaSuccess || devs == 0) { fprintf(stderr, "no CUDA device\n"); return 2; }
  const std::pair<const char *, std::function<void()>> tests[] = {
      {"online_average_rule", test_online_average_rule},
      {"reference_composition_matches_literal_oracle", test_reference_composition_matches_literal_oracle},
      {"fused_layer_matches_float64_oracle", test_fused_layer_matches_float64_oracle},
      {"inference_branch", test_inference_branch},
      {"host_step_equals_resident_calls", test_host_step_equals_resident_calls},
      {"error_behaviour", test_error_behaviour},
      {"sync_layer_world_one", test_sync_layer_world_one},
  };
  int failed = 0;
  for (const auto &t : tests) {
    try { t.second(); printf("ok   %s\n", t.first); }
    catch (const Failure &f) { printf("FAIL %s: %s\n", t.first, f.what.c_str()); ++failed; }
    catch (const std::exception &e) { printf("FAIL %s: exception %s\n", t.first, e.what()); ++failed; }
  }
  printf("%d checks, %d tests failed\n", g_checks, failed);
  return failed ? 1 : 0;
}
