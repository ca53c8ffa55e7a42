// Checks of the C++ host layer with assertions (the reference's tests have none): the shape
// rules and messages of ops::Mul, the result dtypes, values against a plain host loop, value
// semantics of Tensor, and host<->device moves.  Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <functional>
#include <string>
#include <vector>

#include "ops.h"
using namespace via;

static int g_failed = 0;
#define EXPECT(cond)                                                         \
  do {                                                                       \
    if (!(cond)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); ++g_failed; } \
  } while (0)

static std::string thrown(const std::function<void()>& f) {
  try { f(); } catch (const std::runtime_error& e) { return e.what(); }
  return "";
}

int main() {
  // ---- shape rules, with the reference's messages -------------------------------------------
  Tensor a23 = Tensor::Ones({2, 3}), b45 = Tensor::Ones({4, 5}), b3 = Tensor::Ones({3});
  Tensor a234 = Tensor::Ones({2, 3, 4}), b345 = Tensor::Ones({3, 4, 5}), b255 = Tensor::Ones({2, 5, 5});
  EXPECT(thrown([&] { ops::Mul(a23, b45); }) == "Tensors common dim must match,but 2 and 4");
  EXPECT(thrown([&] { ops::Mul(a23, b3); }) == "Tensors a and b must have the same rank,but got 2 and 1");
  EXPECT(thrown([&] { ops::Mul(b3, b3); }) == "Tensors a and b dims must be 2 or 3,but got 1");
  EXPECT(thrown([&] { ops::Mul(a234, b345); }) == "Tensors a and b must have the same batch size");
  EXPECT(thrown([&] { ops::Mul(a234, b255); }) == "Tensors common dim must match,but 4 and 5");
  Tensor host23 = a23; host23.to_host();
  EXPECT(thrown([&] { ops::Mul(host23, Tensor::Ones({3, 2})); }) == "Tensors a and b device mismatch!");
  EXPECT(!thrown([&] { Tensor t({2, 0}, DataType::FLOAT32); }).empty());

  // ---- result dtypes (via::compute_type) ----------------------------------------------------
  const DataType all[] = {DataType::INT8, DataType::INT16, DataType::INT32, DataType::INT64,
                          DataType::BFLOAT16, DataType::FLOAT16, DataType::FLOAT32, DataType::FLOAT64};
  for (DataType x : all)
    for (DataType y : all) {
      Tensor p = Tensor::Ones({3, 4}, x), q = Tensor::Ones({4, 2}, y);
      Tensor r = ops::matmul(p, q);
      EXPECT(r.dtype() == compute_type(x, y));
      EXPECT(r.device() == Device::CUDA && r.shape() == (std::vector<int64_t>{3, 2}));
    }
  EXPECT(compute_type(DataType::BFLOAT16, DataType::BFLOAT16) == DataType::BFLOAT16);
  EXPECT(compute_type(DataType::BFLOAT16, DataType::FLOAT16) == DataType::FLOAT32);
  EXPECT(compute_type(DataType::INT64, DataType::FLOAT16) == DataType::FLOAT64);
  EXPECT(compute_type(DataType::INT8, DataType::INT8) == DataType::INT8);

  // ---- values: fp32 2-D (tensor cores) and batched int8 with wrap-around ---------------------
  {
    const int M = 130, K = 72, N = 264;
    std::vector<float> ha(M * K), hb(K * N);
    for (int i = 0; i < M * K; ++i) ha[i] = std::sin(0.37f * i);
    for (int i = 0; i < K * N; ++i) hb[i] = std::cos(0.11f * i);
    Tensor A(ha.data(), {M, K}, DataType::FLOAT32, Device::CUDA), B(hb.data(), {K, N}, DataType::FLOAT32, Device::CUDA);
    Tensor C = ops::Mul(A, B);
    C.to_host();
    const float* c = static_cast<const float*>(C.data());
    double num = 0, den = 0;
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) {
        double s = 0;
        for (int k = 0; k < K; ++k) s += static_cast<double>(ha[i * K + k]) * hb[k * N + j];
        num += (c[i * N + j] - s) * (c[i * N + j] - s);
        den += s * s;
      }
    EXPECT(std::sqrt(num / den) <= 1e-5);
  }
  {
    const int Bt = 3, M = 20, K = 48, N = 16;
    std::vector<int8_t> ha(Bt * M * K), hb(Bt * K * N);
    for (size_t i = 0; i < ha.size(); ++i) ha[i] = static_cast<int8_t>((i * 37) % 255 - 127);
    for (size_t i = 0; i < hb.size(); ++i) hb[i] = static_cast<int8_t>((i * 91) % 255 - 127);
    Tensor A(ha.data(), {Bt, M, K}, DataType::INT8, Device::CUDA), B(hb.data(), {Bt, K, N}, DataType::INT8, Device::CUDA);
    Tensor C = ops::Mul(A, B);
    EXPECT(C.dtype() == DataType::INT8 && C.shape() == (std::vector<int64_t>{Bt, M, N}));
    int bad = 0;
    for (int b = 0; b < Bt; ++b)
      for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
          int s = 0;
          for (int k = 0; k < K; ++k) s += int(ha[(b * M + i) * K + k]) * int(hb[(b * K + k) * N + j]);
          if (C.at<int8_t>({b, i, j}) != static_cast<int8_t>(s)) ++bad;
        }
    EXPECT(bad == 0);
  }
  // host operands make the round trip and come back on the host
  {
    std::vector<float> ha = {1, 2, 3, 4, 5, 6}, hb = {1, 0, 0, 1, 1, 1};
    Tensor A(ha.data(), {2, 3}, DataType::FLOAT32, Device::CPU), B(hb.data(), {3, 2}, DataType::FLOAT32, Device::CPU);
    Tensor C = ops::Mul(A, B);
    EXPECT(C.device() == Device::CPU);
    EXPECT(C.at<float>({0, 0}) == 4.f && C.at<float>({0, 1}) == 5.f && C.at<float>({1, 0}) == 10.f && C.at<float>({1, 1}) == 11.f);
  }

  // ---- value semantics --------------------------------------------------------------------------
  {
    Tensor x = Tensor::Fill({4, 4}, 2.5f, DataType::FLOAT32);
    Tensor y = x;                        // deep copy
    EXPECT(y.data() != x.data() && y.at<float>({3, 3}) == 2.5f);
    Tensor z = std::move(x);             // move keeps the storage
    EXPECT(z.at<float>({0, 0}) == 2.5f && z.numel() == 16);
    Tensor h = z.clone();
    h.to_host();
    EXPECT(h.device() == Device::CPU && z.device() == Device::CUDA);
    h.to_device(0);
    EXPECT(h.device() == Device::CUDA && h.at<float>({2, 1}) == 2.5f);
    Tensor bf = Tensor::Fill({2, 2}, 0.5f, DataType::BFLOAT16);   // the reference's host bf16 class would store 0
    EXPECT(float(bf.at<bfloat16>({1, 1})) == 0.5f);
    Tensor::ManualSeed(7);
    Tensor r1 = Tensor::Random({8, 8}, -10, 10, DataType::INT8);
    Tensor::ManualSeed(7);
    Tensor r2 = Tensor::Random({8, 8}, -10, 10, DataType::INT8);
    bool same = true, in_range = true;
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 8; ++j) {
        same = same && r1.at<int8_t>({i, j}) == r2.at<int8_t>({i, j});
        in_range = in_range && r1.at<int8_t>({i, j}) >= -10 && r1.at<int8_t>({i, j}) <= 10;
      }
    EXPECT(same && in_range);
  }
  std::printf(g_failed ? "%d check(s) failed\n" : "api_check: all checks passed\n", g_failed);
  return g_failed ? 1 : 0;
}
