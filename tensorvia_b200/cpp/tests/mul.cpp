// The matmul timing scenario of the reference's tests/mul.cpp, written against this layer:
// two random fp32 operands [2592,2048] and [2048,4096] in [-10,10], a loop of ops::Mul calls
// each timed with RUNNING_TIME, and the average at the end.  Pass a count as argv[1]
// (default 100, as the reference runs it).
#include <chrono>
#include <cstdio>
#include <cstdlib>

#include "ops.h"
using namespace via;

int main(int argc, char** argv) {
  const int iters = argc > 1 ? std::atoi(argv[1]) : 100;
  Tensor::ManualSeed(42);
  Tensor a = Tensor::Random({2592, 2048}, -10, 10, DataType::FLOAT32);
  Tensor b = Tensor::Random({2048, 4096}, -10, 10, DataType::FLOAT32);

  const auto t0 = std::chrono::high_resolution_clock::now();
  for (int i = 0; i < iters; ++i) {
    RUNNING_TIME(ops::Mul(a, b));
  }
  const auto t1 = std::chrono::high_resolution_clock::now();
  const double avg_ms = std::chrono::duration<double, std::milli>(t1 - t0).count() / iters;
  std::printf("avg times = %.3fms\n", avg_ms);
  return 0;
}
