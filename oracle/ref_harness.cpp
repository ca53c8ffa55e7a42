// TEST INFRASTRUCTURE — not part of the product.
//
// C entry points around the UNMODIFIED reference library (its CPU/OpenMP backend,
// compiled from the reference tree by oracle/Makefile into oracle/_ref/).  They let
// the Python tests, the golden-vector generator and the benchmark's CPU baseline
// call the reference's own `ops::Mul` on caller-supplied bytes.
//
// Inputs are raw element bits: half and bfloat16 values are never pushed through the
// reference's host conversion classes (its bfloat16_t(float) constructor zeroes
// normal values, include/backend/cuda/bfloat16.hpp:26-34); the tensor constructor
// that copies from a pointer takes the bits as they are (src/tensor.cpp:96-117).
#include <omp.h>

#include <cstdint>
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "ops.h"

namespace {
thread_local std::string g_msg;
std::vector<int64_t> shape_of(int rank, const int64_t* dims) { return std::vector<int64_t>(dims, dims + rank); }
}  // namespace

extern "C" {

const char* tvref_last_error(void) { return g_msg.c_str(); }

int tvref_compute_type(int a, int b) {
  return static_cast<int>(via::compute_type(static_cast<via::DataType>(a), static_cast<via::DataType>(b)));
}

int tvref_dtype_size(int d) { return static_cast<int>(via::calc_dtype_size(static_cast<via::DataType>(d))); }

// threads the reference's matmul will use: min(omp_get_max_threads(), 16)
// (src/backend/cpu/mul.cpp:114)
int tvref_threads(void) {
  const int m = omp_get_max_threads();
  return m < 16 ? m : 16;
}

// ops::Mul on host data.  rank_a/dims_a and rank_b/dims_b are passed as given so
// that the reference's own validation (src/ops.cpp:540-556) is what rejects bad
// shapes.  On success writes the result dtype to *dtype_c, the result rank/dims to
// rank_c/dims_c (dims_c has room for 3) and, if `c` is not null and c_bytes is
// large enough, the result bytes to c.  Returns 0 on success, 1 if the reference
// threw (message in tvref_last_error), 2 if c was too small.
int tvref_mul(const void* a, int dtype_a, int rank_a, const int64_t* dims_a, const void* b, int dtype_b,
              int rank_b, const int64_t* dims_b, void* c, uint64_t c_bytes, int* dtype_c, int* rank_c,
              int64_t* dims_c) {
  try {
    Tensor ta(const_cast<void*>(a), shape_of(rank_a, dims_a), static_cast<via::DataType>(dtype_a),
              via::Device::CPU);
    Tensor tb(const_cast<void*>(b), shape_of(rank_b, dims_b), static_cast<via::DataType>(dtype_b),
              via::Device::CPU);
    Tensor tc = ops::Mul(ta, tb);
    const std::vector<int64_t> sc = tc.shape();
    if (dtype_c) *dtype_c = static_cast<int>(tc.dtype());
    if (rank_c) *rank_c = static_cast<int>(sc.size());
    if (dims_c)
      for (size_t i = 0; i < sc.size() && i < 3; ++i) dims_c[i] = sc[i];
    const uint64_t bytes = static_cast<uint64_t>(tc.numel()) * via::calc_dtype_size(tc.dtype());
    if (c) {
      if (bytes > c_bytes) {
        g_msg = "result buffer too small";
        return 2;
      }
      std::memcpy(c, tc.data(), bytes);
    }
    return 0;
  } catch (const std::exception& e) {
    g_msg = e.what();
    return 1;
  } catch (...) {
    g_msg = "unknown exception";
    return 1;
  }
}

}  // extern "C"
