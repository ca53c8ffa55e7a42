// via:: enums and dtype rules, source-compatible with the subset of the reference's
// include/core/type_traits.h that the matmul path uses.
#pragma once
#include <chrono>
#include <cstddef>
#include <cstdint>
#include <iostream>
#include <stdexcept>
#include <string_view>
#include <vector>

#include "types.h"

// prints the wall time of one expression, as the reference's macro of the same name does
#define RUNNING_TIME(expr)                                                                   \
  do {                                                                                       \
    const auto rt_t0__ = std::chrono::steady_clock::now();                                   \
    expr;                                                                                    \
    const std::chrono::duration<double, std::milli> rt_d__ = std::chrono::steady_clock::now() - rt_t0__; \
    std::cout << "Execution time: " << rt_d__.count() << "ms" << std::endl;                  \
  } while (0)

namespace via {

enum class Device { CPU, CUDA, SYCL, VULKAN };

// numbering is part of the ABI: the C library takes these values as they are
enum class DataType { INT8 = 0, INT16, INT32, INT64, BFLOAT16, FLOAT16, FLOAT32, FLOAT64 };

constexpr std::string_view device_to_string(Device d) {
  constexpr std::string_view n[] = {"CPU", "CUDA", "SYCL", "VULKAN"};
  return static_cast<unsigned>(d) < 4 ? n[static_cast<unsigned>(d)] : "UNKNOWN";
}
constexpr std::string_view dtype_to_string(DataType t) {
  constexpr std::string_view n[] = {"int8", "int16", "int32", "int64", "bfloat16", "float16", "float32", "float64"};
  return static_cast<unsigned>(t) < 8 ? n[static_cast<unsigned>(t)] : "UNKNOWN";
}
inline size_t calc_dtype_size(DataType t) {
  constexpr size_t s[] = {1, 2, 4, 8, 2, 2, 4, 8};
  if (static_cast<unsigned>(t) >= 8) throw std::runtime_error("Unsupported DataType");
  return s[static_cast<unsigned>(t)];
}

// Result dtype of a binary op (the rule the reference executes, type_traits.h:270-287):
// equal types stay; two integers give the wider; two floats give at least FLOAT32; an integer
// with a float gives FLOAT64 if the integer is INT64, else at least FLOAT32.
inline DataType compute_type(DataType a, DataType b) {
  if (a == b) return a;
  const DataType hi = a > b ? a : b;
  const bool ia = a <= DataType::INT64, ib = b <= DataType::INT64;
  if (ia && ib) return hi;
  if (ia != ib && (a == DataType::INT64 || b == DataType::INT64)) return DataType::FLOAT64;
  return hi > DataType::FLOAT32 ? hi : DataType::FLOAT32;
}

// number of elements; every dimension must be positive
inline size_t calc_numel(const std::vector<int64_t>& shape) {
  size_t n = 1;
  for (int64_t d : shape) {
    if (d <= 0) throw std::runtime_error("Invalid tensor dimension");
    n *= static_cast<size_t>(d);
  }
  return n;
}

}  // namespace via
