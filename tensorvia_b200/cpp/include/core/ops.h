// Operators of the host layer: the matmul of the reference (include/core/ops.h:57-59) and the
// few creation helpers its callers need.
#pragma once
#include <vector>

#include "tensor.h"
#include "types.h"

namespace ops {

// [M,K] @ [K,N] -> [M,N];  [b,M,K] @ [b,K,N] -> [b,M,N].  Throws std::runtime_error for
// operands on different devices, different ranks, ranks other than 2 or 3, unequal batch or
// unequal common dimension — the checks and messages of the reference's ops::Mul
// (src/ops.cpp:540-556).  The result dtype is via::compute_type(a.dtype(), b.dtype()).
// CUDA operands are multiplied on the GPU; host operands are copied in, multiplied on the
// GPU and the result copied back (there is no CPU kernel in this library).
Tensor Mul(const Tensor& a, const Tensor& b);
// the name the reference's README uses for the same function
inline Tensor matmul(const Tensor& a, const Tensor& b) { return Mul(a, b); }

Tensor Zeros(const std::vector<int64_t>& shape, via::DataType dtype);
Tensor Ones(const std::vector<int64_t>& shape, via::DataType dtype);
Tensor Fill(const std::vector<int64_t>& shape, via::DataType dtype, float value);
Tensor Random(const std::vector<int64_t>& shape, via::DataType dtype, float min, float max);

}  // namespace ops
