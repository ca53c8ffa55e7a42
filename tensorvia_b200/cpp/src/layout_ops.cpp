// ops::Slice, ops::Concat, ops::Transpose and ops::Typecast over the C ABI (reference front ends:
// src/ops.cpp:158-190, 1277-1353; CUDA back ends: src/backend/cuda/slice.cu, concat.cu,
// transpose.cu).  Host tensors make the round trip through the GPU, as in ops::Mul.
#include <format>
#include <string>

#include "factory.h"
#include "ops.h"
#include "storage.h"
#include "tvb.h"

using namespace via;

namespace {
// a dense device tensor holding what `t` shows
Tensor dense_on_device(const Tensor& t) {
  Tensor d(t);   // copies are dense
  if (d.device() == Device::CPU) d.to_device(static_cast<uint32_t>(default_device()));
  return d;
}
std::shared_ptr<tvhost::CudaStorage> cuda_storage(const Tensor& t) {
  auto s = std::dynamic_pointer_cast<tvhost::CudaStorage>(t.get_impl());
  if (!s) throw std::runtime_error("operand must live on a CUDA device");
  return s;
}
}  // namespace

namespace ops {

Tensor Slice(const Tensor& t, const std::vector<std::pair<int64_t, int64_t>>& ranges) {
  if (ranges.empty()) throw std::runtime_error("Slice ranges cannot be empty");
  if (ranges.size() != t.shape().size()) throw std::runtime_error("Slice ranges size must be equal to tensor shape size");
  std::vector<int64_t> begin, end, shape;
  for (size_t i = 0; i < ranges.size(); ++i) {
    if (ranges[i].first > ranges[i].second) throw std::runtime_error("first must be less than second");
    if (ranges[i].first < 0) throw std::runtime_error("first must be >= 0 and <= second");
    if (ranges[i].second > t.shape(static_cast<int>(i)))
      throw std::runtime_error(std::format("second must be less than {}", t.shape(static_cast<int>(i))));
    begin.push_back(ranges[i].first);
    end.push_back(ranges[i].second);
    shape.push_back(ranges[i].second - ranges[i].first);
  }
  calc_numel(shape);   // an empty window has no tensor: throws as the reference's constructor does
  const bool host = t.device() == Device::CPU;
  Tensor src = dense_on_device(t);
  auto ss = cuda_storage(src);
  auto out = std::make_shared<tvhost::CudaStorage>(nullptr, calc_numel(shape), t.dtype(), ss->cuda());
  const std::vector<int64_t> full = src.shape();
  tvhost::check(tvb_slice(ss->cuda()->device(), src.data(), out->data(), static_cast<int>(t.dtype()),
                          static_cast<int>(full.size()), full.data(), static_cast<int>(begin.size()), begin.data(),
                          end.data(), nullptr),
                "tvb_slice");
  ss->cuda()->wait();
  Tensor res = tvhost::adopt(std::move(shape), t.dtype(), out, Device::CUDA);
  if (host) res.to_host();
  return res;
}

Tensor Concat(const std::vector<Tensor>& tensors, int dim) {
  if (tensors.empty()) throw std::invalid_argument("tensors is empty");
  if (tensors.size() == 1) return tensors[0];
  const DataType dtype = tensors[0].dtype();
  const std::vector<int64_t> first = tensors[0].shape();
  for (const Tensor& t : tensors) {
    if (t.dtype() != dtype) throw std::invalid_argument("tensors must have same dtype");
    if (t.shape().size() != first.size()) throw std::invalid_argument("tensors must have same number of dimensions");
    for (size_t i = 0; i < first.size(); ++i)
      if (static_cast<int>(i) != dim && t.shape()[i] != first[i])
        throw std::invalid_argument("tensors must have same shape except concatenation dimension");
  }
  if (dim < 0 || dim >= static_cast<int>(first.size())) throw std::invalid_argument("concatenation dimension out of range");
  const bool host = tensors[0].device() == Device::CPU;
  std::vector<Tensor> dense;
  dense.reserve(tensors.size());
  std::vector<const void*> ptrs;
  std::vector<int64_t> sizes;
  std::vector<int64_t> shape = first;
  shape[static_cast<size_t>(dim)] = 0;
  for (const Tensor& t : tensors) {
    dense.push_back(dense_on_device(t));
    ptrs.push_back(dense.back().data());
    sizes.push_back(t.shape(dim));
    shape[static_cast<size_t>(dim)] += t.shape(dim);
  }
  auto s0 = cuda_storage(dense[0]);
  for (const Tensor& t : dense)
    if (cuda_storage(t)->cuda()->device() != s0->cuda()->device()) throw std::runtime_error("tensors must live on one device");
  auto out = std::make_shared<tvhost::CudaStorage>(nullptr, calc_numel(shape), dtype, s0->cuda());
  tvhost::check(tvb_concat(s0->cuda()->device(), static_cast<int>(ptrs.size()), ptrs.data(), out->data(),
                           static_cast<int>(dtype), static_cast<int>(first.size()), first.data(), sizes.data(), dim,
                           nullptr),
                "tvb_concat");
  s0->cuda()->wait();
  Tensor res = tvhost::adopt(std::move(shape), dtype, out, Device::CUDA);
  if (host) res.to_host();
  return res;
}

void Transpose(Tensor& a) {
  if (a.data() == nullptr || a.numel() == 0) throw std::runtime_error("tensor a is null");
  if (a.shape().size() != 2) throw std::runtime_error("transpose only support 2D tensor");
  const bool host = a.device() == Device::CPU;
  Tensor src = dense_on_device(a);
  auto ss = cuda_storage(src);
  const int64_t rows = src.shape(0), cols = src.shape(1);
  auto out = std::make_shared<tvhost::CudaStorage>(nullptr, src.numel(), a.dtype(), ss->cuda());
  tvhost::check(tvb_transpose2d(ss->cuda()->device(), src.data(), out->data(), static_cast<int>(a.dtype()), rows, cols,
                                nullptr),
                "tvb_transpose2d");
  ss->cuda()->wait();
  Tensor res = tvhost::adopt({cols, rows}, a.dtype(), out, Device::CUDA);
  if (host) res.to_host();
  a = std::move(res);
}

Tensor Typecast(const Tensor& a, DataType dst_type) {
  if (a.data() == nullptr || a.numel() == 0) throw std::runtime_error("tensor a is null");
  static const char* names[8] = {"int8", "int16", "int32", "int64", "bfloat16", "float16", "float32", "float64"};
  if (a.dtype() == dst_type) return a;
  const bool host = a.device() == Device::CPU;
  Tensor src = dense_on_device(a);
  auto ss = cuda_storage(src);
  auto out = std::make_shared<tvhost::CudaStorage>(nullptr, src.numel(), dst_type, ss->cuda());
  const int rc = tvb_typecast(ss->cuda()->device(), src.data(), out->data(), static_cast<int>(a.dtype()),
                              static_cast<int>(dst_type), src.numel(), nullptr);
  if (rc == TVB_ERR_DTYPE)
    throw std::runtime_error(std::format("Invalid typecast from {} to {}", names[static_cast<int>(a.dtype())],
                                         names[static_cast<int>(dst_type)]));
  tvhost::check(rc, "tvb_typecast");
  ss->cuda()->wait();
  Tensor res = tvhost::adopt(src.shape(), dst_type, out, Device::CUDA);
  if (host) res.to_host();
  return res;
}

}  // namespace ops
