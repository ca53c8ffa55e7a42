// Tensor value type of the host layer: the subset of the reference's include/core/tensor.h
// that ops::Mul and its callers use.  A Tensor is metadata plus a shared storage object
// (TensorImpl); copying a Tensor deep-copies the storage, moving is cheap — the reference's
// value semantics (src/tensor.cpp:396-421).
#pragma once
#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <memory>
#include <vector>

#include "type_traits.h"

class ContextImpl;

struct Metadata {
  size_t numel = 0;
  int64_t offset = 0;
  via::Device device = via::Device::CPU;
  via::DataType dtype = via::DataType::FLOAT32;
  std::vector<int64_t> shape;
  std::vector<int64_t> strides;  // in elements, dense row-major
  void calculate_strides() {
    strides.assign(shape.size(), 1);
    for (size_t i = shape.size(); i-- > 1;) strides[i - 1] = strides[i] * shape[i];
  }
};

// Storage behind a Tensor; one implementation per device kind.
class TensorImpl {
 public:
  virtual ~TensorImpl() = default;
  virtual void* data() = 0;
  virtual const void* data() const = 0;
  virtual size_t numel() const = 0;
  virtual void copy_to(std::shared_ptr<TensorImpl> dst) const = 0;
  virtual std::unique_ptr<TensorImpl> clone() const = 0;
  virtual std::unique_ptr<TensorImpl> clone_as_contiguous(const Metadata&) const = 0;
  virtual std::shared_ptr<ContextImpl> context() const = 0;
};

class Tensor;
namespace tvhost {
// wraps an existing storage object as a tensor of the given shape (used by the operators to
// return device results without a copy)
Tensor adopt(std::vector<int64_t> shape, via::DataType dtype, std::shared_ptr<TensorImpl> impl, via::Device device);
}

class Tensor {
 public:
  Tensor() = default;
  Tensor(const Tensor& other);                 // deep copy
  Tensor(Tensor&& other) noexcept = default;
  Tensor& operator=(const Tensor& other);      // deep copy
  Tensor& operator=(Tensor&& other) noexcept = default;

  // uninitialised storage on the default device (CUDA) or on `device`
  Tensor(std::vector<int64_t> shape, via::DataType dtype);
  Tensor(std::initializer_list<int64_t> shape, via::DataType dtype);
  Tensor(std::vector<int64_t> shape, via::DataType dtype, via::Device device);
  Tensor(std::initializer_list<int64_t> shape, via::DataType dtype, via::Device device);
  // copies numel * sizeof(dtype) bytes from host memory at `ptr` (raw element bits)
  Tensor(void* ptr, std::vector<int64_t> shape, via::DataType dtype, via::Device device);

  void* data();
  const void* data() const;
  via::Device device() const { return m_meta.device; }
  via::DataType dtype() const { return m_meta.dtype; }
  size_t numel() const { return m_meta.numel; }
  size_t dims() const { return m_meta.shape.size(); }
  int64_t shape(int i) const;
  std::vector<int64_t> shape() const { return m_meta.shape; }
  std::vector<int64_t> strides() const { return m_meta.strides; }
  bool is_contiguous() const { return true; }  // this layer creates no strided views
  std::shared_ptr<TensorImpl> get_impl() const { return m_impl; }

  Tensor clone() const;
  void to_host();                    // device -> host copy, in place
  void to_device(uint32_t id = 0);   // host -> device `id`, in place

  // element read for tests (copies one element back if the tensor is on the device)
  template <typename T>
  T at(std::initializer_list<int64_t> idxs) const;

  static Tensor Zeros(std::vector<int64_t> shape, via::DataType dtype = via::DataType::FLOAT32);
  static Tensor Ones(std::vector<int64_t> shape, via::DataType dtype = via::DataType::FLOAT32);
  static Tensor Fill(std::vector<int64_t> shape, float value, via::DataType dtype);
  static Tensor Random(std::vector<int64_t> shape, float min = 0.0f, float max = 1.0f,
                       via::DataType dtype = via::DataType::FLOAT32);
  static Tensor Random(std::initializer_list<int64_t> shape, float min = 0.0f, float max = 1.0f,
                       via::DataType dtype = via::DataType::FLOAT32);
  // Random draws from a process-wide generator; seed it for reproducible tensors
  // (the reference's generator is seeded from the clock and cannot be).
  static void ManualSeed(uint64_t seed);

 private:
  friend Tensor tvhost::adopt(std::vector<int64_t>, via::DataType, std::shared_ptr<TensorImpl>, via::Device);
  void read_element(size_t index, void* out) const;
  Metadata m_meta;
  std::shared_ptr<TensorImpl> m_impl;
};

template <typename T>
T Tensor::at(std::initializer_list<int64_t> idxs) const {
  if (idxs.size() != m_meta.shape.size()) throw std::runtime_error("at(): wrong number of indices");
  if (sizeof(T) != via::calc_dtype_size(m_meta.dtype)) throw std::runtime_error("at(): element size mismatch");
  size_t flat = 0, d = 0;
  for (int64_t i : idxs) {
    if (i < 0 || i >= m_meta.shape[d]) throw std::runtime_error("at(): index out of range");
    flat += static_cast<size_t>(i) * static_cast<size_t>(m_meta.strides[d++]);
  }
  T v;
  read_element(flat, &v);
  return v;
}
