// Storage registry, as in the reference (include/core/factory.h, src/factory.cpp): one factory
// per device kind creates the TensorImpl; `ptr != nullptr` means "copy numel elements from
// host memory at ptr".
#pragma once
#include <functional>
#include <memory>

#include "tensor.h"

using TensorImplFactory = std::function<std::shared_ptr<TensorImpl>(void* ptr, size_t numel, via::DataType)>;

void register_tensor_impl(via::Device device, TensorImplFactory factory);
std::shared_ptr<TensorImpl> create_tensor_impl(size_t numel, via::DataType dtype, via::Device device);
std::shared_ptr<TensorImpl> create_tensor_impl(void* ptr, size_t numel, via::DataType dtype, via::Device device);

void copy_device_to_host(std::shared_ptr<TensorImpl> src, std::shared_ptr<TensorImpl> dst, via::DataType dtype);
void copy_host_to_device(std::shared_ptr<TensorImpl> src, std::shared_ptr<TensorImpl> dst, via::DataType dtype);

// Device index new CUDA tensors are created on (the reference has a single implicit device;
// Tensor::to_device(id) and this setter make the index it already exposes effective).
void set_default_device(int device);
int default_device();
