#pragma once
// Backend context handle, as in the reference (include/core/context.h): ctx_raw_ptr() yields a
// pointer to the backend's native handle — here a `cudaStream_t*` for CUDA, nullptr for CPU.
class ContextImpl {
 public:
  virtual ~ContextImpl() = default;
  virtual void* ctx_raw_ptr() = 0;
};
