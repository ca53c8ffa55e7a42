// ops::Mul front end: validation and dispatch (reference: src/ops.cpp:540-573).
#include <string>

#include "backend/cuda/ops/mul.h"
#include "factory.h"
#include "ops.h"

using namespace via;

namespace ops {

Tensor Mul(const Tensor& a, const Tensor& b) {
  if (a.device() != b.device()) throw std::runtime_error("Tensors a and b device mismatch!");
  const size_t ra = a.dims(), rb = b.dims();
  if (ra != rb)
    throw std::runtime_error("Tensors a and b must have the same rank,but got " + std::to_string(ra) + " and " +
                             std::to_string(rb));
  if (ra != 2 && ra != 3) throw std::runtime_error("Tensors a and b dims must be 2 or 3,but got " + std::to_string(ra));
  if (ra == 3) {
    if (a.shape(0) != b.shape(0)) throw std::runtime_error("Tensors a and b must have the same batch size");
    if (a.shape(2) != b.shape(1))
      throw std::runtime_error("Tensors common dim must match,but " + std::to_string(a.shape(2)) + " and " +
                               std::to_string(b.shape(1)));
  } else if (a.shape(1) != b.shape(0)) {
    // the reference prints a.shape(0) and b.shape(0) in this message (src/ops.cpp:555); kept as is
    throw std::runtime_error("Tensors common dim must match,but " + std::to_string(a.shape(0)) + " and " +
                             std::to_string(b.shape(0)));
  }
  if (a.device() == Device::CPU) {
    // No CPU kernel exists here.  Host operands make the round trip through the GPU, which is
    // what a caller of the reference does by hand with to_device / ops::Mul / to_host.
    Tensor da(a), db(b);
    da.to_device(static_cast<uint32_t>(default_device()));
    db.to_device(static_cast<uint32_t>(default_device()));
    Tensor c = MulImpl<Device::CUDA>::execute(da, db);
    c.to_host();
    return c;
  }
  return MulImpl<Device::CUDA>::execute(a, b);
}

}  // namespace ops
