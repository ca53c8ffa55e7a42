// ops::Mul front end: validation and dispatch (reference: src/ops.cpp:540-573).
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "backend/cuda/ops/mul.h"
#include "factory.h"
#include "ops.h"
#include "storage.h"
#include "tvb.h"

using namespace via;

namespace ops {

namespace {
// the checks of the reference's ops::Mul (src/ops.cpp:540-556), messages included
void check_mul_operands(const Tensor& a, const Tensor& b);
}  // namespace

Tensor matmul_sharded(const Tensor& a, const Tensor& b, int n_gpus) {
  check_mul_operands(a, b);
  int have = 0;
  tvhost::check(tvb_device_count(&have), "tvb_device_count");
  if (n_gpus < 1 || n_gpus > have)
    throw std::runtime_error("matmul_sharded: " + std::to_string(n_gpus) + " GPUs asked, " + std::to_string(have) + " present");
  Tensor ha(a), hb(b);   // dense copies
  ha.to_host();
  hb.to_host();
  const bool batched = ha.dims() == 3;
  const int64_t units = ha.shape(0), granule = batched ? 1 : 128;
  const int64_t a_unit = static_cast<int64_t>(ha.numel()) / units;                 // elements per row / batch of A
  const int64_t b_unit = batched ? static_cast<int64_t>(hb.numel()) / units : 0;    // per batch of B
  const DataType rt = compute_type(ha.dtype(), hb.dtype());
  std::vector<int64_t> shape_c = batched ? std::vector<int64_t>{ha.shape(0), ha.shape(1), hb.shape(2)}
                                         : std::vector<int64_t>{ha.shape(0), hb.shape(1)};
  const int64_t c_unit = static_cast<int64_t>(calc_numel(shape_c)) / units;
  Tensor result(shape_c, rt, Device::CPU);
  const size_t es_a = calc_dtype_size(ha.dtype()), es_b = calc_dtype_size(hb.dtype()), es_c = calc_dtype_size(rt);
  std::vector<std::thread> workers;
  std::vector<std::string> errors(static_cast<size_t>(n_gpus));
  for (int r = 0; r < n_gpus; ++r) {
    workers.emplace_back([&, r] {
      try {
        int64_t begin = 0, count = 0;
        tvhost::check(tvb_shard_range(units, granule, n_gpus, r, &begin, &count), "tvb_shard_range");
        if (count == 0) return;
        std::vector<int64_t> sa = ha.shape(), sb = hb.shape();
        sa[0] = count;
        if (batched) sb[0] = count;
        // a slab of leading rows (or batches) is one contiguous piece of the host buffer
        Tensor a_loc(static_cast<char*>(ha.data()) + static_cast<size_t>(begin * a_unit) * es_a, sa, ha.dtype(), Device::CPU);
        Tensor b_loc(static_cast<char*>(hb.data()) + static_cast<size_t>(begin * b_unit) * es_b, sb, hb.dtype(), Device::CPU);
        a_loc.to_device(static_cast<uint32_t>(r));
        b_loc.to_device(static_cast<uint32_t>(r));
        Tensor c_loc = MulImpl<Device::CUDA>::execute(a_loc, b_loc);
        c_loc.to_host();
        std::memcpy(static_cast<char*>(result.data()) + static_cast<size_t>(begin * c_unit) * es_c, c_loc.data(),
                    static_cast<size_t>(count * c_unit) * es_c);
      } catch (const std::exception& e) {
        errors[static_cast<size_t>(r)] = e.what();
      }
    });
  }
  for (std::thread& t : workers) t.join();
  for (const std::string& e : errors)
    if (!e.empty()) throw std::runtime_error("matmul_sharded: " + e);
  return result;
}

Tensor Mul(const Tensor& a, const Tensor& b) {
  check_mul_operands(a, b);
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

namespace {
void check_mul_operands(const Tensor& a, const Tensor& b) {
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
}
}  // namespace

}  // namespace ops
