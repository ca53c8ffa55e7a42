/*
 * TEST INFRASTRUCTURE — not part of the product.  Only tests/, the smoke check and the
 * benchmark's CPU-baseline leg may call this file; the product never does.
 *
 * A plain-C restatement of the reference's data-layout operations on either side of the
 * matmul (views made contiguous, row slices, concatenation): byte moves, so parity is
 * bit-exact.
 *
 *   tvo_repack     TensorImpl::clone_as_contiguous(Metadata) as the CPU tensor does it
 *                  (include/backend/cpu/cpu_tensor.cpp:32-60) and the CUDA repack kernel
 *                  (src/backend/cuda/repack.cu:5-26): the element with row-major index idx
 *                  of the view comes from storage[offset + sum_i coord_i * strides_i].  This
 *                  is what Tensor::contiguous()/clone() apply to the views Tensor::t(),
 *                  permute() and slice() create (src/tensor.cpp:217-310).
 *   tvo_slice      ops::Slice -> SliceImpl<Device::CPU>::execute (src/ops.cpp:158-190,
 *                  src/backend/cpu/slice.cpp:11-63): a dense copy of the window
 *                  [begin_i, end_i) of a dense tensor.
 *   tvo_concat     ops::Concat -> ConcatImpl<Device::CPU>::execute (src/ops.cpp:1301-1333,
 *                  src/backend/cpu/concat.cpp:8-66): dense tensors joined along `dim`.
 *   tvo_transpose  ops::Transpose on a 2-D tensor (src/backend/cpu/transpose.cpp:8-44):
 *                  out[j][i] = in[i][j].
 *
 * Parity pin: tests/golden/golden_layout.npz holds outputs of the reference library itself for
 * these operations (tests/golden/make_golden.py); tests/test_oracle_layout.py checks this file
 * against them.
 *
 * One reference behaviour is NOT restated: Tensor::contiguous() of a leading-dimension slice
 * view returns the storage from its first element on, because such a view passes
 * is_contiguous() (src/tensor.cpp:312-322) and the copy that follows ignores
 * Metadata::offset (src/tensor.cpp:396-403).  tvo_repack honours the offset in every case.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define TVO_MAX_DIMS 8

/* dst[idx] = src[offset + sum coord_i * strides_i], idx walking the view in row-major order.
 * elem_size bytes per element; shape/strides/offset in elements.  Returns 0, or 1 for a bad
 * argument. */
int tvo_repack(const void* src, void* dst, size_t elem_size, int ndim, const int64_t* shape,
               const int64_t* strides, int64_t offset) {
  if (ndim < 0 || ndim > TVO_MAX_DIMS || elem_size == 0) return 1;
  size_t numel = 1;
  for (int i = 0; i < ndim; ++i) {
    if (shape[i] <= 0) return 1;
    numel *= (size_t)shape[i];
  }
  const char* s = (const char*)src + (size_t)offset * elem_size;
  char* d = (char*)dst;
  for (size_t idx = 0; idx < numel; ++idx) {
    size_t t = idx;
    int64_t off = 0;
    for (int i = ndim - 1; i >= 0; --i) {
      const size_t c = t % (size_t)shape[i];
      t /= (size_t)shape[i];
      off += (int64_t)c * strides[i];
    }
    memcpy(d + idx * elem_size, s + off * (int64_t)elem_size, elem_size);
  }
  return 0;
}

/* Dense window copy.  begin/end have `nranges` <= ndim entries; the remaining dimensions are
 * taken whole (slice.cpp:47-57). */
int tvo_slice(const void* src, void* dst, size_t elem_size, int ndim, const int64_t* shape, int nranges,
              const int64_t* begin, const int64_t* end) {
  if (ndim <= 0 || ndim > TVO_MAX_DIMS || nranges > ndim) return 1;
  int64_t strides[TVO_MAX_DIMS], win[TVO_MAX_DIMS];
  int64_t acc = 1, offset = 0;
  for (int i = ndim - 1; i >= 0; --i) {
    strides[i] = acc;
    acc *= shape[i];
  }
  for (int i = 0; i < ndim; ++i) {
    const int64_t b = i < nranges ? begin[i] : 0, e = i < nranges ? end[i] : shape[i];
    if (b < 0 || e > shape[i] || b >= e) return 1;
    win[i] = e - b;
    offset += b * strides[i];
  }
  return tvo_repack(src, dst, elem_size, ndim, win, strides, offset);
}

/* `count` dense tensors of `ndim` dimensions, equal except along `dim` where tensor t has
 * dim_sizes[t] entries; shape gives the common extents (its entry at `dim` is ignored). */
int tvo_concat(int count, const void* const* srcs, void* dst, size_t elem_size, int ndim,
               const int64_t* shape, const int64_t* dim_sizes, int dim) {
  if (count <= 0 || ndim <= 0 || ndim > TVO_MAX_DIMS || dim < 0 || dim >= ndim) return 1;
  size_t outer = 1, inner = 1;
  int64_t total = 0;
  for (int i = 0; i < dim; ++i) outer *= (size_t)shape[i];
  for (int i = dim + 1; i < ndim; ++i) inner *= (size_t)shape[i];
  for (int t = 0; t < count; ++t) total += dim_sizes[t];
  int64_t at = 0;
  for (int t = 0; t < count; ++t) {
    const size_t chunk = (size_t)dim_sizes[t] * inner * elem_size;
    for (size_t o = 0; o < outer; ++o)
      memcpy((char*)dst + (o * (size_t)total + (size_t)at) * inner * elem_size,
             (const char*)srcs[t] + o * chunk, chunk);
    at += dim_sizes[t];
  }
  return 0;
}

int tvo_transpose(const void* src, void* dst, size_t elem_size, int64_t rows, int64_t cols) {
  const int64_t shape[2] = {cols, rows}, strides[2] = {1, cols};
  return tvo_repack(src, dst, elem_size, 2, shape, strides, 0);
}
