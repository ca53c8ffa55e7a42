// Host-side planning of a strided box copy (no CUDA in this header, so it is unit-tested on the
// CPU): which indices of the box can be merged, how wide a vector both sides allow, and which
// of the copy kernels fits.
#pragma once
#include <cstddef>
#include <cstdint>

namespace tvb {

struct LayoutDim {
  int64_t size;      // extent
  int64_t sstride;   // elements between consecutive values of the index in the source
  int64_t dstride;   // ... in the destination
};

enum class CopyKind {
  kContiguous,   // one dense run on both sides: a plain device-to-device copy
  kVector,       // innermost run contiguous on both sides: strided_copy_kernel with wide vectors
  kTranspose,    // destination runs along an index the source strides over, while another
                 // index is contiguous in the source: tiled_transpose_kernel
  kElement,      // no contiguous run: strided_copy_kernel, one element per thread
};

struct CopyPlan {
  CopyKind kind;
  int ndim;                 // after merging
  LayoutDim dim[8];         // outermost first
  int vector_bytes;         // kVector: bytes per thread
  int unit_dim;             // kTranspose: the index that is contiguous in the source
};

// Drops indices of extent 1 and merges neighbours that form one run on both sides
// (stride[i] == stride[i+1] * size[i+1]).  Returns the new count (0 for a single element).
inline int merge_dims(LayoutDim* d, int n) {
  int m = 0;
  for (int i = 0; i < n; ++i)
    if (d[i].size != 1) d[m++] = d[i];
  if (m == 0) return 0;
  int w = 0;
  for (int i = 1; i < m; ++i) {
    if (d[w].sstride == d[i].sstride * d[i].size && d[w].dstride == d[i].dstride * d[i].size) {
      d[w].size *= d[i].size;
      d[w].sstride = d[i].sstride;
      d[w].dstride = d[i].dstride;
    } else {
      d[++w] = d[i];
    }
  }
  return w + 1;
}

inline CopyPlan plan_copy(const LayoutDim* dims, int n, size_t elem_size, uintptr_t src_addr, uintptr_t dst_addr) {
  CopyPlan p{};
  for (int i = 0; i < n; ++i) p.dim[i] = dims[i];
  p.ndim = merge_dims(p.dim, n);
  p.vector_bytes = static_cast<int>(elem_size);
  p.unit_dim = -1;
  if (p.ndim == 0) {
    p.dim[0] = LayoutDim{1, 1, 1};
    p.ndim = 1;
  }
  const LayoutDim& last = p.dim[p.ndim - 1];
  if (last.sstride == 1 && last.dstride == 1) {
    if (p.ndim == 1) {
      p.kind = CopyKind::kContiguous;
      return p;
    }
    p.kind = CopyKind::kVector;
    int vb = 16;
    auto fits = [&](int v) {
      if ((static_cast<uint64_t>(last.size) * elem_size) % v != 0) return false;
      if (src_addr % v != 0 || dst_addr % v != 0) return false;
      for (int i = 0; i + 1 < p.ndim; ++i)
        if ((static_cast<uint64_t>(p.dim[i].sstride) * elem_size) % v != 0 ||
            (static_cast<uint64_t>(p.dim[i].dstride) * elem_size) % v != 0)
          return false;
      return true;
    };
    while (vb > static_cast<int>(elem_size) && !fits(vb)) vb /= 2;
    p.vector_bytes = vb;
    return p;
  }
  if (last.dstride == 1) {
    for (int i = p.ndim - 2; i >= 0; --i)
      if (p.dim[i].sstride == 1) {
        p.unit_dim = i;
        break;
      }
    // the tile grid carries the innermost index in gridDim.y (at most 65535 tiles of 32)
    if (p.unit_dim >= 0 && last.size <= 65535ll * 32 && p.dim[p.unit_dim].size <= 0x7FFFFFFFll &&
        last.size <= 0x7FFFFFFFll) {
      p.kind = CopyKind::kTranspose;
      return p;
    }
  }
  p.kind = CopyKind::kElement;
  return p;
}

}  // namespace tvb
