// Byte movers for the layout operations on either side of the matmul: a strided view made
// contiguous (Tensor::contiguous / clone, i.e. TensorImpl::clone_as_contiguous), ops::Slice,
// ops::Concat and the 2-D ops::Transpose.  All are HBM-bound: every element is read once and
// written once, so the roofline is 2 * bytes / HBM bandwidth.
//
//   strided_copy_kernel   an n-dimensional box whose innermost run is contiguous on both sides:
//                         one thread per vector of up to 16 bytes, coordinates decoded with
//                         multiply-shift division, loads and stores coalesced along the run.
//                         Also the element-by-element fallback (vector = one element) for
//                         views with no contiguous run at all.
//   tiled_transpose_kernel views whose innermost index is NOT the contiguous one but another
//                         index is (a transposed or permuted view): tiles of the plane spanned
//                         by the two indices go through shared memory, so reads are coalesced
//                         along the source's contiguous index and writes along the
//                         destination's.  tiled_transpose_words_kernel is its form for 1-, 2-
//                         and 4-byte elements in word-aligned runs: 32-bit global accesses,
//                         narrow elements transposed in registers.
//
// The reference does the first job with one thread per element and a per-byte copy loop after
// allocating and copying its shape metadata per call (src/backend/cuda/repack.cu:5-54), the
// slices and concatenations with per-element coordinate kernels on managed-memory metadata
// (src/backend/cuda/slice.cu:7-114, concat.cu:8-158) and the 2-D transpose with a per-element
// kernel (src/backend/cuda/transpose.cu:8-51).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace tvb {

constexpr int kMaxLayoutDims = 8;

// n / d for n < 2^31 by multiply-high and shift (d >= 1).
struct FastDiv {
  uint32_t d, m, s;
};
inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  f.d = d;
  uint32_t s = 0;
  while ((1ull << s) < d) ++s;
  f.s = s;
  f.m = static_cast<uint32_t>(((1ull << 32) * ((1ull << s) - d)) / d + 1);
  return f;
}
__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f) {
  return (__umulhi(n, f.m) + n) >> f.s;
}

// A box of `ndim` indices (index 0 outermost).  The innermost index counts VECTORS of the
// kernel's copy type; strides are in bytes on both sides.
struct BoxParams {
  int32_t ndim;
  uint32_t size[kMaxLayoutDims];
  FastDiv div[kMaxLayoutDims];
  int64_t src_stride[kMaxLayoutDims];
  int64_t dst_stride[kMaxLayoutDims];
};

// V = copy type (uint8_t, uint16_t, uint32_t, uint64_t or uint4).  total < 2^31.
template <typename V>
__global__ void __launch_bounds__(256)
strided_copy_kernel(const char* __restrict__ src, char* __restrict__ dst, uint32_t total, const BoxParams p) {
  // four vectors per thread and trip: all four loads are issued before the first store
  constexpr int UNROLL = 4;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x * UNROLL;
  for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * blockDim.x * UNROLL + threadIdx.x; base < total;
       base += stride) {
    V v[UNROLL];
    int64_t dof[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const uint64_t idx = base + static_cast<uint64_t>(k) * blockDim.x;
      dof[k] = -1;
      if (idx < total) {
        uint32_t rem = static_cast<uint32_t>(idx);
        int64_t so = 0, d = 0;
#pragma unroll
        for (int i = kMaxLayoutDims - 1; i >= 1; --i) {
          if (i < p.ndim) {
            const uint32_t q = fast_div(rem, p.div[i]);
            const uint32_t c = rem - q * p.size[i];
            so += static_cast<int64_t>(c) * p.src_stride[i];
            d += static_cast<int64_t>(c) * p.dst_stride[i];
            rem = q;
          }
        }
        so += static_cast<int64_t>(rem) * p.src_stride[0];
        d += static_cast<int64_t>(rem) * p.dst_stride[0];
        v[k] = *reinterpret_cast<const V*>(src + so);
        dof[k] = d;
      }
    }
#pragma unroll
    for (int k = 0; k < UNROLL; ++k)
      if (dof[k] >= 0) *reinterpret_cast<V*>(dst + dof[k]) = v[k];
  }
}

// The same for boxes of 2^31 vectors and more: plain 64-bit arithmetic.
template <typename V>
__global__ void __launch_bounds__(256)
strided_copy_kernel_big(const char* __restrict__ src, char* __restrict__ dst, uint64_t total, const BoxParams p) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    uint64_t rem = idx;
    int64_t so = 0, dof = 0;
    for (int i = p.ndim - 1; i >= 1; --i) {
      const uint64_t q = rem / p.size[i];
      const uint64_t c = rem - q * p.size[i];
      so += static_cast<int64_t>(c) * p.src_stride[i];
      dof += static_cast<int64_t>(c) * p.dst_stride[i];
      rem = q;
    }
    so += static_cast<int64_t>(rem) * p.src_stride[0];
    dof += static_cast<int64_t>(rem) * p.dst_stride[0];
    *reinterpret_cast<V*>(dst + dof) = *reinterpret_cast<const V*>(src + so);
  }
}

// Transposing copy.  The view has its innermost index `l` (extent nl, source stride sl elements,
// destination stride 1) and another index `u` (extent nu, source stride 1, destination stride du
// elements).  The remaining indices form the `outer` box, decoded once per block from
// blockIdx.z (+ z0); their strides are in elements.  TILE x TILE elements per block, 256 threads.
struct TransposeParams {
  int32_t nl, nu;
  int64_t sl, du;
  int32_t n_outer;                       // number of outer indices
  uint32_t osize[kMaxLayoutDims];
  int64_t osrc[kMaxLayoutDims], odst[kMaxLayoutDims];
  uint32_t z0;
};

template <typename T, int TILE>
__global__ void __launch_bounds__(256)
tiled_transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, const TransposeParams p) {
  // +1 word of padding per row keeps both phases free of bank conflicts for 4-byte elements
  // and at most 2-way for narrower ones
  __shared__ T tile[TILE][TILE + (sizeof(T) >= 4 ? 1 : 4 / sizeof(T))];
  uint32_t z = blockIdx.z + p.z0;
  int64_t so = 0, dof = 0;
  for (int i = p.n_outer - 1; i >= 0; --i) {
    const uint32_t q = z / p.osize[i];
    const uint32_t c = z - q * p.osize[i];
    so += static_cast<int64_t>(c) * p.osrc[i];
    dof += static_cast<int64_t>(c) * p.odst[i];
    z = q;
  }
  const int u0 = blockIdx.x * TILE, l0 = blockIdx.y * TILE;
  constexpr int ROWS_PER_PASS = 256 / TILE;   // TILE = 32: 8 rows per pass, TILE = 64: 4
  const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
  // read: rows of the tile run along u (contiguous in the source)
#pragma unroll
  for (int r = ty; r < TILE; r += ROWS_PER_PASS) {
    const int l = l0 + r, u = u0 + tx;
    if (l < p.nl && u < p.nu) tile[r][tx] = src[so + static_cast<int64_t>(l) * p.sl + u];
  }
  __syncthreads();
  // write: rows run along l (contiguous in the destination)
#pragma unroll
  for (int r = ty; r < TILE; r += ROWS_PER_PASS) {
    const int u = u0 + r, l = l0 + tx;
    if (u < p.nu && l < p.nl) dst[dof + static_cast<int64_t>(u) * p.du + l] = tile[tx][r];
  }
}

// The transposing copy for 1-, 2- and 4-byte elements when every run starts on a 4-byte boundary
// and holds whole 32-bit words on both sides (extents, strides and bases multiples of SUB
// elements): global memory is touched only in 32-bit words, 128 bytes per warp and row on the
// way in, and the SUB x SUB blocks of narrow elements are transposed in registers with byte
// permutes on the way out.  SUB = elements per word.  A tile holds ROWS values of l by UW words
// of u; its shared-memory rows are UW + 1 words long, and the lane-to-item maps below keep every
// shared-memory access free of bank conflicts.
template <int SUB, int ROWS, int UW>
__global__ void __launch_bounds__(256)
tiled_transpose_words_kernel(const char* __restrict__ src, char* __restrict__ dst, const TransposeParams p) {
  constexpr int ES = 4 / SUB;
  __shared__ uint32_t tile[ROWS][UW + 1];
  uint32_t z = blockIdx.z + p.z0;
  int64_t so = 0, dof = 0;
  for (int i = p.n_outer - 1; i >= 0; --i) {
    const uint32_t q = z / p.osize[i];
    const uint32_t c = z - q * p.osize[i];
    so += static_cast<int64_t>(c) * p.osrc[i];
    dof += static_cast<int64_t>(c) * p.odst[i];
    z = q;
  }
  const char* sbase = src + so * ES;
  char* dbase = dst + dof * ES;
  const int u0 = blockIdx.x * UW * SUB, l0 = blockIdx.y * ROWS;
#pragma unroll
  for (int it = threadIdx.x; it < ROWS * UW; it += 256) {
    const int r = it / UW, c = it % UW;
    const int l = l0 + r, u = u0 + c * SUB;
    if (l < p.nl && u < p.nu)
      tile[r][c] = *reinterpret_cast<const uint32_t*>(sbase + (static_cast<int64_t>(l) * p.sl + u) * ES);
  }
  __syncthreads();
  auto put = [&](int u, int l, uint32_t w) {
    if (u < p.nu) *reinterpret_cast<uint32_t*>(dbase + (static_cast<int64_t>(u) * p.du + l) * ES) = w;
  };
  if constexpr (SUB == 1) {
#pragma unroll
    for (int it = threadIdx.x; it < ROWS * UW; it += 256) {
      const int l = it % ROWS, uu = it / ROWS;
      if (l0 + l < p.nl) put(u0 + uu, l0 + l, tile[l][uu]);
    }
  } else if constexpr (SUB == 2) {
#pragma unroll
    constexpr int LP = ROWS / 2;   // pairs of l per tile
    for (int it = threadIdx.x; it < LP * UW; it += 256) {
      // 16 consecutive pairs x 2 words per warp: banks 2*lp + uw are all different
      const int lp = (it & 15) | (((it >> 5) % (LP / 16)) << 4), uw = ((it >> 4) & 1) | (((it >> 5) / (LP / 16)) << 1);
      const uint32_t w0 = tile[2 * lp][uw], w1 = tile[2 * lp + 1][uw];
      const int l = l0 + 2 * lp, u = u0 + 2 * uw;
      if (l < p.nl) {
        put(u, l, __byte_perm(w0, w1, 0x5410));
        put(u + 1, l, __byte_perm(w0, w1, 0x7632));
      }
    }
  } else {
#pragma unroll
    constexpr int LQ = ROWS / 4;   // quads of l per tile
    for (int it = threadIdx.x; it < LQ * UW; it += 256) {
      // 8 consecutive quads x 4 words per warp: banks 4*lq + uw are all different
      const int lq = (it & 7) | (((it >> 5) % (LQ / 8)) << 3), uw = ((it >> 3) & 3) | (((it >> 5) / (LQ / 8)) << 2);
      const uint32_t w0 = tile[4 * lq][uw], w1 = tile[4 * lq + 1][uw], w2 = tile[4 * lq + 2][uw],
                     w3 = tile[4 * lq + 3][uw];
      const int l = l0 + 4 * lq, u = u0 + 4 * uw;
      if (l < p.nl) {
        const uint32_t t0 = __byte_perm(w0, w1, 0x5140), t1 = __byte_perm(w2, w3, 0x5140);
        const uint32_t t2 = __byte_perm(w0, w1, 0x7362), t3 = __byte_perm(w2, w3, 0x7362);
        put(u, l, __byte_perm(t0, t1, 0x5410));
        put(u + 1, l, __byte_perm(t0, t1, 0x7632));
        put(u + 2, l, __byte_perm(t2, t3, 0x5410));
        put(u + 3, l, __byte_perm(t2, t3, 0x7632));
      }
    }
  }
}

// The transposing copy at full width: 16-byte global accesses on both sides.  Needs every run
// to start on a 16-byte boundary and to hold whole 16-byte vectors (extents of the two plane
// indices, all strides and both bases multiples of 16 bytes).  A tile is 128 bytes of u by
// LR x 128 bytes of l.  Each thread loads one 16-byte vector from each of SUB consecutive rows of
// l (LR times),
// transposes the SUB x SUB blocks of narrow elements in registers, and writes words that hold
// SUB consecutive values of l into a shared tile whose rows run along l.  That tile is not
// padded: its 16-byte groups are XOR-swizzled with the source vector index, which makes the
// word stores of a warp hit 32 different banks and keeps the 16-byte reads of the second
// phase conflict-free too.
template <int SUB, int LR>
__global__ void __launch_bounds__(256)
tiled_transpose_vec_kernel(const char* __restrict__ src, char* __restrict__ dst, const TransposeParams p) {
  constexpr int ES = 4 / SUB;
  constexpr int TU = 32 * SUB;        // values of u per tile
  constexpr int TL = 32 * SUB * LR;   // values of l per tile: LR groups of SUB rows per thread
  constexpr int ROW_WORDS = 32 * LR;
  __shared__ uint4 tile[TU][8 * LR];  // [u][ROW_WORDS words along l]
  uint32_t z = blockIdx.z + p.z0;
  int64_t so = 0, dof = 0;
  for (int i = p.n_outer - 1; i >= 0; --i) {
    const uint32_t q = z / p.osize[i];
    const uint32_t c = z - q * p.osize[i];
    so += static_cast<int64_t>(c) * p.osrc[i];
    dof += static_cast<int64_t>(c) * p.odst[i];
    z = q;
  }
  const char* sbase = src + so * ES;
  char* dbase = dst + dof * ES;
  const int u0 = blockIdx.x * TU, l0 = blockIdx.y * TL;
  {
    const int uv = threadIdx.x & 7;
    const int u = u0 + uv * 4 * SUB;
    uint32_t w[LR][SUB][4];
    // every load of the thread is issued before the first shared-memory store
#pragma unroll
    for (int r = 0; r < LR; ++r) {
      const int l = l0 + ((threadIdx.x >> 3) + 32 * r) * SUB;
      if (u < p.nu && l < p.nl) {
#pragma unroll
        for (int h = 0; h < SUB; ++h) {
          const uint4 v = *reinterpret_cast<const uint4*>(sbase + (static_cast<int64_t>(l + h) * p.sl + u) * ES);
          w[r][h][0] = v.x; w[r][h][1] = v.y; w[r][h][2] = v.z; w[r][h][3] = v.w;
        }
      }
    }
    uint32_t* t = reinterpret_cast<uint32_t*>(tile);
#pragma unroll
    for (int r = 0; r < LR; ++r) {
      const int lg = (threadIdx.x >> 3) + 32 * r;
      if (!(u < p.nu && l0 + lg * SUB < p.nl)) continue;
      const int col = lg ^ (uv << 2);
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int row = uv * 4 * SUB + m * SUB;
        if constexpr (SUB == 1) {
          t[row * ROW_WORDS + col] = w[r][0][m];
        } else if constexpr (SUB == 2) {
          t[row * ROW_WORDS + col] = __byte_perm(w[r][0][m], w[r][1][m], 0x5410);
          t[(row + 1) * ROW_WORDS + col] = __byte_perm(w[r][0][m], w[r][1][m], 0x7632);
        } else {
          const uint32_t t0 = __byte_perm(w[r][0][m], w[r][1][m], 0x5140), t1 = __byte_perm(w[r][2][m], w[r][3][m], 0x5140);
          const uint32_t t2 = __byte_perm(w[r][0][m], w[r][1][m], 0x7362), t3 = __byte_perm(w[r][2][m], w[r][3][m], 0x7362);
          t[row * ROW_WORDS + col] = __byte_perm(t0, t1, 0x5410);
          t[(row + 1) * ROW_WORDS + col] = __byte_perm(t0, t1, 0x7632);
          t[(row + 2) * ROW_WORDS + col] = __byte_perm(t2, t3, 0x5410);
          t[(row + 3) * ROW_WORDS + col] = __byte_perm(t2, t3, 0x7632);
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = threadIdx.x; it < TU * 8 * LR; it += 256) {
    const int c = it % (8 * LR), row = it / (8 * LR);
    const int u = u0 + row, l = l0 + c * 4 * SUB;
    if (u < p.nu && l < p.nl)
      *reinterpret_cast<uint4*>(dbase + (static_cast<int64_t>(u) * p.du + l) * ES) = tile[row][c ^ ((row / (4 * SUB)) & 7)];
  }
}

}  // namespace tvb
