// CUDA-core GEMM for every (A dtype, B dtype) pair of the eight Tensorvia dtypes.
//
// It carries the semantics of the reference kernel mul_cuda_3d
// (src/backend/cuda/mul.cu:8-48) for the pairs and shapes the tensor-core kernel
// does not take:
//   * accumulator type = decltype(compute_type_t<T>() + compute_type_t<R>()) with
//     half/bf16 computing as float (mul.cu:19, include/core/types.h:111-117);
//   * one accumulator per output, k walked in increasing order;
//   * result = static_cast<S>(sum), S = via::compute_type(dtype(A), dtype(B))
//     (mul.cu:46,63; include/core/type_traits.h:270-287).
// Unlike the reference, FLOAT64 results use the real column count (the reference
// passes `rows` for `cols` at mul.cu:91 and is wrong for non-square outputs).
//
// Tiling: 64x64 outputs per 256-thread CTA, 4x4 per thread, K in steps of 16
// through shared memory; operands are converted to the accumulator type on load.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <type_traits>

namespace tvb {

// dtype number -> C++ type on the device
template <int DT> struct DevType;
template <> struct DevType<0> { using type = int8_t; };
template <> struct DevType<1> { using type = int16_t; };
template <> struct DevType<2> { using type = int32_t; };
template <> struct DevType<3> { using type = int64_t; };
template <> struct DevType<4> { using type = __nv_bfloat16; };
template <> struct DevType<5> { using type = __half; };
template <> struct DevType<6> { using type = float; };
template <> struct DevType<7> { using type = double; };

// via::compute_type (include/core/type_traits.h:270-287) as a constant expression.
__host__ __device__ constexpr int compute_type_of(int a, int b) {
  if (a == b) return a;
  const int mx = a > b ? a : b;
  if (a <= 3 && b <= 3) return mx;                       // both integers: the wider
  if (a > 3 && b > 3) return mx > 6 ? mx : 6;            // both floats: at least FLOAT32
  if (a == 3 || b == 3) return 7;                        // INT64 with a float: FLOAT64
  return mx > 6 ? mx : 6;                                // other int with float
}

template <typename T> struct ComputeOf { using type = T; };
template <> struct ComputeOf<__half> { using type = float; };
template <> struct ComputeOf<__nv_bfloat16> { using type = float; };

template <int DA, int DB>
struct PairTraits {
  using A = typename DevType<DA>::type;
  using B = typename DevType<DB>::type;
  using Out = typename DevType<compute_type_of(DA, DB)>::type;
  using Acc = decltype(std::declval<typename ComputeOf<A>::type>() +
                       std::declval<typename ComputeOf<B>::type>());
};

template <typename Acc, typename T>
__device__ __forceinline__ Acc to_acc(T x) {
  if constexpr (std::is_same_v<T, __half>) return static_cast<Acc>(__half2float(x));
  else if constexpr (std::is_same_v<T, __nv_bfloat16>) return static_cast<Acc>(__bfloat162float(x));
  else return static_cast<Acc>(x);
}
template <typename Out, typename Acc>
__device__ __forceinline__ Out from_acc(Acc x) {
  if constexpr (std::is_same_v<Out, __half>) return __float2half_rn(static_cast<float>(x));
  else if constexpr (std::is_same_v<Out, __nv_bfloat16>) return __float2bfloat16_rn(static_cast<float>(x));
  else return static_cast<Out>(x);
}

// Element strides of the two operands: A(b, m, k) = A[b*a_b + m*a_r + k*a_c], B(b, k, n) likewise.
// Dense row-major operands have a_b = M*K, a_r = K, a_c = 1 and b_b = K*N, b_r = N, b_c = 1.
struct SimtStrides {
  int64_t a_b, a_r, a_c, b_b, b_r, b_c;
};

template <int DA, int DB>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(const void* __restrict__ Av, const void* __restrict__ Bv, void* __restrict__ Cv,
                 int M, int N, int K, const SimtStrides st) {
  using PT = PairTraits<DA, DB>;
  using TA = typename PT::A;
  using TB = typename PT::B;
  using Acc = typename PT::Acc;
  using Out = typename PT::Out;
  constexpr int TM = 64, TN = 64, TK = 16;

  __shared__ Acc As[TK][TM + 1];
  __shared__ Acc Bs[TK][TN];

  const size_t batch = blockIdx.z;
  const TA* A = static_cast<const TA*>(Av) + static_cast<int64_t>(batch) * st.a_b;
  const TB* B = static_cast<const TB*>(Bv) + static_cast<int64_t>(batch) * st.b_b;
  Out* C = static_cast<Out*>(Cv) + batch * static_cast<size_t>(M) * N;

  const int tx = threadIdx.x & 15;   // 4 columns each
  const int ty = threadIdx.x >> 4;   // 4 rows each
  const int m0 = blockIdx.y * TM;
  const int n0 = blockIdx.x * TN;

  Acc acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = Acc(0);

  for (int k0 = 0; k0 < K; k0 += TK) {
    // A tile: 64 rows x 16 k; thread t loads row t/4, 4 consecutive k
    {
      const int r = threadIdx.x >> 2;
      const int kk = (threadIdx.x & 3) * 4;
      const int gr = m0 + r;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gk = k0 + kk + j;
        As[kk + j][r] = (gr < M && gk < K) ? to_acc<Acc>(A[gr * st.a_r + gk * st.a_c]) : Acc(0);
      }
    }
    // B tile: 16 k x 64 columns; thread t loads k row t/16, 4 consecutive columns
    {
      const int kk = threadIdx.x >> 4;
      const int c = (threadIdx.x & 15) * 4;
      const int gk = k0 + kk;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gc = n0 + c + j;
        Bs[kk][c + j] = (gk < K && gc < N) ? to_acc<Acc>(B[gk * st.b_r + gc * st.b_c]) : Acc(0);
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      Acc a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = m0 + ty * 4 + i;
    if (gr >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = n0 + tx * 4 + j;
      if (gc < N) C[static_cast<size_t>(gr) * N + gc] = from_acc<Out>(acc[i][j]);
    }
  }
}

}  // namespace tvb
