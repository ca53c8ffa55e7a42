/*
 * TEST INFRASTRUCTURE — not part of the product.  Only tests/, the smoke check and the
 * benchmark's CPU-baseline leg may call this file; the product never does.
 *
 * A plain-C restatement of the reference's ops::Typecast (src/ops.cpp:1277-1300): which casts
 * are allowed (valid_casts / is_cast_valid, include/core/type_traits.h:237-291) and what each
 * one computes on the CUDA backend (cast_cuda, src/backend/cuda/typecast.cu:6-27):
 * static_cast between the C types; float -> half and float -> bfloat16 round to nearest even
 * (__float2half, __float2bfloat16); half <-> bfloat16 go through float; float -> integer
 * truncates toward zero.
 *
 * Parity pin: tests/golden/golden_layout.npz holds the reference library's own outputs for the
 * casts whose host arithmetic is the C language's (integers, float, double, and reading half /
 * bfloat16 values); tests/test_oracle_layout.py checks this file against them.  The reference's
 * HOST conversions INTO half and bfloat16 are not used as a pin: its bfloat16_t(float)
 * constructor zeroes normal values (include/backend/cuda/bfloat16.hpp:26-34); for those casts
 * the CUDA backend's round-to-nearest-even is restated and checked against numpy.
 */
#include <stddef.h>
#include <stdint.h>

enum { DT_I8 = 0, DT_I16, DT_I32, DT_I64, DT_BF16, DT_F16, DT_F32, DT_F64 };

float tvo_bf16_to_f32(uint16_t h);
float tvo_f16_to_f32(uint16_t h);
uint16_t tvo_f32_to_bf16(float f);
uint16_t tvo_f32_to_f16(float f);

/* valid_casts, include/core/type_traits.h:237-260, plus the identity (is_cast_valid, :289-291) */
int tvo_cast_valid(int src, int dst) {
  static const int8_t ok[22][2] = {
      {DT_I8, DT_F32},  {DT_I16, DT_F32},  {DT_I16, DT_F64},  {DT_I32, DT_F32},   {DT_I32, DT_F64},  {DT_I64, DT_F64},
      {DT_F32, DT_F16}, {DT_F32, DT_I32},  {DT_F32, DT_I64},  {DT_I8, DT_I16},    {DT_I8, DT_I32},   {DT_I8, DT_I64},
      {DT_I16, DT_I32}, {DT_I32, DT_I64},  {DT_F16, DT_F32},  {DT_F16, DT_F64},   {DT_F16, DT_BF16}, {DT_BF16, DT_F32},
      {DT_BF16, DT_F64}, {DT_BF16, DT_F16}, {DT_F32, DT_F64}, {DT_F64, DT_F32}};
  if (src < 0 || src > 7 || dst < 0 || dst > 7) return 0;
  if (src == dst) return 1;
  for (int i = 0; i < 22; ++i)
    if (ok[i][0] == src && ok[i][1] == dst) return 1;
  return 0;
}

static double load_as_double(const void* p, int dt, size_t i, int64_t* as_int, int* is_int) {
  *is_int = dt <= DT_I64;
  switch (dt) {
    case DT_I8: *as_int = ((const int8_t*)p)[i]; return (double)*as_int;
    case DT_I16: *as_int = ((const int16_t*)p)[i]; return (double)*as_int;
    case DT_I32: *as_int = ((const int32_t*)p)[i]; return (double)*as_int;
    case DT_I64: *as_int = ((const int64_t*)p)[i]; return (double)*as_int;
    case DT_BF16: return (double)tvo_bf16_to_f32(((const uint16_t*)p)[i]);
    case DT_F16: return (double)tvo_f16_to_f32(((const uint16_t*)p)[i]);
    case DT_F32: return (double)((const float*)p)[i];
    default: return ((const double*)p)[i];
  }
}

/* dst[i] = static_cast<dst type>(src[i]); returns 0, or 1 for a cast ops::Typecast refuses. */
int tvo_typecast(const void* src, int sdt, void* dst, int ddt, size_t n) {
  if (!tvo_cast_valid(sdt, ddt)) return 1;
  for (size_t i = 0; i < n; ++i) {
    int64_t iv = 0;
    int is_int = 0;
    const double v = load_as_double(src, sdt, i, &iv, &is_int);
    switch (ddt) {
      case DT_I8: ((int8_t*)dst)[i] = is_int ? (int8_t)iv : (int8_t)v; break;
      case DT_I16: ((int16_t*)dst)[i] = is_int ? (int16_t)iv : (int16_t)v; break;
      case DT_I32: ((int32_t*)dst)[i] = is_int ? (int32_t)iv : (int32_t)(sdt == DT_F32 ? ((const float*)src)[i] : v); break;
      case DT_I64: ((int64_t*)dst)[i] = is_int ? iv : (int64_t)(sdt == DT_F32 ? ((const float*)src)[i] : v); break;
      /* every source that may become half or bfloat16 is itself a float: no double rounding */
      case DT_BF16: ((uint16_t*)dst)[i] = tvo_f32_to_bf16((float)v); break;
      case DT_F16: ((uint16_t*)dst)[i] = tvo_f32_to_f16((float)v); break;
      case DT_F32: ((float*)dst)[i] = is_int ? (float)iv : (float)v; break;
      default: ((double*)dst)[i] = is_int ? (double)iv : v; break;
    }
  }
  return 0;
}
