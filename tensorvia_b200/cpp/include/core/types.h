// Element types of the host layer.  Names follow Tensorvia (include/core/types.h of the
// reference: float32, float64, float16, bfloat16, compute_type_t); the half types here are
// plain 16-bit storage with correct round-to-nearest-even conversion — the reference's own
// host bfloat16 constructor zeroes normal values (include/backend/cuda/bfloat16.hpp:26-34),
// which is not reproduced.
#pragma once
#include <cstdint>
#include <cstring>

using float32 = float;
using float64 = double;

namespace tv_detail {
inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

inline uint16_t f32_to_bf16(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
inline uint16_t f32_to_f16(float f) {
  const uint32_t u = f32_bits(f), sign = (u >> 16) & 0x8000u, a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return static_cast<uint16_t>(sign | 0x7E00u);
  if (a >= 0x477FF000u) return static_cast<uint16_t>(sign | 0x7C00u);
  if (a < 0x33000001u) return static_cast<uint16_t>(sign);
  const int e = static_cast<int>(a >> 23) - 127;
  const uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  const uint32_t shift = e < -14 ? static_cast<uint32_t>(13 + (-14 - e)) : 13u;
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  const uint32_t r = e < -14 ? q : ((static_cast<uint32_t>(e + 15) - 1u) << 10) + q;
  return static_cast<uint16_t>(sign | r);
}
inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16, ex = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
  if (ex == 0) {
    const float v = static_cast<float>(man) * (1.0f / 16777216.0f);
    return sign ? -v : v;
  }
  if (ex == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
  return bits_f32(sign | ((ex + 112u) << 23) | (man << 13));
}
}  // namespace tv_detail

struct float16 {
  uint16_t bits = 0;
  float16() = default;
  float16(float f) : bits(tv_detail::f32_to_f16(f)) {}
  operator float() const { return tv_detail::f16_to_f32(bits); }
};
struct bfloat16 {
  uint16_t bits = 0;
  bfloat16() = default;
  bfloat16(float f) : bits(tv_detail::f32_to_bf16(f)) {}
  operator float() const { return tv_detail::bits_f32(static_cast<uint32_t>(bits) << 16); }
};
static_assert(sizeof(float16) == 2 && sizeof(bfloat16) == 2, "half types are 16-bit storage");

// type an element computes in (half types compute as float)
template <typename T> struct compute_type_helper { using type = T; };
template <> struct compute_type_helper<float16> { using type = float; };
template <> struct compute_type_helper<bfloat16> { using type = float; };
template <typename T> using compute_type_t = typename compute_type_helper<T>::type;
