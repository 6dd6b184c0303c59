// Element rules of every reduction, written once for the host loops and the device kernels.
//
// Operand convention: `a` is the value already held (accumulator / local), `b` the value that
// arrives; the result replaces `a`. The rules restate the reference's (src/elem.h:20-79):
//   integers      Sum and Prod wrap (computed unsigned); Max = a<b ? b : a; Min = b<a ? b : a
//   float/double  Sum a+b, Prod a*b. A NaN operand wins: the result is the first NaN operand
//                 (a before b) with its quiet bit set, sign and payload kept, which is what an
//                 x86 SSE add/mul returns. A NaN produced from non-NaN operands (inf-inf,
//                 0*inf) is the x86 default NaN (sign set, quiet bit only). Max/Min use the
//                 plain comparisons above, so a NaN on either side keeps `a`.
//   fp16/bf16/fp8 both operands are widened to fp32, combined, and rounded back (fpconv.h).
//                 Max/Min follow glibc fmaxf/fminf on x86-64: a NaN operand yields the other
//                 operand, equal values (also +0 against -0) yield `b`.
// Scaling (Avg on floats, PreMulSum) is Prod with the value as `a` and the scalar as `b`.
// Integer Avg divides the wrapped sum by the rank count in 64 bits, truncating toward zero.
#pragma once
#include <cstdint>
#include <type_traits>

#include "fpconv.h"

namespace hx {

enum : int { kSum = 0, kProd = 1, kMax = 2, kMin = 3 };

HX_HD uint64_t f64_bits(double d) {
#if defined(__CUDA_ARCH__)
  return static_cast<uint64_t>(__double_as_longlong(d));
#else
  uint64_t u;
  std::memcpy(&u, &d, 8);
  return u;
#endif
}
HX_HD double bits_f64(uint64_t u) {
#if defined(__CUDA_ARCH__)
  return __longlong_as_double(static_cast<long long>(u));
#else
  double d;
  std::memcpy(&d, &u, 8);
  return d;
#endif
}

HX_HD bool is_nan(float x) { return (f32_bits(x) & 0x7fffffffu) > 0x7f800000u; }
HX_HD bool is_nan(double x) {
  return (f64_bits(x) & 0x7fffffffffffffffull) > 0x7ff0000000000000ull;
}

// One correctly rounded add / multiply. On the device the intrinsics keep the compiler from
// contracting a scale followed by a sum into a fused multiply-add, which would skip the
// rounding of the product.
HX_HD float add_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fadd_rn(a, b);
#else
  return a + b;
#endif
}
HX_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}
HX_HD double add_rn(double a, double b) {
#if defined(__CUDA_ARCH__)
  return __dadd_rn(a, b);
#else
  return a + b;
#endif
}
HX_HD double mul_rn(double a, double b) {
#if defined(__CUDA_ARCH__)
  return __dmul_rn(a, b);
#else
  return a * b;
#endif
}

HX_HD float arith(float a, float b, int op) {
  if (is_nan(a)) return bits_f32(f32_bits(a) | 0x00400000u);
  if (is_nan(b)) return bits_f32(f32_bits(b) | 0x00400000u);
  const float r = op == kSum ? add_rn(a, b) : mul_rn(a, b);
  return is_nan(r) ? bits_f32(0xffc00000u) : r;
}
HX_HD double arith(double a, double b, int op) {
  if (is_nan(a)) return bits_f64(f64_bits(a) | 0x0008000000000000ull);
  if (is_nan(b)) return bits_f64(f64_bits(b) | 0x0008000000000000ull);
  const double r = op == kSum ? add_rn(a, b) : mul_rn(a, b);
  return is_nan(r) ? bits_f64(0xfff8000000000000ull) : r;
}

// integers
template <typename T>
HX_HD typename std::enable_if<std::is_integral<T>::value, T>::type apply(T a, T b, int op) {
  using U = typename std::make_unsigned<T>::type;
  switch (op) {
    case kSum: return static_cast<T>(static_cast<U>(static_cast<U>(a) + static_cast<U>(b)));
    case kProd: return static_cast<T>(static_cast<U>(static_cast<U>(a) * static_cast<U>(b)));
    case kMax: return a < b ? b : a;
    default: return b < a ? b : a;
  }
}
// float, double
template <typename T>
HX_HD typename std::enable_if<std::is_floating_point<T>::value, T>::type apply(T a, T b,
                                                                                int op) {
  switch (op) {
    case kSum:
    case kProd: return arith(a, b, op);
    case kMax: return a < b ? b : a;
    default: return b < a ? b : a;
  }
}

HX_HD float narrow_combine(float a, float b, int op) {
  switch (op) {
    case kSum: return add_rn(a, b);
    case kProd: return mul_rn(a, b);
    case kMax: return is_nan(b) ? a : is_nan(a) ? b : (a > b ? a : b);
    default: return is_nan(b) ? a : is_nan(a) ? b : (a < b ? a : b);
  }
}
template <typename S>
HX_HD S apply_narrow(S a, S b, int op) {
  S out;
  from_f32(narrow_combine(to_f32(a), to_f32(b), op), &out);
  return out;
}
HX_HD f16 apply(f16 a, f16 b, int op) { return apply_narrow(a, b, op); }
HX_HD bf16 apply(bf16 a, bf16 b, int op) { return apply_narrow(a, b, op); }
HX_HD e4m3 apply(e4m3 a, e4m3 b, int op) { return apply_narrow(a, b, op); }
HX_HD e5m2 apply(e5m2 a, e5m2 b, int op) { return apply_narrow(a, b, op); }

// value * scalar under the Prod rule, value on the left
template <typename T>
HX_HD T scale(T v, T k) { return apply(v, k, kProd); }

// integer Avg: 64-bit division truncating toward zero (wide type follows signedness)
template <typename T>
HX_HD typename std::enable_if<std::is_integral<T>::value, T>::type div_trunc(T v, int d) {
  using W = typename std::conditional<std::is_signed<T>::value, int64_t, uint64_t>::type;
  return static_cast<T>(static_cast<W>(v) / static_cast<W>(d));
}
template <typename T>
HX_HD typename std::enable_if<!std::is_integral<T>::value, T>::type div_trunc(T v, int) {
  return v;
}

template <typename T> struct is_int_elem : std::is_integral<T> {};

}  // namespace hx
