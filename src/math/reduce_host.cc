#include "reduce_host.h"

#include <cstring>
#include <memory>
#include <mutex>
#if defined(__x86_64__) && defined(__GNUC__)
#include <immintrin.h>
#endif

// The loops of this file are the host data path: let the compiler unroll and vectorise them
// whatever level the rest of the library is built at (no value-changing option is implied;
// contraction stays off through the command line).
#if defined(__GNUC__) && !defined(__clang__)
#pragma GCC optimize("O3")
#endif

namespace hx {

namespace {
// float / double Sum and Prod. The element rule (elem.h: arith) differs from the machine's plain
// a + b / a * b only where the result is a NaN (a NaN operand, inf - inf, 0 * inf): there it
// fixes which NaN comes out. So a tile is first computed with plain arithmetic, which the
// compiler vectorises, and the rule is applied element by element only to tiles whose plain
// results contain a NaN. Bit-identical to the rule everywhere, several times faster on finite
// data (the reference's host loop is the plain form throughout, src/reduce.cc:16-18, and gets
// its NaN behaviour from the x86 instruction; this one does not depend on the machine).
template <typename F>
void arith_tiles(F* out, const F* a, const F* b, size_t count, int op) {
  constexpr size_t kTile = 256;
  F tile[kTile];
  for (size_t i0 = 0; i0 < count; i0 += kTile) {
    const size_t n = count - i0 < kTile ? count - i0 : kTile;
    if (op == kSum) {
      for (size_t i = 0; i < n; ++i) tile[i] = a[i0 + i] + b[i0 + i];
    } else {
      for (size_t i = 0; i < n; ++i) tile[i] = a[i0 + i] * b[i0 + i];
    }
    int special = 0;  // a loop of its own: both then vectorise
    for (size_t i = 0; i < n; ++i) special += tile[i] != tile[i];
    if (special) {
      for (size_t i = 0; i < n; ++i) out[i0 + i] = arith(a[i0 + i], b[i0 + i], op);
    } else {
      std::memcpy(out + i0, tile, n * sizeof(F));
    }
  }
}
// The same for value * scalar.
template <typename F>
void scale_tiles(F* out, const F* src, F k, size_t count) {
  constexpr size_t kTile = 256;
  F tile[kTile];
  for (size_t i0 = 0; i0 < count; i0 += kTile) {
    const size_t n = count - i0 < kTile ? count - i0 : kTile;
    for (size_t i = 0; i < n; ++i) tile[i] = src[i0 + i] * k;
    int special = 0;
    for (size_t i = 0; i < n; ++i) special += tile[i] != tile[i];
    if (special) {
      for (size_t i = 0; i < n; ++i) out[i0 + i] = arith(src[i0 + i], k, kProd);
    } else {
      std::memcpy(out + i0, tile, n * sizeof(F));
    }
  }
}
// The narrow floats have few codes: for a long vector the scaled value of every code is worked
// out once with the rule and the vector is mapped through that table.
template <typename T>
bool table_scale(T*, const T*, T, size_t) { return false; }
template <typename T, typename Bits>
bool map_codes(T* o, const T* s, T k, size_t n) {
  constexpr size_t kCodes = size_t(1) << (8 * sizeof(Bits));
  if (n < 4 * kCodes) return false;
  std::unique_ptr<Bits[]> table(new Bits[kCodes]);
  for (size_t c = 0; c < kCodes; ++c) table[c] = scale(T{Bits(c)}, k).b;
  for (size_t i = 0; i < n; ++i) o[i].b = table[s[i].b];
  return true;
}
template <>
bool table_scale<e4m3>(e4m3* o, const e4m3* s, e4m3 k, size_t n) { return map_codes<e4m3, uint8_t>(o, s, k, n); }
template <>
bool table_scale<e5m2>(e5m2* o, const e5m2* s, e5m2 k, size_t n) { return map_codes<e5m2, uint8_t>(o, s, k, n); }
template <>
bool table_scale<f16>(f16* o, const f16* s, f16 k, size_t n) { return map_codes<f16, uint16_t>(o, s, k, n); }
template <>
bool table_scale<bf16>(bf16* o, const bf16* s, bf16 k, size_t n) { return map_codes<bf16, uint16_t>(o, s, k, n); }
template <typename T>
bool fast_scale(T*, const T*, T, size_t) { return false; }
template <>
bool fast_scale<float>(float* o, const float* s, float k, size_t n) {
  scale_tiles(o, s, k, n);
  return true;
}
template <>
bool fast_scale<double>(double* o, const double* s, double k, size_t n) {
  scale_tiles(o, s, k, n);
  return true;
}
// The 8-bit float types have 256 x 256 operand pairs: the element rule is evaluated once per
// pair into a 64 KiB table per type and operator, on first use, and a reduce is one lookup per
// element after that (the rule itself decodes to float, combines, and rounds back per element).
template <typename T>
const uint8_t* pair_table(int op) {
  static uint8_t table[4][256 * 256];
  static std::once_flag built[4];
  std::call_once(built[op], [op] {
    for (int a = 0; a < 256; ++a)
      for (int b = 0; b < 256; ++b)
        table[op][a * 256 + b] = apply(T{uint8_t(a)}, T{uint8_t(b)}, op).b;
  });
  return table[op];
}
template <typename T>
bool fast_pairs(T*, const T*, const T*, size_t, int) { return false; }
template <typename T>
bool lookup_pairs(T* o, const T* a, const T* b, size_t n, int op) {
  if (op < 0 || op >= 4) return false;
  const uint8_t* t = pair_table<T>(op);
  for (size_t i = 0; i < n; ++i) o[i].b = t[a[i].b * 256 + b[i].b];
  return true;
}
template <>
bool fast_pairs<e4m3>(e4m3* o, const e4m3* a, const e4m3* b, size_t n, int op) { return lookup_pairs(o, a, b, n, op); }
template <>
bool fast_pairs<e5m2>(e5m2* o, const e5m2* a, const e5m2* b, size_t n, int op) { return lookup_pairs(o, a, b, n, op); }
#if defined(__x86_64__) && defined(__GNUC__)
#define HX_HAVE_F16C_PATH 1
// fp16 Sum / Prod with the machine's half <-> float conversions, eight elements at a time. The
// conversions are exact (widening) and round to nearest even with gradual underflow and
// overflow to infinity (narrowing), as the element rule does; the rule differs only in what
// NaN comes out (always the canonical one), which is patched in afterwards.
__attribute__((target("avx2,f16c"))) void f16_arith_x86(uint16_t* o, const uint16_t* a, const uint16_t* b,
                                                       size_t n, bool sum) {
  const __m128i exp = _mm_set1_epi16(0x7c00), man = _mm_set1_epi16(0x03ff);
  const __m128i canon = _mm_set1_epi16(0x7e00), zero = _mm_setzero_si128();
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 fa = _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i*>(a + i)));
    const __m256 fb = _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i*>(b + i)));
    const __m256 r = sum ? _mm256_add_ps(fa, fb) : _mm256_mul_ps(fa, fb);
    __m128i h = _mm256_cvtps_ph(r, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
    const __m128i all_ones_exp = _mm_cmpeq_epi16(_mm_and_si128(h, exp), exp);
    const __m128i no_mantissa = _mm_cmpeq_epi16(_mm_and_si128(h, man), zero);
    const __m128i nan = _mm_andnot_si128(no_mantissa, all_ones_exp);
    h = _mm_blendv_epi8(h, canon, nan);
    _mm_storeu_si128(reinterpret_cast<__m128i*>(o + i), h);
  }
  for (; i < n; ++i) o[i] = apply(f16{a[i]}, f16{b[i]}, sum ? kSum : kProd).b;
}
bool f16_hw() {
  static const bool yes = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c");
  return yes;
}
#endif
template <typename T>
bool fast_arith(T*, const T*, const T*, size_t, int) { return false; }
#ifdef HX_HAVE_F16C_PATH
template <>
bool fast_arith<f16>(f16* o, const f16* a, const f16* b, size_t n, int op) {
  if (!f16_hw()) return false;
  static_assert(sizeof(f16) == 2, "f16 is its 16 bits");
  f16_arith_x86(reinterpret_cast<uint16_t*>(o), reinterpret_cast<const uint16_t*>(a),
                reinterpret_cast<const uint16_t*>(b), n, op == kSum);
  return true;
}
#endif
template <>
bool fast_arith<float>(float* o, const float* a, const float* b, size_t n, int op) {
  arith_tiles(o, a, b, n, op);
  return true;
}
template <>
bool fast_arith<double>(double* o, const double* a, const double* b, size_t n, int op) {
  arith_tiles(o, a, b, n, op);
  return true;
}
}  // namespace

void combine(void* out, const void* in_a, const void* in_b, size_t count, int dt, int op) {
  HX_DISPATCH_DTYPE(dt, {
    T* o = static_cast<T*>(out);
    const T* a = static_cast<const T*>(in_a);
    const T* b = static_cast<const T*>(in_b);
    if ((op == kSum || op == kProd) && fast_arith<T>(o, a, b, count, op)) break;
    if (count >= 4096 && fast_pairs<T>(o, a, b, count, op)) break;  // small calls do not pay for the table
    switch (op) {  // hoisted so each loop body is branch-free
      case kSum: for (size_t i = 0; i < count; ++i) o[i] = apply(a[i], b[i], kSum); break;
      case kProd: for (size_t i = 0; i < count; ++i) o[i] = apply(a[i], b[i], kProd); break;
      case kMax: for (size_t i = 0; i < count; ++i) o[i] = apply(a[i], b[i], kMax); break;
      case kMin: for (size_t i = 0; i < count; ++i) o[i] = apply(a[i], b[i], kMin); break;
      default: break;
    }
  })
}

void reduce_into(void* dst, const void* src, size_t count, int dt, int op) {
  combine(dst, dst, src, count, dt, op);
}

void scale_into(void* dst, const void* src, size_t count, int dt, const void* scalar) {
  HX_DISPATCH_DTYPE(dt, {
    T k;
    std::memcpy(&k, scalar, sizeof(T));
    T* o = static_cast<T*>(dst);
    const T* s = static_cast<const T*>(src);
    if (fast_scale<T>(o, s, k, count)) break;
    if (table_scale<T>(o, s, k, count)) break;
    for (size_t i = 0; i < count; ++i) o[i] = scale(s[i], k);
  })
}

namespace {
template <typename T>
typename std::enable_if<std::is_integral<T>::value>::type div_loop(T* p, size_t n, int d) {
  for (size_t i = 0; i < n; ++i) p[i] = div_trunc(p[i], d);
}
template <typename T>
typename std::enable_if<!std::is_integral<T>::value>::type div_loop(T*, size_t, int) {}
}  // namespace

void divide_trunc(void* buf, size_t count, int dt, int divisor) {
  HX_DISPATCH_DTYPE(dt, { div_loop(static_cast<T*>(buf), count, divisor); })
}

void store_scalar(double v, int dt, void* out) {
  const float f = static_cast<float>(v);
  switch (dt) {
    case hxcclFloat64: std::memcpy(out, &v, 8); break;
    case hxcclFloat32: std::memcpy(out, &f, 4); break;
    case hxcclFloat16: { f16 h; from_f32(f, &h); std::memcpy(out, &h, 2); } break;
    case hxcclBfloat16: { bf16 h; from_f32(f, &h); std::memcpy(out, &h, 2); } break;
    case hxcclFloat8e4m3: { e4m3 h; from_f32(f, &h); std::memcpy(out, &h, 1); } break;
    case hxcclFloat8e5m2: { e5m2 h; from_f32(f, &h); std::memcpy(out, &h, 1); } break;
    default: break;
  }
}

}  // namespace hx
