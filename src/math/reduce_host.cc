#include "reduce_host.h"

#include <cstring>

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
template <typename T>
bool fast_arith(T*, const T*, const T*, size_t, int) { return false; }
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
