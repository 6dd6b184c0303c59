#include "reduce_host.h"

#include <cstring>

namespace hx {

void combine(void* out, const void* in_a, const void* in_b, size_t count, int dt, int op) {
  HX_DISPATCH_DTYPE(dt, {
    T* o = static_cast<T*>(out);
    const T* a = static_cast<const T*>(in_a);
    const T* b = static_cast<const T*>(in_b);
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
