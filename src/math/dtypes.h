// Element-type table: sizes, classes, and a switch that turns a run-time hxcclDataType_t
// into a C++ type for templates. (Reference: src/reduce.cc:30-55.)
#pragma once
#include <cstddef>
#include <cstdint>

#include "elem.h"
#include "hxccl.h"

namespace hx {

HX_HD size_t dtype_size(int dt) {
  switch (dt) {
    case hxcclInt8: case hxcclUint8: case hxcclFloat8e4m3: case hxcclFloat8e5m2: return 1;
    case hxcclFloat16: case hxcclBfloat16: return 2;
    case hxcclInt32: case hxcclUint32: case hxcclFloat32: return 4;
    case hxcclInt64: case hxcclUint64: case hxcclFloat64: return 8;
    default: return 0;  // unknown
  }
}
HX_HD bool is_integer(int dt) { return dt >= hxcclInt8 && dt <= hxcclUint64; }
HX_HD bool is_builtin_op(int op) { return op >= hxcclSum && op <= hxcclMin; }

}  // namespace hx

// Runs `...` with `T` bound to the C++ element type of `dt`; unknown types run nothing.
#define HX_DTYPE_CASE(CODE, TYPE, ...) \
  case CODE: {                         \
    using T = TYPE;                    \
    __VA_ARGS__;                       \
  } break;
#define HX_DISPATCH_DTYPE(dt, ...)                           \
  switch (dt) {                                              \
    HX_DTYPE_CASE(hxcclInt8, int8_t, __VA_ARGS__)            \
    HX_DTYPE_CASE(hxcclUint8, uint8_t, __VA_ARGS__)          \
    HX_DTYPE_CASE(hxcclInt32, int32_t, __VA_ARGS__)          \
    HX_DTYPE_CASE(hxcclUint32, uint32_t, __VA_ARGS__)        \
    HX_DTYPE_CASE(hxcclInt64, int64_t, __VA_ARGS__)          \
    HX_DTYPE_CASE(hxcclUint64, uint64_t, __VA_ARGS__)        \
    HX_DTYPE_CASE(hxcclFloat16, hx::f16, __VA_ARGS__)        \
    HX_DTYPE_CASE(hxcclFloat32, float, __VA_ARGS__)          \
    HX_DTYPE_CASE(hxcclFloat64, double, __VA_ARGS__)         \
    HX_DTYPE_CASE(hxcclBfloat16, hx::bf16, __VA_ARGS__)      \
    HX_DTYPE_CASE(hxcclFloat8e4m3, hx::e4m3, __VA_ARGS__)    \
    HX_DTYPE_CASE(hxcclFloat8e5m2, hx::e5m2, __VA_ARGS__)    \
    default: break;                                          \
  }
