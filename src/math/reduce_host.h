// Host-side elementwise loops over the shared element rules (elem.h). They are the CPU data
// path and the bit-exact oracle the device kernels are tested against.
// (Reference: src/reduce.h:6-19, src/reduce.cc:57-126.)
#pragma once
#include <cstddef>

#include "dtypes.h"

namespace hx {

// dst[i] = dst[i] (op) src[i]; op is one of kSum/kProd/kMax/kMin
void reduce_into(void* dst, const void* src, size_t count, int dt, int op);
// out[i] = in_a[i] (op) in_b[i] with in_a as the left operand; out may alias either input
void combine(void* out, const void* in_a, const void* in_b, size_t count, int dt, int op);
// dst[i] = src[i] * scalar (Prod rule, value on the left); dst may equal src
void scale_into(void* dst, const void* src, size_t count, int dt, const void* scalar);
// integer types only: buf[i] /= divisor in 64 bits, toward zero
void divide_trunc(void* buf, size_t count, int dt, int divisor);
// the scalar of a float Avg: v goes double -> float -> dt (fp64 keeps the double); no-op for
// integer types
void store_scalar(double v, int dt, void* out);

}  // namespace hx
