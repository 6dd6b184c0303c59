// Narrow floating-point formats: fp16, bf16, fp8 e4m3fn and fp8 e5m2, converted to and from
// fp32. The reference implementation (NarrowFmt) uses integer bit operations only and runs on
// host and device alike; the device entry points (to_f32 / from_f32) take the hardware
// converters where they exist and patch the cases in which hardware and rules differ, and are
// checked against NarrowFmt for every input on the GPU.
//
// Rules (they are the reference's, src/fp.h:12-59, stated here as a specification):
//   * decode is exact; an IEEE-style format (fp16, bf16, e5m2) has inf and NaN in its all-ones
//     exponent, e4m3fn has only the single NaN code S.1111.111 and no inf;
//   * encode rounds to nearest, ties to even, also into the subnormal range;
//   * a value that rounds above the largest finite number becomes +-inf for the IEEE-style
//     formats and the NaN code with the value's sign (0x7f / 0xff) for e4m3fn;
//   * a NaN encodes to one canonical code without sign: fp16 0x7e00, bf16 0x7fc0, e4m3fn 0x7f,
//     e5m2 0x7e.
#pragma once
#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define HX_HD __host__ __device__ __forceinline__
#else
#define HX_HD inline
#endif

namespace hx {

HX_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
#endif
}
HX_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  std::memcpy(&f, &u, 4);
  return f;
#endif
}

// Format description: E exponent bits, M mantissa bits, IEEE = has inf/NaN exponent.
template <int E, int M, bool IEEE>
struct NarrowFmt {
  static constexpr int kBias = (1 << (E - 1)) - 1;
  static constexpr int kEmin = 1 - kBias;  // exponent of the smallest normal
  static constexpr uint32_t kExpMask = (1u << E) - 1;
  static constexpr uint32_t kManMask = (1u << M) - 1;
  static constexpr uint32_t kSign = 1u << (E + M);
  static constexpr uint32_t kNan =
      IEEE ? ((kExpMask << M) | (1u << (M - 1))) : ((kExpMask << M) | kManMask);
  static constexpr uint32_t kOverflow = IEEE ? (kExpMask << M) : kNan;  // magnitude code
  static constexpr uint32_t kMaxFinite =
      IEEE ? (((kExpMask - 1) << M) | kManMask) : ((kExpMask << M) | (kManMask - 1));

  HX_HD static float decode(uint32_t v) {
    const uint32_t e = (v >> M) & kExpMask, m = v & kManMask;
    const uint32_t s = (v & kSign) ? 0x80000000u : 0u;
    if (IEEE && e == kExpMask) return bits_f32(m ? 0x7fc00000u : (s | 0x7f800000u));
    if (!IEEE && e == kExpMask && m == kManMask) return bits_f32(0x7fc00000u);
    if (e == 0) {
      // a format with fp32's exponent range (bf16) has fp32's subnormals: only the width differs
      if (kBias == 127) return bits_f32(s | (m << (23 - M)));
      // subnormal: m * 2^(kEmin - M), exact in fp32 for every other format here
      const float scale = bits_f32(static_cast<uint32_t>(kEmin - M + 127) << 23);
      const float mag = static_cast<float>(m) * scale;
      return bits_f32(f32_bits(mag) | s);
    }
    return bits_f32(s | ((e + 127u - kBias) << 23) | (m << (23 - M)));
  }

  HX_HD static uint32_t encode(float x) {
    const uint32_t u = f32_bits(x);
    const uint32_t s = (u >> 31) ? kSign : 0u;
    const uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return kNan;
    if (a == 0x7f800000u) return s | kOverflow;
    int e;
    uint32_t mant;  // value = mant * 2^(e - 23)
    if ((a >> 23) == 0) {
      e = -126;
      mant = a;
    } else {
      e = static_cast<int>(a >> 23) - 127;
      mant = (a & 0x7fffffu) | 0x800000u;
    }
    int drop = 23 - M;               // low bits that do not fit a normal result
    if (e < kEmin) drop += kEmin - e;  // the subnormal grid is coarser
    uint32_t q = 0;
    if (drop < 25) {                   // otherwise the value is below a quarter of one step
      q = mant >> drop;
      const uint32_t rest = mant & ((1u << drop) - 1), half = 1u << (drop - 1);
      if (rest > half || (rest == half && (q & 1u))) ++q;
    }
    // A normal q is in [2^M, 2^(M+1)]; adding it to (exponent-1) << M lets a rounding carry
    // run into the exponent field. A subnormal q is the code itself.
    const uint32_t code = e >= kEmin ? (static_cast<uint32_t>(e + kBias - 1) << M) + q : q;
    if (code > kMaxFinite) return s | kOverflow;
    return s | code;
  }
};

using FmtF16 = NarrowFmt<5, 10, true>;
using FmtE4M3 = NarrowFmt<4, 3, false>;
using FmtE5M2 = NarrowFmt<5, 2, true>;

// Storage wrappers, so that templates can tell the 12 element types apart by C++ type.
struct f16 { uint16_t b; };
struct bf16 { uint16_t b; };
struct e4m3 { uint8_t b; };
struct e5m2 { uint8_t b; };

HX_HD float to_f32(f16 v) {
#if defined(__CUDA_ARCH__)
  float f;  // exact in hardware
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(v.b));
  // the all-ones exponent with a payload decodes to the canonical NaN like the software path;
  // only NaN-ness is observable after re-encoding, so the payload is left alone
  return f;
#else
  return FmtF16::decode(v.b);
#endif
}
HX_HD float to_f32(bf16 v) { return bits_f32(static_cast<uint32_t>(v.b) << 16); }
HX_HD float to_f32(e4m3 v) {
#if defined(__CUDA_ARCH__)
  // hardware decode of a pair (exact); the low byte lands in the low half
  unsigned int pair;
  float f;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(static_cast<unsigned short>(v.b)));
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(static_cast<unsigned short>(pair & 0xffffu)));
  return f;
#else
  return FmtE4M3::decode(v.b);
#endif
}
HX_HD float to_f32(e5m2 v) {
#if defined(__CUDA_ARCH__)
  float f;  // e5m2 is the upper byte of an fp16
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(static_cast<unsigned short>(v.b << 8)));
  return f;
#else
  return FmtE5M2::decode(v.b);
#endif
}

HX_HD void from_f32(float x, f16* out) {
#if defined(__CUDA_ARCH__)
  // cvt.rn.f16.f32 rounds to nearest even, overflows to inf and handles subnormals; only the
  // NaN code differs (hardware 0x7fff), so NaN is fixed up
  uint16_t h;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(x));
  out->b = (x != x) ? static_cast<uint16_t>(0x7e00) : h;
#else
  out->b = static_cast<uint16_t>(FmtF16::encode(x));
#endif
}
HX_HD void from_f32(float x, bf16* out) {
  const uint32_t u = f32_bits(x);
  if ((u & 0x7fffffffu) > 0x7f800000u) {
    out->b = 0x7fc0;
    return;
  }
  // same exponent range as fp32: rounding the low 16 bits away carries correctly into the
  // exponent, up to and including inf
  out->b = static_cast<uint16_t>((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
// On the device the fp8 encoders use the hardware converter, which rounds to nearest even
// (subnormals included) but saturates at the largest finite value; the library's rule for
// values that round past it (NaN with the sign for e4m3fn, infinity for e5m2) and its
// canonical NaN codes are patched in. 464 is the tie that still rounds down to 448;
// 61440 is the tie that rounds up past 57344. Checked against the software encoder for all
// 2^32 inputs by tests/test_device_math_gpu.py.
HX_HD void from_f32(float x, e4m3* out) {
#if defined(__CUDA_ARCH__)
  unsigned short pair;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(x));
  const uint32_t u = f32_bits(x), a = u & 0x7fffffffu;
  uint8_t r = static_cast<uint8_t>(pair & 0xffu);
  if (a > 0x43e80000u) r = a > 0x7f800000u ? 0x7f : static_cast<uint8_t>(((u >> 24) & 0x80u) | 0x7fu);
  out->b = r;
#else
  out->b = static_cast<uint8_t>(FmtE4M3::encode(x));
#endif
}
HX_HD void from_f32(float x, e5m2* out) {
#if defined(__CUDA_ARCH__)
  unsigned short pair;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(x));
  const uint32_t u = f32_bits(x), a = u & 0x7fffffffu;
  uint8_t r = static_cast<uint8_t>(pair & 0xffu);
  if (a >= 0x47700000u) r = a > 0x7f800000u ? 0x7e : static_cast<uint8_t>(((u >> 24) & 0x80u) | 0x7cu);
  out->b = r;
#else
  out->b = static_cast<uint8_t>(FmtE5M2::encode(x));
#endif
}

}  // namespace hx
