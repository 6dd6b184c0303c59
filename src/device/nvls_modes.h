// Which multimem.ld_reduce form serves an (element type, operator) pair. Host and device
// code share this table.
#pragma once
#include "hxccl.h"
#include "math/elem.h"

namespace hx {

enum NvlsMode : int {
  kNvF32Add, kNvF64Add,
  kNvF16Add, kNvF16Min, kNvF16Max,
  kNvBf16Add, kNvBf16Min, kNvBf16Max,
  kNvS32Add, kNvS32Min, kNvS32Max, kNvU32Min, kNvU32Max,
  kNvU64Add, kNvS64Min, kNvS64Max, kNvU64Min, kNvU64Max,
  kNvE4m3Add, kNvE4m3Min, kNvE4m3Max, kNvE5m2Add, kNvE5m2Min, kNvE5m2Max,
  kNvNone
};

// which multimem form serves (dtype, op), or kNvNone
inline int nvls_mode(int dt, int op) {
  const bool add = op == kSum, mn = op == kMin, mx = op == kMax;
  if (!add && !mn && !mx) return kNvNone;
  switch (dt) {
    case hxcclFloat32: return add ? kNvF32Add : kNvNone;
    case hxcclFloat64: return add ? kNvF64Add : kNvNone;
    case hxcclFloat16: return add ? kNvF16Add : mn ? kNvF16Min : kNvF16Max;
    case hxcclBfloat16: return add ? kNvBf16Add : mn ? kNvBf16Min : kNvBf16Max;
    case hxcclInt32: return add ? kNvS32Add : mn ? kNvS32Min : kNvS32Max;
    case hxcclUint32: return add ? kNvS32Add : mn ? kNvU32Min : kNvU32Max;
    case hxcclInt64: return add ? kNvU64Add : mn ? kNvS64Min : kNvS64Max;
    case hxcclUint64: return add ? kNvU64Add : mn ? kNvU64Min : kNvU64Max;
    case hxcclFloat8e4m3: return add ? kNvE4m3Add : mn ? kNvE4m3Min : kNvE4m3Max;
    case hxcclFloat8e5m2: return add ? kNvE5m2Add : mn ? kNvE5m2Min : kNvE5m2Max;
    default: return kNvNone;
  }
}


}  // namespace hx
