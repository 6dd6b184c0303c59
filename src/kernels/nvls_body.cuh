// AllReduce through NVSwitch multicast (NVLS). Each rank copies its input into its window,
// then reduces the slice it owns with multimem.ld_reduce (the switch fetches the slice from
// every GPU and combines it on the way) and publishes the result to every GPU with one
// multimem.st. The switch's combining order and precision are not specified, so for floating
// types this variant is offered only when bit-exactness is switched off (HXCCL_EXACT=0);
// integer sum/min/max are exact under any order and may use it always.
#pragma once
#include "hxccl.h"
#include "kernels/fold.cuh"
#include "device/nvls_modes.h"
#include "math/dtypes.h"

namespace hx {

#define HX_MM_V4(INSTR, p, v)                                                   \
  asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " {%0,%1,%2,%3}, [%4];" \
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)                     \
               : "l"(p)                                                          \
               : "memory")
#define HX_MM_S32(INSTR, p, v)                                                              \
  do {                                                                                       \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v.x) : "l"(p) : "memory");       \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v.y) : "l"(p + 4) : "memory");   \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v.z) : "l"(p + 8) : "memory");   \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=r"(v.w) : "l"(p + 12) : "memory");  \
  } while (0)
#define HX_MM_S64(INSTR, p, v)                                                              \
  do {                                                                                       \
    unsigned long long lo_, hi_;                                                             \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=l"(lo_) : "l"(p) : "memory");       \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " %0, [%1];" : "=l"(hi_) : "l"(p + 8) : "memory");   \
    v.x = unsigned(lo_); v.y = unsigned(lo_ >> 32); v.z = unsigned(hi_); v.w = unsigned(hi_ >> 32);                  \
  } while (0)

template <int kMode>
__device__ __forceinline__ uint4 mm_reduce16(const char* p) {
  uint4 v;
  if (kMode == kNvF32Add) HX_MM_V4("add.v4.f32", p, v);
  else if (kMode == kNvF64Add) HX_MM_S64("add.f64", p, v);
  else if (kMode == kNvF16Add) HX_MM_V4("add.acc::f32.v4.f16x2", p, v);
  else if (kMode == kNvF16Min) HX_MM_V4("min.v4.f16x2", p, v);
  else if (kMode == kNvF16Max) HX_MM_V4("max.v4.f16x2", p, v);
  else if (kMode == kNvBf16Add) HX_MM_V4("add.acc::f32.v4.bf16x2", p, v);
  else if (kMode == kNvBf16Min) HX_MM_V4("min.v4.bf16x2", p, v);
  else if (kMode == kNvBf16Max) HX_MM_V4("max.v4.bf16x2", p, v);
  else if (kMode == kNvS32Add) HX_MM_S32("add.u32", p, v);
  else if (kMode == kNvS32Min) HX_MM_S32("min.s32", p, v);
  else if (kMode == kNvS32Max) HX_MM_S32("max.s32", p, v);
  else if (kMode == kNvU32Min) HX_MM_S32("min.u32", p, v);
  else if (kMode == kNvU32Max) HX_MM_S32("max.u32", p, v);
  else if (kMode == kNvU64Add) HX_MM_S64("add.u64", p, v);
  else if (kMode == kNvS64Min) HX_MM_S64("min.s64", p, v);
  else if (kMode == kNvS64Max) HX_MM_S64("max.s64", p, v);
  else if (kMode == kNvU64Min) HX_MM_S64("min.u64", p, v);
  else if (kMode == kNvU64Max) HX_MM_S64("max.u64", p, v);
  else if (kMode == kNvE4m3Add) HX_MM_V4("add.acc::f16.v4.e4m3x4", p, v);
  else if (kMode == kNvE4m3Min) HX_MM_V4("min.v4.e4m3x4", p, v);
  else if (kMode == kNvE4m3Max) HX_MM_V4("max.v4.e4m3x4", p, v);
  else if (kMode == kNvE5m2Add) HX_MM_V4("add.acc::f16.v4.e5m2x4", p, v);
  else if (kMode == kNvE5m2Min) HX_MM_V4("min.v4.e5m2x4", p, v);
  else HX_MM_V4("max.v4.e5m2x4", p, v);
  return v;
}

// Reduces `len` bytes (a multiple of 16) at multicast address `in`, applies the integer
// post-divide, publishes the result at multicast address `out` and, when `direct` is set, also
// stores it at `direct`. Four reductions are in flight per thread: a multimem.ld_reduce is a
// round trip through the switch, far longer than a local load.
template <typename T, int kMode>
__device__ inline void mm_reduce_range(const char* in, char* out, char* direct, size_t len, int postdiv) {
  constexpr int V = 16 / sizeof(T);
  constexpr int U = 4;
  const size_t nvec = len >> 4, nt = blockDim.x;
  for (size_t v0 = threadIdx.x; v0 < nvec; v0 += nt * U) {
    Vec16<T> r[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (v0 + u * nt < nvec) r[u].raw = mm_reduce16<kMode>(in + ((v0 + u * nt) << 4));
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + u * nt;
      if (v >= nvec) continue;
      if (postdiv) {
#pragma unroll
        for (int l = 0; l < V; ++l) r[u].e[l] = div_trunc(r[u].e[l], postdiv);
      }
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(out + (v << 4)),
                   "r"(r[u].raw.x), "r"(r[u].raw.y), "r"(r[u].raw.z), "r"(r[u].raw.w)
                   : "memory");
      if (direct) st16(direct + (v << 4), r[u].raw);
    }
  }
}

template <typename T, int kMode>
__device__ void nvls_body(const NvlsArgs& a, int cta, int ncta, FoldShared& sh) {
  const WinView& w = a.w;
  const int me = w.rank, n = w.n;
  T scalar{};
  if (a.premul) {
    FoldSpec f{};
    f.scalar_bits = a.scalar_bits;
    f.scalar_ptr = a.scalar_ptr;
    scalar = load_scalar<T>(f);
  }
  if (threadIdx.x == 0) sh.fail = 0;
  __syncthreads();
  char* mine = w.win[me];
  const Staging stg(w, a.epoch0, a.steps);
  const bool multi = a.steps > 1;
  const unsigned long long e_step0 = multi ? a.epoch0 + 1 : a.epoch0;
  const size_t slice = size_t(ncta) * a.sub_bytes;
  const size_t out_base = (stg.buf_bytes / 2) & ~size_t(255);
  const size_t in_slice = size_t(cta) * a.sub_bytes;
  PhaseTimer tm(w, cta);

  auto copy_in = [&](int step) {  // my input, every slice's part of this CTA, into my own window
    const size_t step0 = size_t(step) * n * slice, buf = stg.at(step);
    for (int j = 0; j < n; ++j) {
      const size_t lo = step0 + size_t(j) * slice + in_slice;
      if (lo >= a.bytes) continue;
      const size_t len = min_sz(a.sub_bytes, a.bytes - lo);
      char* to = mine + buf + size_t(j) * slice + in_slice;
      if (a.premul)
        cta_scale_copy<T>(to, a.send + lo, len, scalar);
      else
        cta_copy(to, a.send + lo, len);
    }
    __syncthreads();
    tm.lap(kTrIn);
    signal_all(w, kOffFlagsA, cta, e_step0 + step);
    tm.lap(kTrSigA);
  };
  auto reduce = [&](int step) {  // my slice: the switch combines all ranks' copies
    const size_t step0 = size_t(step) * n * slice, buf = stg.at(step);
    const size_t lo = step0 + size_t(me) * slice + in_slice;
    if (lo < a.bytes) {
      const size_t len = min_sz(a.sub_bytes, a.bytes - lo);  // a multiple of 16 (the host checks)
      const char* in = w.mc + buf + size_t(me) * slice + in_slice;
      char* out = w.mc + buf + out_base + size_t(me) * slice + in_slice;
      const bool direct = (reinterpret_cast<uintptr_t>(a.recv + lo) & 15u) == 0;
      mm_reduce_range<T, kMode>(in, out, direct ? a.recv + lo : nullptr, len, a.postdiv);
    }
    __syncthreads();
    tm.lap(kTrMid);
    signal_all(w, kOffFlagsB, cta, e_step0 + step);
    tm.lap(kTrSigB);
  };
  auto copy_out = [&](int step) {
    const size_t step0 = size_t(step) * n * slice, buf = stg.at(step);
    for (int ii = 0; ii < n; ++ii) {
      const int i = (me + ii) % n;
      const size_t lo = step0 + size_t(i) * slice + in_slice;
      if (lo >= a.bytes) continue;
      if (i == me && (reinterpret_cast<uintptr_t>(a.recv + lo) & 15u) == 0) continue;  // stored directly
      cta_copy(a.recv + lo, mine + buf + out_base + size_t(i) * slice + in_slice,
               min_sz(a.sub_bytes, a.bytes - lo));
    }
    __syncthreads();
    tm.lap(kTrOut);
  };

  if (!multi) {
    copy_in(0);
    if (!wait_all(w, kOffFlagsA, cta, e_step0, &sh.fail)) return;
    tm.lap(kTrWaitA);
    reduce(0);
    if (!wait_all(w, kOffFlagsB, cta, e_step0, &sh.fail)) return;
    tm.lap(kTrWaitB);
    copy_out(0);
    tm.done();
    return;
  }
  // the same software pipeline as the two-shot kernel (see coll_body.cuh): copy_in(k+1)
  // overwrites the input slots of step k-3, which every rank finished reducing before its
  // B(k-3); reduce(k) overwrites result slots of step k-4, copied out before A(k-1)
  if (!signal_and_wait(w, kOffFlagsA, cta, a.epoch0, &sh.fail)) return;
  copy_in(0);
  for (int k = 0; k < a.steps; ++k) {
    if (k + 1 < a.steps) copy_in(k + 1);
    if (!wait_all(w, kOffFlagsA, cta, e_step0 + k, &sh.fail)) return;
    tm.lap(kTrWaitA);
    reduce(k);
    if (k > 0) {
      if (!wait_all(w, kOffFlagsB, cta, e_step0 + k - 1, &sh.fail)) return;
      tm.lap(kTrWaitB);
      copy_out(k - 1);
    }
  }
  if (!wait_all(w, kOffFlagsB, cta, e_step0 + a.steps - 1, &sh.fail)) return;
  tm.lap(kTrWaitB);
  copy_out(a.steps - 1);
  signal_and_wait(w, kOffFlagsA, cta, e_step0 + a.steps, &sh.fail);
  tm.lap(kTrWaitB);
  tm.done();
}

}  // namespace hx
