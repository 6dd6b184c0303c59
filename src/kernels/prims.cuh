// Device-side building blocks: system-scope flag accesses, bounded waits, vector copies.
#pragma once
#include <cstdint>

#include "device/proto.h"
#include "math/elem.h"

namespace hx {

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned long long* flag_at(char* win, size_t base, int cta, int src) {
  return reinterpret_cast<unsigned long long*>(win + base) + size_t(cta) * kMaxRanks + src;
}

// Records a sticky failure and tells every peer to stop waiting.
__device__ inline void raise_failure(const WinView& w, unsigned code, unsigned long long detail) {
  const unsigned long long word = (static_cast<unsigned long long>(code) << 56) | (detail & 0xffffffffffffffull);
  atomicCAS(w.status, 0ull, word);
  for (int p = 0; p < w.n; ++p)
    if (p != w.rank)
      st_relaxed_sys(reinterpret_cast<unsigned long long*>(w.win[p] + kOffAbort), 1ull);
  __threadfence_system();
}

// Spins until *flag >= want. Gives up when the limit passes (timeout) or a peer raised this
// window's abort word (remote failure). Returns true on success.
__device__ inline bool wait_flag(const WinView& w, const unsigned long long* flag,
                                 unsigned long long want, int peer) {
  if (ld_acquire_sys(flag) >= want) return true;
  const unsigned long long t0 = now_ns();
  const unsigned long long* abort_word =
      reinterpret_cast<const unsigned long long*>(w.win[w.rank] + kOffAbort);
  for (unsigned spins = 1;; ++spins) {
    if (ld_acquire_sys(flag) >= want) return true;
    if ((spins & 63u) == 0) {
      if (ld_relaxed_sys(abort_word) != 0) {
        atomicCAS(w.status, 0ull, (static_cast<unsigned long long>(kStatRemote) << 56) | unsigned(peer));
        return false;
      }
      if (now_ns() - t0 > w.wait_ns) {
        raise_failure(w, kStatTimeout, unsigned(peer));
        return false;
      }
    }
  }
}

// Hand-over between ranks, called by every thread of the CTA. signal_all: threads 0..n-1 each
// tell one peer "my stores up to here are in your window" (the CTA's stores are fenced first).
// wait_all: the same threads wait for their peer's signal of `epoch`; false (to all threads)
// when any wait gave up.
__device__ inline void signal_all(const WinView& w, size_t flag_base, int cta, unsigned long long epoch) {
  __syncthreads();
  const int t = threadIdx.x;
  // st.release.sys orders the flag after every store the CTA made before the barrier above
  // (release is cumulative over what the barrier made visible to this thread); no separate
  // fence.sc is needed, and it is expensive at system scope
  if (t < w.n && t != w.rank) st_release_sys(flag_at(w.win[t], flag_base, cta, w.rank), epoch);
}
__device__ inline bool wait_all(const WinView& w, size_t flag_base, int cta, unsigned long long epoch,
                                int* sh_fail) {
  const int t = threadIdx.x;
  if (t < w.n && t != w.rank)
    if (!wait_flag(w, flag_at(w.win[w.rank], flag_base, cta, t), epoch, t)) *sh_fail = 1;
  __syncthreads();
  return *sh_fail == 0;
}
__device__ inline bool signal_and_wait(const WinView& w, size_t flag_base, int cta,
                                       unsigned long long epoch, int* sh_fail) {
  signal_all(w, flag_base, cta, epoch);
  return wait_all(w, flag_base, cta, epoch, sh_fail);
}

// Where step k of a launch stages its data. A single-step launch uses the half picked by its
// epoch's parity (see proto.h). A multi-step launch owns the whole staging area between its
// entry hand-shake and its closing one and cycles through kRing buffers, so that step k+1 can
// be pushed while step k is still being consumed.
constexpr int kRing = 4;
struct Staging {
  size_t base0, buf_bytes;
  int ring;
  __device__ Staging(const WinView& w, unsigned long long epoch0, int steps) {
    if (steps == 1) {
      base0 = w.half_off[epoch0 & 1];
      buf_bytes = w.half_bytes;
      ring = 1;
    } else {
      base0 = w.half_off[0];
      buf_bytes = (2 * w.half_bytes / kRing) & ~size_t(255);
      ring = kRing;
    }
  }
  __device__ size_t at(int step) const { return base0 + size_t(step % ring) * buf_bytes; }
};

// Phase timer of one CTA (see WinView::trace). lap(slot) adds the time since the previous lap.
struct PhaseTimer {
  unsigned long long* acc;
  unsigned long long last, first;
  __device__ PhaseTimer(const WinView& w, int cta) : acc(nullptr), last(0), first(0) {
    if (w.trace && threadIdx.x == 0) {
      acc = w.trace + size_t(cta) * kTraceSlots;
      last = first = now_ns();
    }
  }
  __device__ __forceinline__ void lap(int slot) {
    if (acc) {
      const unsigned long long t = now_ns();
      acc[slot] += t - last;
      last = t;
    }
  }
  __device__ __forceinline__ void done() {
    if (acc) acc[kTrAll] += now_ns() - first;
  }
};

// ---- bulk copies (all threads of the CTA take part) --------------------------------------------

__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
// streaming variants for data that is touched once
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// dst[0,n) = src[0,n); any alignment. The fast path needs both 16-byte aligned.
__device__ inline void cta_copy(char* dst, const char* src, size_t n) {
  const int t = threadIdx.x, nt = blockDim.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0) {
    const size_t nv = n >> 4;
    size_t i = t;
    for (; i + 7 * size_t(nt) < nv; i += 8 * size_t(nt)) {  // eight loads in flight per thread
      uint4 r[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) r[u] = ld16(src + ((i + u * size_t(nt)) << 4));
#pragma unroll
      for (int u = 0; u < 8; ++u) st16(dst + ((i + u * size_t(nt)) << 4), r[u]);
    }
    for (; i < nv; i += nt) st16(dst + (i << 4), ld16(src + (i << 4)));
    for (size_t k = (nv << 4) + t; k < n; k += nt) dst[k] = src[k];
    return;
  }
  for (size_t k = t; k < n; k += nt) dst[k] = src[k];
}

// 16 bytes of elements of type T
template <typename T>
union Vec16 {
  uint4 raw;
  T e[16 / sizeof(T)];
};

}  // namespace hx
