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

__device__ __forceinline__ void mc_st16(char* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// The same bytes to every rank at once: mc_dst is an address in the multicast alias of the
// windows. Whole 16-byte vectors only (both addresses 16-byte aligned); returns the bytes it
// covered, the caller sends the rest peer by peer.
__device__ inline size_t cta_copy_multicast(char* mc_dst, const char* src, size_t n) {
  const int t = threadIdx.x, nt = blockDim.x;
  const size_t nv = n >> 4;
  size_t i = t;
  for (; i + 3 * size_t(nt) < nv; i += 4 * size_t(nt)) {
    uint4 r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) r[u] = ld16(src + ((i + u * size_t(nt)) << 4));
#pragma unroll
    for (int u = 0; u < 4; ++u) mc_st16(mc_dst + ((i + u * size_t(nt)) << 4), r[u]);
  }
  for (; i < nv; i += nt) mc_st16(mc_dst + (i << 4), ld16(src + (i << 4)));
  return nv << 4;
}

// ---- bulk asynchronous copies (the TMA unit, untiled form) ------------------------------------------
// A copy whose source is this GPU's memory and whose destination is a peer's window can be
// driven by one thread: cp.async.bulk brings a chunk into shared memory (completion on an
// mbarrier), a second cp.async.bulk writes it to the destination, and several chunks are in
// flight at once. The copy unit issues large transactions on its own, so no warp spends
// instructions on moving bytes. Loads never use cluster multicast. Both addresses and the size
// must be multiples of 16 bytes (the caller checks). Every wait is bounded: when one runs out,
// the function stops issuing, waits for its stores in flight and returns false.
constexpr int kBulkStages = 4;
constexpr unsigned kBulkChunk = 32 * 1024;
constexpr size_t kBulkSmemBytes = size_t(kBulkStages) * kBulkChunk;
struct BulkPipe {
  unsigned char* buf;        // kBulkSmemBytes of shared memory, 128-byte aligned
  unsigned long long* bars;  // kBulkStages mbarriers, initialised once per kernel by bulk_pipe_init
  unsigned phase;            // bit s = parity the next wait on stage s expects (kept by the issuing thread)
};
__device__ __forceinline__ unsigned smem_addr(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
// all threads call; leaves with a barrier
__device__ inline void bulk_pipe_init(BulkPipe& pipe, unsigned char* buf, unsigned long long* bars) {
  pipe.buf = buf;
  pipe.bars = bars;
  pipe.phase = 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kBulkStages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars[s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
}
// Called by ONE thread. dst[0, n) = src[0, n).
__device__ inline bool bulk_copy_by_one_thread(BulkPipe& pipe, char* dst, const char* src, size_t n) {
  const size_t chunks = (n + kBulkChunk - 1) / kBulkChunk;
  auto chunk_len = [&](size_t c) { return unsigned(n - c * kBulkChunk < kBulkChunk ? n - c * kBulkChunk : kBulkChunk); };
  auto load = [&](size_t c) {
    const int s = int(c % kBulkStages);
    const unsigned len = chunk_len(c), bar = smem_addr(&pipe.bars[s]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(len) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(pipe.buf + size_t(s) * kBulkChunk)),
                 "l"(src + c * kBulkChunk), "r"(len), "r"(bar)
                 : "memory");
  };
  // loads run kBulkStages - 1 chunks ahead of the stores; a stage is loaded again only after the
  // store that read it has finished reading (wait_group.read keeps one store group outstanding)
  size_t issued = 0;
  for (; issued < chunks && issued < size_t(kBulkStages - 1); ++issued) load(issued);
  bool ok = true;
  for (size_t c = 0; c < chunks && ok; ++c) {
    const int s = int(c % kBulkStages);
    const unsigned bar = smem_addr(&pipe.bars[s]), parity = (pipe.phase >> s) & 1u;
    unsigned done = 0;
    for (unsigned spins = 0; !done; ++spins) {
      asm volatile(
          "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
          : "=r"(done)
          : "r"(bar), "r"(parity)
          : "memory");
      if (!done && spins > (1u << 22)) {  // far beyond any copy: give up
        ok = false;
        break;
      }
    }
    if (!ok) break;
    pipe.phase ^= 1u << s;
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + c * kBulkChunk),
                 "r"(smem_addr(pipe.buf + size_t(s) * kBulkChunk)), "r"(chunk_len(c))
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    if (issued < chunks) {
      // chunk `issued` reuses the stage of chunk issued - kBulkStages = c - 1, whose store is one group back
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      load(issued);
      ++issued;
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every store has been performed
  return ok;
}

// 16 bytes of elements of type T
template <typename T>
union Vec16 {
  uint4 raw;
  T e[16 / sizeof(T)];
};

// ---- a whole vector of elements through the element rule ------------------------------------------
// out.e[l] = apply(a.e[l], b.e[l], op) for every lane. The generic form is the lane loop; the
// fp8 types go two lanes at a time, because their hardware converters work on pairs
// (cvt...x2) and converting one value per instruction, as the scalar rule in math/fpconv.h does,
// leaves half of the converter's rate unused, which is what bounds an fp8 fold.
template <typename T>
__device__ __forceinline__ Vec16<T> apply_lanes(const Vec16<T>& a, const Vec16<T>& b, int op) {
  Vec16<T> out;
#pragma unroll
  for (int l = 0; l < int(16 / sizeof(T)); ++l) out.e[l] = apply(a.e[l], b.e[l], op);
  return out;
}

template <typename T>
__device__ __forceinline__ Vec16<T> splat(T k) {
  Vec16<T> v;
#pragma unroll
  for (int l = 0; l < int(16 / sizeof(T)); ++l) v.e[l] = k;
  return v;
}

__device__ __forceinline__ float2 f16x2_to_f32(unsigned pair) {
  float lo, hi;
  asm("cvt.f32.f16 %0, %1;" : "=f"(lo) : "h"(static_cast<unsigned short>(pair & 0xffffu)));
  asm("cvt.f32.f16 %0, %1;" : "=f"(hi) : "h"(static_cast<unsigned short>(pair >> 16)));
  return make_float2(lo, hi);
}
// two e4m3 codes (low byte = first element) -> two floats, exact
__device__ __forceinline__ float2 decode_pair(unsigned short codes, e4m3) {
  unsigned pair;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(codes));
  return f16x2_to_f32(pair);
}
// an e5m2 code is the upper byte of an fp16
__device__ __forceinline__ float2 decode_pair(unsigned short codes, e5m2) {
  return f16x2_to_f32(((unsigned(codes) & 0xff00u) << 16) | ((unsigned(codes) & 0xffu) << 8));
}
// two floats -> two codes under the library's rules (math/fpconv.h: hardware rounding, then the
// overflow and NaN codes patched in, per element exactly as from_f32 does)
__device__ __forceinline__ unsigned short encode_pair(float lo, float hi, e4m3) {
  unsigned short pair;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(hi), "f"(lo));
  const uint32_t ul = f32_bits(lo), al = ul & 0x7fffffffu, uh = f32_bits(hi), ah = uh & 0x7fffffffu;
  unsigned r0 = pair & 0xffu, r1 = pair >> 8;
  if (al > 0x43e80000u) r0 = al > 0x7f800000u ? 0x7fu : (((ul >> 24) & 0x80u) | 0x7fu);
  if (ah > 0x43e80000u) r1 = ah > 0x7f800000u ? 0x7fu : (((uh >> 24) & 0x80u) | 0x7fu);
  return static_cast<unsigned short>(r0 | (r1 << 8));
}
__device__ __forceinline__ unsigned short encode_pair(float lo, float hi, e5m2) {
  unsigned short pair;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(hi), "f"(lo));
  const uint32_t ul = f32_bits(lo), al = ul & 0x7fffffffu, uh = f32_bits(hi), ah = uh & 0x7fffffffu;
  unsigned r0 = pair & 0xffu, r1 = pair >> 8;
  if (al >= 0x47700000u) r0 = al > 0x7f800000u ? 0x7eu : (((ul >> 24) & 0x80u) | 0x7cu);
  if (ah >= 0x47700000u) r1 = ah > 0x7f800000u ? 0x7eu : (((uh >> 24) & 0x80u) | 0x7cu);
  return static_cast<unsigned short>(r0 | (r1 << 8));
}
template <typename F8>
__device__ __forceinline__ Vec16<F8> apply_lanes_fp8(const Vec16<F8>& a, const Vec16<F8>& b, int op) {
  Vec16<F8> out;
  const unsigned wa[4] = {a.raw.x, a.raw.y, a.raw.z, a.raw.w}, wb[4] = {b.raw.x, b.raw.y, b.raw.z, b.raw.w};
  unsigned wo[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    unsigned short half[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float2 x = decode_pair(static_cast<unsigned short>(wa[k] >> (16 * h)), F8{});
      const float2 y = decode_pair(static_cast<unsigned short>(wb[k] >> (16 * h)), F8{});
      half[h] = encode_pair(narrow_combine(x.x, y.x, op), narrow_combine(x.y, y.y, op), F8{});
    }
    wo[k] = unsigned(half[0]) | (unsigned(half[1]) << 16);
  }
  out.raw = make_uint4(wo[0], wo[1], wo[2], wo[3]);
  return out;
}
template <>
__device__ __forceinline__ Vec16<e4m3> apply_lanes<e4m3>(const Vec16<e4m3>& a, const Vec16<e4m3>& b, int op) {
  return apply_lanes_fp8<e4m3>(a, b, op);
}
template <>
__device__ __forceinline__ Vec16<e5m2> apply_lanes<e5m2>(const Vec16<e5m2>& a, const Vec16<e5m2>& b, int op) {
  return apply_lanes_fp8<e5m2>(a, b, op);
}

}  // namespace hx
