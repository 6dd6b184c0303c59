// Small-message AllReduce with the flag inside the data ("LL" lines). The ordinary one-shot
// kernel pushes a block, then raises a flag with st.release.sys, which cannot leave before
// every pushed byte was acknowledged by the peer: two link round trips before anything can be
// combined. Here every 16-byte store carries 8 bytes of payload and two copies of the launch's
// epoch, { data0, epoch, data1, epoch }: each 8-byte half validates itself, so the receiver
// simply polls the line until both epochs match and needs no flag, no fence and no CTA-wide
// barrier. The lines live in a region of the window of their own that only this kernel writes
// (anything else there could imitate an epoch): two halves chosen by the epoch's parity, each
// with one slot per source rank. Like every single-step launch it uses one epoch; a writer that
// reaches epoch e+2 has been through a launch in which it heard from the window's owner after
// that owner had finished reading epoch e (device/proto.h), so the halves need no hand-shake.
// The 32-bit epoch in a line wraps after 2^32 steps; the host clears the region and runs one
// ordinary launch whenever the upper half of the epoch changes (device/engine.cc), so a stale
// line never matches.
// With NVSwitch multicast a line reaches every peer with one multimem.st.
// This replaces the reference's recursive doubling for small messages (src/algo_rd.cc:7-37,
// src/select.h:10) and keeps its operand order: every rank folds all n contributions itself.
#pragma once
#include "kernels/fold.cuh"

namespace hx {

__device__ __forceinline__ uint4 ld16_volatile(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st16_volatile(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Polls one line until both halves carry `flag`. Bounded like wait_flag (prims.cuh).
__device__ inline bool ll_wait_line(const WinView& w, const char* line, unsigned flag, int peer, uint2* data) {
  uint4 v = ld16_volatile(line);
  if (v.y == flag && v.w == flag) {
    *data = make_uint2(v.x, v.z);
    return true;
  }
  const unsigned long long t0 = now_ns();
  const unsigned long long* abort_word = reinterpret_cast<const unsigned long long*>(w.win[w.rank] + kOffAbort);
  for (unsigned spins = 1;; ++spins) {
    v = ld16_volatile(line);
    if (v.y == flag && v.w == flag) {
      *data = make_uint2(v.x, v.z);
      return true;
    }
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

template <typename T, int N>
__device__ __forceinline__ T ll_fold_pow2(const uint2* data, int lane, int rank, int op) {
  T x[N];
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const unsigned long long bits = (static_cast<unsigned long long>(data[i].y) << 32) | data[i].x;
    T e[8 / sizeof(T)];
    memcpy(e, &bits, 8);
    x[i] = e[lane];
  }
  return fold_doubling_pow2<T, N>(x, rank, op);
}

// kN: the rank count when it is 2, 4 or 8 (loops unroll, every line lives in registers), else
// kMaxRanks with run-time bounds.
template <typename T, int kN>
__device__ void ll_ranks(const LLArgs& a, int cta, int ncta, FoldShared& sh) {
  constexpr int E = 8 / sizeof(T);  // elements of one line
  constexpr bool kFixed = kN != kMaxRanks;
  const WinView& w = a.w;
  const int me = w.rank, n = kFixed ? kN : w.n;
  const FoldSpec& f = a.fold;
  const unsigned flag = unsigned(a.epoch);
  const size_t slot = kLLBytes / 2 / size_t(n) / 256 * 256;  // ll_slot_bytes(n)
  const size_t half = kOffLL + size_t(a.epoch & 1) * slot * n;
  const size_t total = a.bytes / sizeof(T), nlines = (total + E - 1) / E;
  const T* in = reinterpret_cast<const T*>(a.send);
  T* out = reinterpret_cast<T*>(a.recv);
  T scalar{};
  if (f.premul) scalar = load_scalar<T>(f);
  if (f.kind == kFoldLinear && f.ring) {
    fill_ring_bounds(sh, f.ring_count, n);
    __syncthreads();
  }
  const size_t first = size_t(cta) * blockDim.x + threadIdx.x, stride = size_t(ncta) * blockDim.x;

  auto own_line = [&](size_t i) {  // this rank's (scaled) contribution to line i
    T e[E];
#pragma unroll
    for (int l = 0; l < E; ++l) {
      e[l] = T{};
      if (i * E + l < total) {
        e[l] = in[i * E + l];
        if (f.premul) e[l] = scale(e[l], scalar);
      }
    }
    unsigned long long bits;
    memcpy(&bits, e, 8);
    return make_uint2(unsigned(bits), unsigned(bits >> 32));
  };

  for (size_t i = first; i < nlines; i += stride) {
    const uint2 d = own_line(i);
    const uint4 line = make_uint4(d.x, flag, d.y, flag);
    const size_t off = half + size_t(me) * slot + (i << 4);
    if (a.use_mc) {
      mc_st16(w.mc + off, line);
    } else {
#pragma unroll
      for (int pp = 1; pp < kN; ++pp)
        if (pp < n) st16_volatile(w.win[(me + pp) % n] + off, line);
    }
  }
  // The lines of all sources are loaded together (their latencies overlap) and only those that
  // have not arrived yet are polled one by one.
  for (size_t i = first; i < nlines; i += stride) {
    uint2 data[kN];
    uint4 seen[kN];
    const char* mine = w.win[me] + half + (i << 4);
#pragma unroll
    for (int p = 0; p < kN; ++p)
      if (p < n && p != me) seen[p] = ld16_volatile(mine + size_t(p) * slot);
    const uint2 own = own_line(i);
#pragma unroll
    for (int p = 0; p < kN; ++p) {
      if (p >= n) continue;
      if (p == me)
        data[p] = own;
      else if (seen[p].y == flag && seen[p].w == flag)
        data[p] = make_uint2(seen[p].x, seen[p].z);
      else if (!ll_wait_line(w, mine + size_t(p) * slot, flag, p, &data[p]))
        return;
    }
#pragma unroll
    for (int l = 0; l < E; ++l) {
      if (i * E + l >= total) break;
      T r;
      if (kFixed && f.kind == kFoldDoubling) {
        r = ll_fold_pow2<T, kFixed ? kN : 2>(data, l, me, f.op);
      } else {
        T x[kN];
#pragma unroll
        for (int p = 0; p < kN; ++p) {
          if (p >= n) continue;
          const unsigned long long bits = (static_cast<unsigned long long>(data[p].y) << 32) | data[p].x;
          T e[E];
          memcpy(e, &bits, 8);
          x[p] = e[l];
        }
        const int b = (f.kind == kFoldLinear && f.ring) ? ring_block_of(sh, i * E + l, n) : 0;
        r = fold_one(x, n, me, f, b);
      }
      if (f.postdiv) r = div_trunc(r, f.postdiv);
      out[i * E + l] = r;
    }
  }
}

template <typename T>
__device__ void ll_body(const LLArgs& a, int cta, int ncta, FoldShared& sh) {
  switch (a.w.n) {
    case 2: ll_ranks<T, 2>(a, cta, ncta, sh); break;
    case 4: ll_ranks<T, 4>(a, cta, ncta, sh); break;
    case 8: ll_ranks<T, 8>(a, cta, ncta, sh); break;
    default: ll_ranks<T, kMaxRanks>(a, cta, ncta, sh); break;
  }
}

}  // namespace hx
