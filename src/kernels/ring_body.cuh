// AllReduce as a device-driven ring: reduce-scatter around the ring, then all-gather around
// it, with every hop a store into the right neighbour's window followed by a flag. A rank
// talks to two peers only, so this is the variant for a node without multicast or without
// all-to-all peer bandwidth, and the direct comparison for the two-shot kernel on two GPUs.
// It is also the one kernel whose data flow IS the reference's ring schedule
// (src/algo_ring.cc:12-39): block c starts at rank c and travels c+1, c+2, ..., each rank
// combining its own value as the left operand, so the ring order needs no replay logic.
// The reference tried this shape as an experiment with one CTA and unbounded spins
// (experimental/device_allreduce.cu:57-85); here every CTA runs its own ring over a sub-range
// of each block, waits are bounded, and scale / divide are folded into the hops.
//
// Blocks are the host path's: block b covers elements [bound[b], bound[b+1]) with the first
// count % n blocks one element longer. In round k CTA c handles bytes
// [(k * ncta + c) * sub, + sub) of every block (clipped to the block). One round is 2n-1
// hops at rank r; hop s concerns block (r - s) mod n:
//
//   s = 0            right.slot[0] = scale(own)
//   s = 1 .. n-2     right.slot[s] = apply(scale(own), mine.slot[s-1])
//   s = n-1          v = divide(apply(scale(own), mine.slot[n-2])); recv = v; right.slot[n-1] = v
//   s = n .. 2n-3    v = mine.slot[s-1]; recv = v; right.slot[s] = v
//   s = 2n-2         recv = mine.slot[2n-3]
//
// Every hop with a store to the right neighbour raises that neighbour's flag (row of this
// CTA, column of this rank) to the hop's epoch; every hop that reads a slot first waits for
// the left neighbour's flag. A slot is written once per round. The writer of slot s in round
// k+1 has by then received hop s-1 of round k+1 (or, for s = 0, the last hop of round k),
// which by the ring's chain of dependencies was sent only after the slot's owner had
// finished hop s+1 of round k, so no extra hand-shake is needed between rounds. The launch
// opens and closes with a hand-shake among all ranks like every multi-step launch
// (coll_body.cuh). Epochs used: rounds * (2n-2) + 2.
//
// ReduceScatter (ring_rs) is the first half alone with every chain shifted by one rank, which is
// the reference's ring_reducescatter schedule (src/algo_ring.cc:59-80): block b starts at rank
// b+1 and ends, complete, on rank b. Hop s at rank r concerns block (r - s - 1) mod n and a round
// has n hops (n-1 flags). Without the all-gather half the chain of dependencies around the ring
// is one hop too short to protect a slot from the next round's writer (it proves only that the
// slot's owner has finished hop s of the previous round, not hop s+1, which reads the slot), so
// the slots alternate between two sets by the round's parity: the writer of a slot in round k+2
// has seen, through that chain, every rank past hop s of round k+1, hence through with round k.
// Epochs used: rounds * (n-1) + 2.
#pragma once
#include "kernels/coll_body.cuh"

namespace hx {

template <typename T>
struct RingRule {
  int op;
  int premul;
  int postdiv;  // applied by the hop that completes a block
  T scalar;
};

// One hop's element work for `nbytes` bytes. kOwn: the local input takes part; kArr: the
// arrived partial result takes part. The value goes to d0 and d1 (either may be null).
template <typename T, bool kOwn, bool kArr>
__device__ inline void ring_pass(char* d0, char* d1, const char* own, const char* arr, size_t nbytes,
                                 const RingRule<T>& r, bool completes) {
  constexpr int V = 16 / sizeof(T);
  constexpr int U = 4;
  const int t = threadIdx.x, nt = blockDim.x;
  auto one = [&](T x_own, T x_arr) -> T {
    T v;
    if (kOwn) {
      v = r.premul ? scale(x_own, r.scalar) : x_own;
      if (kArr) v = apply(v, x_arr, r.op);
    } else {
      v = x_arr;
    }
    if (completes && r.postdiv) v = div_trunc(v, r.postdiv);
    return v;
  };
  auto lanes = [&](const Vec16<T>& x_own, const Vec16<T>& x_arr) -> Vec16<T> {  // `one` for 16 bytes
    Vec16<T> v;
    if (kOwn) {
      v = r.premul ? apply_lanes(x_own, splat(r.scalar), kProd) : x_own;
      if (kArr) v = apply_lanes(v, x_arr, r.op);
    } else {
      v = x_arr;
    }
    if (completes && r.postdiv) {
#pragma unroll
      for (int l = 0; l < V; ++l) v.e[l] = div_trunc(v.e[l], r.postdiv);
    }
    return v;
  };
  const uintptr_t bits = reinterpret_cast<uintptr_t>(d0) | reinterpret_cast<uintptr_t>(d1) |
                         (kOwn ? reinterpret_cast<uintptr_t>(own) : 0) |
                         (kArr ? reinterpret_cast<uintptr_t>(arr) : 0);
  const size_t nvec = (bits & 15u) == 0 ? nbytes >> 4 : 0;
  size_t i = t;
  for (; i + (U - 1) * size_t(nt) < nvec; i += U * size_t(nt)) {
    Vec16<T> a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t off = (i + u * size_t(nt)) << 4;
      if (kOwn) a[u].raw = ld16(own + off);
      if (kArr) b[u].raw = ld16(arr + off);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t off = (i + u * size_t(nt)) << 4;
      const Vec16<T> o = lanes(a[u], b[u]);
      if (d0) st16(d0 + off, o.raw);
      if (d1) st16(d1 + off, o.raw);
    }
  }
  for (; i < nvec; i += nt) {
    Vec16<T> a, b;
    if (kOwn) a.raw = ld16(own + (i << 4));
    if (kArr) b.raw = ld16(arr + (i << 4));
    const Vec16<T> o = lanes(a, b);
    if (d0) st16(d0 + (i << 4), o.raw);
    if (d1) st16(d1 + (i << 4), o.raw);
  }
  const size_t first = (nvec << 4) / sizeof(T), total = nbytes / sizeof(T);
  for (size_t e = first + t; e < total; e += nt) {
    const T v = one(kOwn ? reinterpret_cast<const T*>(own)[e] : T{}, kArr ? reinterpret_cast<const T*>(arr)[e] : T{});
    if (d0) reinterpret_cast<T*>(d0)[e] = v;
    if (d1) reinterpret_cast<T*>(d1)[e] = v;
  }
}

template <typename T>
__device__ void ring_body(const TwoShotArgs& a, int cta, int ncta, FoldShared& sh) {
  const WinView& w = a.w;
  const int me = w.rank, n = w.n;
  const int left = (me + n - 1) % n, right = (me + 1) % n;
  RingRule<T> rule{a.fold.op, a.fold.premul, a.fold.postdiv, T{}};
  if (a.fold.premul) rule.scalar = load_scalar<T>(a.fold);
  fill_ring_bounds(sh, a.fold.ring_count, n);
  if (threadIdx.x == 0) sh.fail = 0;
  __syncthreads();
  PhaseTimer tm(w, cta);
  if (!signal_and_wait(w, kOffFlagsA, cta, a.epoch0, &sh.fail)) return;  // entry
  tm.lap(kTrWaitB);

  const bool rs = a.ring_rs != 0;
  const int shift = rs ? 1 : 0;
  const int hops = rs ? n - 1 : 2 * n - 2;  // flags raised per round (and slots of one set)
  const size_t base = w.half_off[0];
  // ReduceScatter alternates between two slot sets by the round's parity (see the file comment)
  auto slot = [&](char* win, int k, int s) {
    return win + base + (size_t((rs ? (k & 1) : 0) * hops + s) * ncta + cta) * a.sub_bytes;
  };
  unsigned long long* to_right = flag_at(w.win[right], kOffFlagsA, cta, me);
  const unsigned long long* from_left = flag_at(w.win[me], kOffFlagsA, cta, left);
  char* mine = w.win[me];
  char* peer = w.win[right];

  // the element work of hop s of round k: no waiting, no flag
  auto hop = [&](int k, int s) {
    const size_t rel = (size_t(k) * ncta + cta) * a.sub_bytes;
    int b = (me - s - shift) % n;
    if (b < 0) b += n;
    const size_t blk0 = sh.bound[b] * sizeof(T), blk_bytes = (sh.bound[b + 1] - sh.bound[b]) * sizeof(T);
    const size_t len = rel < blk_bytes ? min_sz(a.sub_bytes, blk_bytes - rel) : 0;
    if (!len) return;
    const char* own = a.send + blk0 + rel;
    char* out = rs ? a.recv + rel : a.recv + blk0 + rel;
    if (s == 0)
      ring_pass<T, true, false>(slot(peer, k, 0), nullptr, own, nullptr, len, rule, false);
    else if (s < n - 1)
      ring_pass<T, true, true>(slot(peer, k, s), nullptr, own, slot(mine, k, s - 1), len, rule, false);
    else if (s == n - 1)
      ring_pass<T, true, true>(rs ? nullptr : slot(peer, k, s), out, own, slot(mine, k, s - 1), len, rule, true);
    else
      ring_pass<T, false, true>(s < hops ? slot(peer, k, s) : nullptr, out, nullptr, slot(mine, k, s - 1), len, rule, false);
  };
  auto epoch_of = [&](int k, int s) {
    return a.epoch0 + 1 + static_cast<unsigned long long>(k) * hops + static_cast<unsigned long long>(s);
  };
  auto raise = [&](int k, int s) {
    __syncthreads();  // the CTA's stores come before the flag (release is cumulative)
    if (threadIdx.x == 0) st_release_sys(to_right, epoch_of(k, s));
    tm.lap(kTrSigA);
  };

  // The first hop of a round only sends and the last one only receives. Run on their own they
  // leave one direction of the link idle for two hops out of 2n-1 (n+1 for ReduceScatter); so
  // the last hop of round k and the first hop of round k+1, which do not depend on each other,
  // share one step. The slot that first hop writes was consumed long before: the wait of this
  // step (for the left neighbour's last flag of round k) is the one the file comment's argument
  // for slot 0 rests on.
  hop(0, 0);
  tm.lap(kTrMid);
  raise(0, 0);
  for (int k = 0; k < a.steps; ++k) {
    for (int s = 1; s <= hops; ++s) {
      if (threadIdx.x == 0 && !wait_flag(w, from_left, epoch_of(k, s - 1), left)) sh.fail = 1;
      __syncthreads();
      if (sh.fail) return;
      tm.lap(kTrWaitA);
      hop(k, s);
      const bool next_first = s == hops && k + 1 < a.steps;
      if (next_first) hop(k + 1, 0);
      tm.lap(s < n ? kTrMid : kTrOut);
      if (s < hops)
        raise(k, s);
      else if (next_first)
        raise(k + 1, 0);
    }
  }
  signal_and_wait(w, kOffFlagsA, cta, a.epoch0 + 1 + static_cast<unsigned long long>(a.steps) * hops, &sh.fail);  // closing
  tm.lap(kTrWaitB);
  tm.done();
}

}  // namespace hx
