// Bodies of the collective kernels. Each body is written for "rank a.w.rank, CTA `cta` of
// `ncta`" so that the same code runs as one launch per GPU (production) or as one launch that
// carries every rank of a small world on a single GPU (blockIdx.y = rank), which is how the
// kernels are tested where only one GPU is at hand.
//
// Epochs of a launch: a single-step launch uses one epoch (its step). A multi-step launch
// uses steps + 2: an entry hand-shake (every rank is inside this launch, so every earlier
// launch on every rank is over and the whole staging area is free), one per step, and a
// closing hand-shake (every rank has finished reading its window, so whatever launch comes
// next may write at once). Between the two the steps are software-pipelined: a CTA pushes
// step k+1 before it consumes step k, so its waits are almost always already satisfied and
// link traffic overlaps the folding. With kRing = 4 buffers a writer reaches buffer k mod 4
// again only after it has seen a later signal of the owner that the owner sent after it had
// consumed step k (see the comments at each loop).
#pragma once
#include "kernels/fold.cuh"

namespace hx {

__device__ __forceinline__ size_t min_sz(size_t a, size_t b) { return a < b ? a : b; }

// ---- generic exchange --------------------------------------------------------------------------
// AllGather, AlltoAll(v), Broadcast, Gather, Scatter (copy mode); ReduceScatter, Reduce and the
// one-shot AllReduce (fold mode) are all "push blocks into peers' windows, hand over, take
// what arrived".
template <typename T, bool kFold>
__device__ void xchg_body(const XchgArgs& a, int cta, int ncta, FoldShared& sh) {
  const WinView& w = a.w;
  const int me = w.rank, n = w.n;
  T scalar{};
  if (kFold) {
    if (a.fold.premul) scalar = load_scalar<T>(a.fold);
    if (a.fold.kind == kFoldLinear && a.fold.ring) fill_ring_bounds(sh, a.fold.ring_count, n);
  }
  if (threadIdx.x == 0) sh.fail = 0;
  __syncthreads();
  char* mine = w.win[me];
  const Staging stg(w, a.epoch0, a.steps);
  const bool multi = a.steps > 1;
  const unsigned long long e_step0 = multi ? a.epoch0 + 1 : a.epoch0;
  const size_t in_slot = size_t(cta) * a.sub_bytes;
  PhaseTimer tm(w, cta);

  auto push = [&](int step) {
    const size_t lo = (size_t(step) * ncta + cta) * a.sub_bytes;  // offset inside a pair's block
    const size_t buf = stg.at(step);
    const size_t slot_off = buf + size_t(me) * a.slot_stride + in_slot;
    size_t by_mc = 0;  // bytes of this step's piece that went out through the switch's multicast
    if (!kFold && a.mc_bytes > lo)
      by_mc = cta_copy_multicast(w.mc + slot_off, a.mc_src + lo, min_sz(a.sub_bytes, a.mc_bytes - lo));
    for (int jj = 1; jj < n; ++jj) {
      const int j = (me + jj) % n;
      if (a.send_bytes[j] <= lo + by_mc) continue;
      const size_t len = min_sz(a.sub_bytes, a.send_bytes[j] - lo) - by_mc;
      char* to = w.win[j] + slot_off + by_mc;
      if (kFold && a.push_scaled)
        cta_scale_copy<T>(to, a.send_ptr[j] + lo, len, scalar);
      else
        cta_copy(to, a.send_ptr[j] + lo + by_mc, len);
    }
    __syncthreads();
    tm.lap(kTrIn);
    signal_all(w, kOffFlagsA, cta, e_step0 + step);
    tm.lap(kTrSigA);
  };
  auto consume = [&](int step) {
    const size_t lo = (size_t(step) * ncta + cta) * a.sub_bytes;
    const size_t buf = stg.at(step);
    if (!kFold) {
      for (int ii = 0; ii < n; ++ii) {
        const int i = (me + ii) % n;
        if (a.recv_bytes[i] <= lo) continue;
        const size_t len = min_sz(a.sub_bytes, a.recv_bytes[i] - lo);
        const char* from = i == me ? a.send_ptr[me] + lo : mine + buf + size_t(i) * a.slot_stride + in_slot;
        if (from != a.recv_ptr[i] + lo) cta_copy(a.recv_ptr[i] + lo, from, len);
      }
    } else if (a.fold_bytes > lo) {
      const size_t len = min_sz(a.sub_bytes, a.fold_bytes - lo);
      __syncthreads();  // the previous fold is done with sh.src
      if (threadIdx.x < unsigned(n)) {
        const int i = threadIdx.x;
        sh.src[i] = i == me ? a.own_ptr + lo : mine + buf + size_t(i) * a.slot_stride + in_slot;
      }
      if (threadIdx.x == 0) sh.mc_dst = nullptr;
      __syncthreads();
      cta_fold<T>(a.fold_dst + lo, sh, 0, len, a.fold_elem0 + lo / sizeof(T), a.fold, me, n, scalar);
    }
  };

  if (!multi) {
    push(0);
    if (!wait_all(w, kOffFlagsA, cta, e_step0, &sh.fail)) return;
    tm.lap(kTrWaitA);
    consume(0);
    __syncthreads();
    tm.lap(kTrOut);
    tm.done();
    return;
  }
  if (!signal_and_wait(w, kOffFlagsA, cta, a.epoch0, &sh.fail)) return;  // entry
  tm.lap(kTrWaitB);
  push(0);
  for (int k = 0; k < a.steps; ++k) {
    // push(k+1) reuses the buffer of step k-3. The owner consumed that step before it pushed
    // step k-1, and this CTA saw the owner's signal of step k-1 in the previous iteration.
    if (k + 1 < a.steps) push(k + 1);
    if (!wait_all(w, kOffFlagsA, cta, e_step0 + k, &sh.fail)) return;
    tm.lap(kTrWaitA);
    consume(k);
    __syncthreads();
    tm.lap(kTrOut);
  }
  signal_and_wait(w, kOffFlagsA, cta, e_step0 + a.steps, &sh.fail);  // closing
  tm.lap(kTrWaitB);
  tm.done();
}

// ---- two-shot AllReduce ------------------------------------------------------------------------
// Per step the message advances by n * ncta * sub_bytes. Slice j of a step belongs to rank j:
// everyone pushes its part of slice j into rank j's window (phase A), rank j folds the n
// contributions in the prescribed order and stores the result into its own output and into
// every peer's window (phase B), and everyone copies the other slices out of its window.
// A staging buffer holds the phase A slots in its first half and the phase B slots in its
// second half.
//
// kCast: the caller's buffers hold fp32 while T (fp16 or bf16) travels and is summed: a gradient
// bucket reduced in half the bytes without separate cast passes. a.bytes, the slices and all
// offsets count bytes of T; the fp32 buffers are indexed by element. The push rounds to T and
// pre-scales, and stages this rank's own contribution in its own window too, so that the fold
// reads n sources of T as always; the fold leaves the own slice's result in the window, and the
// gather widens every slice, the own one included, into the fp32 output. Bit for bit this is
// "cast to T, AllReduce in T, cast back".
template <typename T, bool kCast = false>
__device__ void twoshot_body(const TwoShotArgs& a, int cta, int ncta, FoldShared& sh) {
  const WinView& w = a.w;
  const int me = w.rank, n = w.n;
  T scalar{};
  if (a.fold.premul) scalar = load_scalar<T>(a.fold);
  if (a.fold.kind == kFoldLinear && a.fold.ring) fill_ring_bounds(sh, a.fold.ring_count, n);
  if (threadIdx.x == 0) sh.fail = 0;
  __syncthreads();
  char* mine = w.win[me];
  const Staging stg(w, a.epoch0, a.steps);
  const bool multi = a.steps > 1;
  const unsigned long long e_step0 = multi ? a.epoch0 + 1 : a.epoch0;
  const size_t slice = size_t(ncta) * a.sub_bytes;  // bytes of one slice per step
  const size_t ag_base = (stg.buf_bytes / 2) & ~size_t(255);
  const size_t in_slice = size_t(cta) * a.sub_bytes;
  PhaseTimer tm(w, cta);

  // In the pipelined loop the flag of push(k+1) is raised only after fold(k): the release has
  // to wait until the pushed bytes have landed on the peers, and that wait then overlaps the
  // fold instead of stalling the CTA twice per step.
  auto push = [&](int step, bool signal) {  // phase A: my contribution to every other owner's slice
    const size_t step0 = size_t(step) * n * slice, buf = stg.at(step);
    for (int jj = kCast ? 0 : 1; jj < n; ++jj) {
      const int j = (me + jj) % n;
      const size_t lo = step0 + size_t(j) * slice + in_slice;
      if (lo >= a.bytes) continue;
      const size_t len = min_sz(a.sub_bytes, a.bytes - lo);
      char* to = w.win[j] + buf + size_t(me) * slice + in_slice;
      if constexpr (kCast)
        cta_narrow_scale_copy<T>(to, reinterpret_cast<const float*>(a.send) + lo / sizeof(T), len, scalar,
                                 a.fold.premul != 0);
      else if (a.fold.premul)
        cta_scale_copy<T>(to, a.send + lo, len, scalar);
      else
        cta_copy(to, a.send + lo, len);
    }
    __syncthreads();
    tm.lap(kTrIn);
    if (signal) {
      signal_all(w, kOffFlagsA, cta, e_step0 + step);
      tm.lap(kTrSigA);
    }
  };
  auto fold = [&](int step, bool also_signal_next_push) {  // my slice: combine, keep, fan out
    const size_t step0 = size_t(step) * n * slice, buf = stg.at(step);
    const size_t lo = step0 + size_t(me) * slice + in_slice;
    __syncthreads();
    if (threadIdx.x < unsigned(n)) {
      const int i = threadIdx.x;
      sh.src[i] = (i == me && !kCast) ? a.send + lo : mine + buf + size_t(i) * slice + in_slice;
      const int q = i < me ? i : i - 1;  // compact list of the other ranks
      if (i != me) sh.remote[q] = w.win[i] + buf + ag_base + size_t(me) * slice + in_slice;
    }
    if (threadIdx.x == 0)
      sh.mc_dst = a.use_mc ? w.mc + buf + ag_base + size_t(me) * slice + in_slice : nullptr;
    __syncthreads();
    if (lo < a.bytes) {
      if (kCast) {  // every source is staged and already scaled; the result stays in the window
        FoldSpec plain = a.fold;
        plain.premul = 0;
        cta_fold<T>(mine + buf + ag_base + size_t(me) * slice + in_slice, sh, n - 1,
                    min_sz(a.sub_bytes, a.bytes - lo), lo / sizeof(T), plain, me, n, scalar);
      } else {
        cta_fold<T>(a.recv + lo, sh, n - 1, min_sz(a.sub_bytes, a.bytes - lo), lo / sizeof(T), a.fold,
                    me, n, scalar);
      }
    }
    __syncthreads();
    tm.lap(kTrMid);
    signal_all(w, kOffFlagsB, cta, e_step0 + step);
    if (also_signal_next_push) signal_all(w, kOffFlagsA, cta, e_step0 + step + 1);
    tm.lap(kTrSigB);
  };
  auto gather = [&](int step) {  // phase B: the other owners' results
    const size_t step0 = size_t(step) * n * slice, buf = stg.at(step);
    for (int ii = kCast ? 0 : 1; ii < n; ++ii) {
      const int i = (me + ii) % n;
      const size_t lo = step0 + size_t(i) * slice + in_slice;
      if (lo >= a.bytes) continue;
      const char* from = mine + buf + ag_base + size_t(i) * slice + in_slice;
      if constexpr (kCast)
        cta_widen_copy<T>(reinterpret_cast<float*>(a.recv) + lo / sizeof(T), from, min_sz(a.sub_bytes, a.bytes - lo));
      else
        cta_copy(a.recv + lo, from, min_sz(a.sub_bytes, a.bytes - lo));
    }
    __syncthreads();
    tm.lap(kTrOut);
  };

  if (!multi) {
    push(0, true);
    if (!wait_all(w, kOffFlagsA, cta, e_step0, &sh.fail)) return;
    tm.lap(kTrWaitA);
    fold(0, false);
    if (!wait_all(w, kOffFlagsB, cta, e_step0, &sh.fail)) return;
    tm.lap(kTrWaitB);
    gather(0);
    tm.done();
    return;
  }
  if (!signal_and_wait(w, kOffFlagsA, cta, a.epoch0, &sh.fail)) return;  // entry
  push(0, true);
  for (int k = 0; k < a.steps; ++k) {
    // push(k+1) overwrites phase A slots of step k-3: their owners folded that step before
    // they signalled B(k-3), which this CTA waited for two iterations ago.
    if (k + 1 < a.steps) push(k + 1, false);
    if (!wait_all(w, kOffFlagsA, cta, e_step0 + k, &sh.fail)) return;
    tm.lap(kTrWaitA);
    // fold(k) overwrites phase B slots of step k-4 on the peers: a peer copied those out
    // before it pushed step k-1 (signal A(k-1)), which is older than the A(k) just seen.
    fold(k, k + 1 < a.steps);
    if (k > 0) {
      if (!wait_all(w, kOffFlagsB, cta, e_step0 + k - 1, &sh.fail)) return;
      tm.lap(kTrWaitB);
      gather(k - 1);
    }
  }
  if (!wait_all(w, kOffFlagsB, cta, e_step0 + a.steps - 1, &sh.fail)) return;
  tm.lap(kTrWaitB);
  gather(a.steps - 1);
  signal_and_wait(w, kOffFlagsA, cta, e_step0 + a.steps, &sh.fail);  // closing
  tm.lap(kTrWaitB);
  tm.done();
}

}  // namespace hx
