// Bodies of the collective kernels. Each body is written for "rank a.w.rank, CTA `cta` of
// `ncta`" so that the same code runs as one launch per GPU (production) or as one launch that
// carries every rank of a small world on a single GPU (blockIdx.y = rank), which is how the
// kernels are tested where only one GPU is at hand.
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
  char* mine = w.win[me];
  for (int step = 0; step < a.steps; ++step) {
    const unsigned long long epoch = a.epoch0 + step;
    const size_t half = w.half_off[epoch & 1];
    const size_t lo = (size_t(step) * ncta + cta) * a.sub_bytes;  // offset inside a pair's block
    const size_t in_slot = size_t(cta) * a.sub_bytes;
    for (int jj = 1; jj < n; ++jj) {
      const int j = (me + jj) % n;
      if (a.send_bytes[j] <= lo) continue;
      const size_t len = min_sz(a.sub_bytes, a.send_bytes[j] - lo);
      char* to = w.win[j] + half + size_t(me) * a.slot_stride + in_slot;
      if (kFold && a.push_scaled)
        cta_scale_copy<T>(to, a.send_ptr[j] + lo, len, scalar);
      else
        cta_copy(to, a.send_ptr[j] + lo, len);
    }
    if (!signal_and_wait(w, kOffFlagsA, cta, epoch, &sh.fail)) return;
    if (!kFold) {
      for (int ii = 0; ii < n; ++ii) {
        const int i = (me + ii) % n;
        if (a.recv_bytes[i] <= lo) continue;
        const size_t len = min_sz(a.sub_bytes, a.recv_bytes[i] - lo);
        const char* from = i == me ? a.send_ptr[me] + lo
                                   : mine + half + size_t(i) * a.slot_stride + in_slot;
        if (from != a.recv_ptr[i] + lo) cta_copy(a.recv_ptr[i] + lo, from, len);
      }
    } else if (a.fold_bytes > lo) {
      const size_t len = min_sz(a.sub_bytes, a.fold_bytes - lo);
      if (threadIdx.x < unsigned(n)) {
        const int i = threadIdx.x;
        sh.src[i] = i == me ? a.own_ptr + lo : mine + half + size_t(i) * a.slot_stride + in_slot;
      }
      if (threadIdx.x == 0) sh.mc_dst = nullptr;
      __syncthreads();
      cta_fold<T>(a.fold_dst + lo, sh, 0, len, a.fold_elem0 + lo / sizeof(T), a.fold, me, n, scalar);
    }
  }
}

// ---- two-shot AllReduce ------------------------------------------------------------------------
// Per step the message advances by n * ncta * sub_bytes. Slice j of a step belongs to rank j:
// everyone pushes its part of slice j into rank j's window (phase A), rank j folds the n
// contributions in the prescribed order and stores the result into its own output and into
// every peer's window (phase B), and everyone copies the other slices out of its window.
template <typename T>
__device__ void twoshot_body(const TwoShotArgs& a, int cta, int ncta, FoldShared& sh) {
  const WinView& w = a.w;
  const int me = w.rank, n = w.n;
  T scalar{};
  if (a.fold.premul) scalar = load_scalar<T>(a.fold);
  if (a.fold.kind == kFoldLinear && a.fold.ring) fill_ring_bounds(sh, a.fold.ring_count, n);
  if (threadIdx.x == 0) sh.fail = 0;
  char* mine = w.win[me];
  const size_t slice = size_t(ncta) * a.sub_bytes;  // bytes of one slice per step
  const size_t ag_base = w.half_bytes / 2;          // second half of a staging half
  const size_t in_slice = size_t(cta) * a.sub_bytes;
  for (int step = 0; step < a.steps; ++step) {
    const unsigned long long epoch = a.epoch0 + step;
    const size_t half = w.half_off[epoch & 1];
    const size_t step0 = size_t(step) * n * slice;
    // phase A: my contribution to every other owner's slice
    for (int jj = 1; jj < n; ++jj) {
      const int j = (me + jj) % n;
      const size_t lo = step0 + size_t(j) * slice + in_slice;
      if (lo >= a.bytes) continue;
      const size_t len = min_sz(a.sub_bytes, a.bytes - lo);
      char* to = w.win[j] + half + size_t(me) * slice + in_slice;
      if (a.fold.premul)
        cta_scale_copy<T>(to, a.send + lo, len, scalar);
      else
        cta_copy(to, a.send + lo, len);
    }
    if (!signal_and_wait(w, kOffFlagsA, cta, epoch, &sh.fail)) return;
    // fold my slice; results fan out
    {
      const size_t lo = step0 + size_t(me) * slice + in_slice;
      if (threadIdx.x < unsigned(n)) {
        const int i = threadIdx.x;
        sh.src[i] = i == me ? a.send + lo : mine + half + size_t(i) * slice + in_slice;
        const int q = i < me ? i : i - 1;  // compact list of the other ranks
        if (i != me) sh.remote[q] = w.win[i] + half + ag_base + size_t(me) * slice + in_slice;
      }
      if (threadIdx.x == 0)
        sh.mc_dst = a.use_mc ? w.mc + half + ag_base + size_t(me) * slice + in_slice : nullptr;
      __syncthreads();
      if (lo < a.bytes)
        cta_fold<T>(a.recv + lo, sh, n - 1, min_sz(a.sub_bytes, a.bytes - lo), lo / sizeof(T),
                    a.fold, me, n, scalar);
    }
    if (!signal_and_wait(w, kOffFlagsB, cta, epoch, &sh.fail)) return;
    // phase B: the other owners' results
    for (int ii = 1; ii < n; ++ii) {
      const int i = (me + ii) % n;
      const size_t lo = step0 + size_t(i) * slice + in_slice;
      if (lo >= a.bytes) continue;
      cta_copy(a.recv + lo, mine + half + ag_base + size_t(i) * slice + in_slice,
               min_sz(a.sub_bytes, a.bytes - lo));
    }
  }
}

}  // namespace hx
