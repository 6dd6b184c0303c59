// Large-message AllReduce as a three-role pipeline. The single-role kernels (coll_body.cuh,
// nvls_body.cuh) make every CTA walk through "stage in, combine, stage out" one after the
// other, so link-bound and memory-bound phases take turns. Here each lane of the message is
// served by three CTAs that run at the same time, one per role:
//
//   in   brings this rank's input to where the combiners read it
//        (two-shot: stores into the owners' windows; NVLS: copy into the own window)
//   mid  combines the slice this rank owns and publishes the result to every rank
//        (two-shot: ordered fold + peer/multicast stores; NVLS: multimem.ld_reduce + multimem.st)
//   out  copies the other owners' results from the own window to the output buffer
//
// Steps cycle through kRing staging buffers. Flags (one epoch per step, per lane and source
// rank, also signalled to the own rank so the roles of one rank see each other):
//   A(k)  "my step-k input is staged"        in  -> every rank's mid
//   B(k)  "I combined step k"                mid -> every rank's out, and every rank's in
//   C(k)  "I copied step k out"              out -> every rank's mid
// in(k) reuses the buffer of step k-kRing and waits for B(k-kRing) from all ranks; mid(k)
// overwrites result slots of step k-kRing and waits for C(k-kRing) from all ranks. The launch
// opens with a hand-shake among the in CTAs (no rank writes a window before every rank has
// left its previous launch) and closes when in has seen B(K-1) and mid has seen C(K-1) from
// all ranks, so the next launch finds every window idle. Epochs used: steps + 1.
#pragma once
#include "kernels/coll_body.cuh"
#include "kernels/nvls_body.cuh"

namespace hx {

__device__ inline void signal_everyone(const WinView& w, size_t flag_base, int lane, unsigned long long epoch) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < w.n) st_release_sys(flag_at(w.win[t], flag_base, lane, w.rank), epoch);
}
__device__ inline bool wait_everyone(const WinView& w, size_t flag_base, int lane, unsigned long long epoch,
                                     int* sh_fail) {
  const int t = threadIdx.x;
  if (t < w.n)
    if (!wait_flag(w, flag_at(w.win[w.rank], flag_base, lane, t), epoch, t)) *sh_fail = 1;
  __syncthreads();
  return *sh_fail == 0;
}

// Ops provides stage_in(k), combine(k), stage_out(k), each executed by all threads of a CTA.
template <typename Ops>
__device__ void roles_pipeline(Ops& ops, const WinView& w, unsigned long long epoch0, int steps, int lane,
                               int role, int* sh_fail) {
  if (threadIdx.x == 0) *sh_fail = 0;
  __syncthreads();
  const unsigned long long e1 = epoch0 + 1;  // epoch of step 0
  if (role == 0) {
    signal_everyone(w, kOffFlagsA, lane, epoch0);
    if (!wait_everyone(w, kOffFlagsA, lane, epoch0, sh_fail)) return;
    for (int k = 0; k < steps; ++k) {
      if (k >= kRing && !wait_everyone(w, kOffFlagsB, lane, e1 + k - kRing, sh_fail)) return;
      ops.stage_in(k);
      signal_everyone(w, kOffFlagsA, lane, e1 + k);
    }
    wait_everyone(w, kOffFlagsB, lane, e1 + steps - 1, sh_fail);
  } else if (role == 1) {
    for (int k = 0; k < steps; ++k) {
      if (!wait_everyone(w, kOffFlagsA, lane, e1 + k, sh_fail)) return;
      if (k >= kRing && !wait_everyone(w, kOffFlagsC, lane, e1 + k - kRing, sh_fail)) return;
      ops.combine(k);
      signal_everyone(w, kOffFlagsB, lane, e1 + k);
    }
    wait_everyone(w, kOffFlagsC, lane, e1 + steps - 1, sh_fail);
  } else {
    for (int k = 0; k < steps; ++k) {
      if (!wait_everyone(w, kOffFlagsB, lane, e1 + k, sh_fail)) return;
      ops.stage_out(k);
      signal_everyone(w, kOffFlagsC, lane, e1 + k);
    }
  }
}

// geometry shared by both variants: a step covers n slices of lanes * sub_bytes
struct RolesGeom {
  size_t slice, in_slice, buf_bytes, base0, second;
  __device__ RolesGeom(const WinView& w, int lanes, int lane, size_t sub) {
    slice = size_t(lanes) * sub;
    in_slice = size_t(lane) * sub;
    base0 = w.half_off[0];
    buf_bytes = (2 * w.half_bytes / kRing) & ~size_t(255);
    second = (buf_bytes / 2) & ~size_t(255);  // result slots live in the second half of a buffer
  }
  __device__ size_t buf(int step) const { return base0 + size_t(step % kRing) * buf_bytes; }
};

template <typename T>
struct TwoShotRoleOps {
  const TwoShotArgs& a;
  FoldShared& sh;
  RolesGeom g;
  T scalar;
  __device__ TwoShotRoleOps(const TwoShotArgs& args, FoldShared& s, int lanes, int lane)
      : a(args), sh(s), g(args.w, lanes, lane, args.sub_bytes), scalar{} {
    if (a.fold.premul) scalar = load_scalar<T>(a.fold);
  }
  __device__ void stage_in(int k) {
    const WinView& w = a.w;
    const size_t step0 = size_t(k) * w.n * g.slice, buf = g.buf(k);
    for (int jj = 1; jj < w.n; ++jj) {
      const int j = (w.rank + jj) % w.n;
      const size_t lo = step0 + size_t(j) * g.slice + g.in_slice;
      if (lo >= a.bytes) continue;
      const size_t len = min_sz(a.sub_bytes, a.bytes - lo);
      char* to = w.win[j] + buf + size_t(w.rank) * g.slice + g.in_slice;
      if (a.fold.premul)
        cta_scale_copy<T>(to, a.send + lo, len, scalar);
      else
        cta_copy(to, a.send + lo, len);
    }
  }
  __device__ void combine(int k) {
    const WinView& w = a.w;
    const int me = w.rank, n = w.n;
    const size_t step0 = size_t(k) * n * g.slice, buf = g.buf(k);
    const size_t lo = step0 + size_t(me) * g.slice + g.in_slice;
    __syncthreads();
    if (threadIdx.x < unsigned(n)) {
      const int i = threadIdx.x;
      sh.src[i] = i == me ? a.send + lo : w.win[me] + buf + size_t(i) * g.slice + g.in_slice;
      const int q = i < me ? i : i - 1;
      if (i != me) sh.remote[q] = w.win[i] + buf + g.second + size_t(me) * g.slice + g.in_slice;
    }
    if (threadIdx.x == 0)
      sh.mc_dst = a.use_mc ? w.mc + buf + g.second + size_t(me) * g.slice + g.in_slice : nullptr;
    __syncthreads();
    if (lo < a.bytes)
      cta_fold<T>(a.recv + lo, sh, n - 1, min_sz(a.sub_bytes, a.bytes - lo), lo / sizeof(T), a.fold, me, n, scalar);
  }
  __device__ void stage_out(int k) {
    const WinView& w = a.w;
    const size_t step0 = size_t(k) * w.n * g.slice, buf = g.buf(k);
    for (int ii = 1; ii < w.n; ++ii) {
      const int i = (w.rank + ii) % w.n;
      const size_t lo = step0 + size_t(i) * g.slice + g.in_slice;
      if (lo >= a.bytes) continue;
      cta_copy(a.recv + lo, w.win[w.rank] + buf + g.second + size_t(i) * g.slice + g.in_slice,
               min_sz(a.sub_bytes, a.bytes - lo));
    }
  }
};

template <typename T>
__device__ void twoshot_roles_body(const TwoShotArgs& a, int cta, int ncta, FoldShared& sh) {
  const int lanes = ncta / 3, lane = cta / 3, role = cta % 3;
  if (lane >= lanes) return;
  if (a.fold.kind == kFoldLinear && a.fold.ring) fill_ring_bounds(sh, a.fold.ring_count, a.w.n);
  TwoShotRoleOps<T> ops(a, sh, lanes, lane);
  roles_pipeline(ops, a.w, a.epoch0, a.steps, lane, role, &sh.fail);
}

template <typename T, int kMode>
struct NvlsRoleOps {
  const NvlsArgs& a;
  RolesGeom g;
  T scalar;
  __device__ NvlsRoleOps(const NvlsArgs& args, int lanes, int lane) : a(args), g(args.w, lanes, lane, args.sub_bytes), scalar{} {
    if (a.premul) {
      FoldSpec f{};
      f.scalar_bits = a.scalar_bits;
      f.scalar_ptr = a.scalar_ptr;
      scalar = load_scalar<T>(f);
    }
  }
  __device__ void stage_in(int k) {
    const WinView& w = a.w;
    const size_t step0 = size_t(k) * w.n * g.slice, buf = g.buf(k);
    for (int j = 0; j < w.n; ++j) {
      const size_t lo = step0 + size_t(j) * g.slice + g.in_slice;
      if (lo >= a.bytes) continue;
      const size_t len = min_sz(a.sub_bytes, a.bytes - lo);
      char* to = w.win[w.rank] + buf + size_t(j) * g.slice + g.in_slice;
      if (a.premul)
        cta_scale_copy<T>(to, a.send + lo, len, scalar);
      else
        cta_copy(to, a.send + lo, len);
    }
  }
  __device__ void combine(int k) {
    const WinView& w = a.w;
    const size_t step0 = size_t(k) * w.n * g.slice, buf = g.buf(k);
    const size_t lo = step0 + size_t(w.rank) * g.slice + g.in_slice;
    if (lo >= a.bytes) return;
    const size_t len = min_sz(a.sub_bytes, a.bytes - lo);
    const char* in = w.mc + buf + size_t(w.rank) * g.slice + g.in_slice;
    char* out = w.mc + buf + g.second + size_t(w.rank) * g.slice + g.in_slice;
    mm_reduce_range<T, kMode>(in, out, nullptr, len, a.postdiv);
  }
  __device__ void stage_out(int k) {  // every slice, the own one included (it came back through the switch)
    const WinView& w = a.w;
    const size_t step0 = size_t(k) * w.n * g.slice, buf = g.buf(k);
    for (int ii = 0; ii < w.n; ++ii) {
      const int i = (w.rank + ii) % w.n;
      const size_t lo = step0 + size_t(i) * g.slice + g.in_slice;
      if (lo >= a.bytes) continue;
      cta_copy(a.recv + lo, w.win[w.rank] + buf + g.second + size_t(i) * g.slice + g.in_slice,
               min_sz(a.sub_bytes, a.bytes - lo));
    }
  }
};

template <typename T, int kMode>
__device__ void nvls_roles_body(const NvlsArgs& a, int cta, int ncta, FoldShared& sh) {
  const int lanes = ncta / 3, lane = cta / 3, role = cta % 3;
  if (lane >= lanes) return;
  NvlsRoleOps<T, kMode> ops(a, lanes, lane);
  roles_pipeline(ops, a.w, a.epoch0, a.steps, lane, role, &sh.fail);
}

}  // namespace hx
