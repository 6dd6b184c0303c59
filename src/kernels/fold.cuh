// Combining the ranks' values in a prescribed order (device/proto.h: FoldSpec), fused with the
// pre-scale of the local input and the integer post-divide, so a reduction needs no separate
// scale, reduce or divide pass (the reference runs k_scale, k_reduce and k_div as separate
// kernels around its copies: src/gpu_reduce.cu:20-39, src/memops_device.cc:33-57).
#pragma once
#include "kernels/prims.cuh"

namespace hx {

template <typename T>
__device__ __forceinline__ T load_scalar(const FoldSpec& f) {
  T k;
  if (f.scalar_ptr) {
    k = *reinterpret_cast<const T*>(f.scalar_ptr);
  } else {
    const unsigned long long bits = f.scalar_bits;  // little endian: low bytes hold the value
    memcpy(&k, &bits, sizeof(T));
  }
  return k;
}

struct FoldShared {
  const char* src[kMaxRanks];       // per rank: where this CTA's part of its data starts
  char* remote[kMaxRanks];          // extra destinations of the result (peers' windows)
  char* mc_dst;                     // multicast alias of those destinations, or null
  unsigned long long bound[kMaxRanks + 1];  // ring-block boundaries, in elements
  int fail;
};

// ring-block boundaries of `count` elements over n ranks, once per kernel
__device__ inline void fill_ring_bounds(FoldShared& sh, size_t count, int n) {
  if (threadIdx.x <= unsigned(n)) {
    const int k = threadIdx.x;
    const size_t base = count / n, extra = count % n;
    sh.bound[k] = k == n ? count : size_t(k) * base + (size_t(k) < extra ? size_t(k) : extra);
  }
}
__device__ __forceinline__ int ring_block_of(const FoldShared& sh, unsigned long long e, int n) {
  int c = 0;
  for (int k = 1; k < n; ++k) c += (e >= sh.bound[k]) ? 1 : 0;
  return c;
}

// The order-defining part for one element. x[i] is rank i's (already scaled) value.
template <typename T>
__device__ inline T fold_one(const T* x, int n, int rank, const FoldSpec& f, int block) {
  const int op = f.op;
  if (f.kind == kFoldLinear) {
    int idx = (f.start + (f.ring ? block : 0)) % n;
    T acc = x[idx];
    for (int k = 1; k < n; ++k) {
      idx += f.dir;
      idx = idx >= n ? idx - n : (idx < 0 ? idx + n : idx);
      acc = apply(x[idx], acc, op);
    }
    return acc;
  }
  if (f.kind == kFoldDoubling) {
    int p = 1;
    while (2 * p <= n) p *= 2;
    const int spare = n - p;
    T lv[kMaxRanks];
    for (int q = 0; q < p; ++q)  // pairs first: the odd rank combines its own value with the even one's
      lv[q] = q < spare ? apply(x[2 * q + 1], x[2 * q], op) : x[q + spare];
    for (int bit = 1; bit < p; bit <<= 1) {
      T nx[kMaxRanks];
      for (int q = 0; q < p; ++q) nx[q] = apply(lv[q], lv[q ^ bit], op);
      for (int q = 0; q < p; ++q) lv[q] = nx[q];
    }
    const int mine = rank < 2 * spare ? rank / 2 : rank - spare;
    return lv[mine];
  }
  // binomial tree toward the root, in positions relative to it
  T acc[kMaxRanks];
  for (int v = n - 1; v >= 0; --v) {
    int real = v + f.root;
    real = real >= n ? real - n : real;
    T a = x[real];
    const int low = v == 0 ? n : (v & -v);  // children sit at v+1, v+2, v+4, ... below v's low bit
    for (int m = 1; m < low && v + m < n; m <<= 1) a = apply(a, acc[v + m], op);
    acc[v] = a;
  }
  return acc[0];
}

// One 16-byte vector through the general path: any fold kind, any rank count.
template <typename T>
__device__ inline void fold_vector_general(Vec16<T>& out, const FoldShared& sh, size_t v, size_t e_first,
                                           const FoldSpec& f, int rank, int n, T scalar) {
  constexpr int V = 16 / sizeof(T);
  Vec16<T> in[kMaxRanks];
  for (int i = 0; i < n; ++i) in[i].raw = ld16(sh.src[i] + (v << 4));
  for (int l = 0; l < V; ++l) {
    T x[kMaxRanks];
    for (int i = 0; i < n; ++i) x[i] = in[i].e[l];
    if (f.premul) x[rank] = scale(x[rank], scalar);
    const int b = (f.kind == kFoldLinear && f.ring) ? ring_block_of(sh, e_first + l, n) : 0;
    out.e[l] = fold_one(x, n, rank, f, b);
  }
}

template <typename T>
__device__ __forceinline__ void fold_store(char* dst, const FoldShared& sh, int nremote, size_t v,
                                           Vec16<T>& out, const FoldSpec& f) {
  constexpr int V = 16 / sizeof(T);
  if (f.postdiv) {
#pragma unroll
    for (int l = 0; l < V; ++l) out.e[l] = div_trunc(out.e[l], f.postdiv);
  }
  st16(dst + (v << 4), out.raw);
  if (sh.mc_dst) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(sh.mc_dst + (v << 4)),
                 "r"(out.raw.x), "r"(out.raw.y), "r"(out.raw.z), "r"(out.raw.w)
                 : "memory");
  } else {
    for (int r = 0; r < nremote; ++r) st16(sh.remote[r] + (v << 4), out.raw);
  }
}

// The streaming loop of the linear orders for N ranks known at compile time: U vectors per
// thread and iteration, all N * U loads issued before the first combine.
template <typename T, int N, int U>
__device__ inline void fold_linear_vectors(char* dst, const FoldShared& sh, int nremote, size_t nvec,
                                           size_t elem0, const FoldSpec& f, int rank, T scalar) {
  constexpr int V = 16 / sizeof(T);
  const size_t t = threadIdx.x, nt = blockDim.x;
  for (size_t v0 = t; v0 < nvec; v0 += nt * U) {
    Vec16<T> in[U][N];
    int first[U];
    bool general[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + u * nt;
      general[u] = false;
      first[u] = f.start;
      if (v >= nvec) continue;
      if (f.ring) {
        const size_t e_first = elem0 + v * V;
        const int block = ring_block_of(sh, e_first, N);
        general[u] = ring_block_of(sh, e_first + V - 1, N) != block;
        first[u] = (f.start + block) % N;
      }
      if (general[u]) continue;
      int idx = first[u];
#pragma unroll
      for (int k = 0; k < N; ++k) {
        in[u][k].raw = ld16(sh.src[idx] + (v << 4));
        idx += f.dir;
        idx = idx >= N ? idx - N : (idx < 0 ? idx + N : idx);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + u * nt;
      if (v >= nvec) continue;
      Vec16<T> out;
      if (general[u]) {  // the vector straddles two ring blocks: element by element
        fold_vector_general<T>(out, sh, v, elem0 + v * V, f, rank, N, scalar);
      } else {
        int idx = first[u];
#pragma unroll
        for (int k = 0; k < N; ++k) {
          if (f.premul && idx == rank) in[u][k] = apply_lanes(in[u][k], splat(scalar), kProd);
          out = k == 0 ? in[u][0] : apply_lanes(in[u][k], out, f.op);
          idx += f.dir;
          idx = idx >= N ? idx - N : (idx < 0 ? idx + N : idx);
        }
      }
      fold_store<T>(dst, sh, nremote, v, out, f);
    }
  }
}

// Recursive doubling over N = 2, 4 or 8 ranks (no spare ranks) with everything in registers:
// the butterfly keeps all N partial values per level because every rank combines with its own
// value on the left, so the values differ between ranks for non-commutative cases.
template <typename T, int N>
__device__ __forceinline__ T fold_doubling_pow2(const T (&x)[N], int rank, int op) {
  T lv[N];
#pragma unroll
  for (int q = 0; q < N; ++q) lv[q] = x[q];
#pragma unroll
  for (int bit = 1; bit < N; bit <<= 1) {
    T nx[N];
#pragma unroll
    for (int q = 0; q < N; ++q) nx[q] = apply(lv[q], lv[q ^ bit], op);
#pragma unroll
    for (int q = 0; q < N; ++q) lv[q] = nx[q];
  }
  T r = lv[0];
#pragma unroll
  for (int q = 1; q < N; ++q)
    if (q == rank) r = lv[q];
  return r;
}

// Element-per-thread loop for that order: small messages spread over many threads instead of
// 16-byte vectors walked lane by lane.
template <typename T, int N>
__device__ inline void fold_doubling_elems(char* dst, const FoldShared& sh, int nremote, size_t nbytes,
                                           const FoldSpec& f, int rank, T scalar) {
  const size_t total = nbytes / sizeof(T);
  for (size_t e = threadIdx.x; e < total; e += blockDim.x) {
    T x[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      x[i] = reinterpret_cast<const T*>(sh.src[i])[e];
      if (f.premul && i == rank) x[i] = scale(x[i], scalar);
    }
    T r = fold_doubling_pow2<T, N>(x, rank, f.op);
    if (f.postdiv) r = div_trunc(r, f.postdiv);
    reinterpret_cast<T*>(dst)[e] = r;
    for (int q = 0; q < nremote; ++q) reinterpret_cast<T*>(sh.remote[q])[e] = r;
  }
}

// Folds `nbytes` bytes (whole elements). sh.src[i] points at rank i's data for this range
// (sh.src[rank] is the unscaled local input), elem0 is the index of the first element in the
// full vector. The result goes to dst and to each of sh.remote[0..nremote); when sh.mc_dst is
// set, whole vectors reach the remote destinations through one multimem.st instead (tails
// still go peer by peer).
template <typename T>
__device__ inline void cta_fold(char* dst, FoldShared& sh, int nremote, size_t nbytes,
                                size_t elem0, const FoldSpec& f, int rank, int n, T scalar) {
  constexpr int V = 16 / sizeof(T);
  const int t = threadIdx.x, nt = blockDim.x;
  bool aligned = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
  for (int i = 0; i < n; ++i) aligned = aligned && (reinterpret_cast<uintptr_t>(sh.src[i]) & 15u) == 0;
  const size_t nvec = aligned ? nbytes >> 4 : 0;

  if (f.kind == kFoldDoubling && !sh.mc_dst && (n == 2 || n == 4 || n == 8)) {
    if (n == 2) fold_doubling_elems<T, 2>(dst, sh, nremote, nbytes, f, rank, scalar);
    else if (n == 4) fold_doubling_elems<T, 4>(dst, sh, nremote, nbytes, f, rank, scalar);
    else fold_doubling_elems<T, 8>(dst, sh, nremote, nbytes, f, rank, scalar);
    return;
  }
  if (f.kind == kFoldLinear && (n == 2 || n == 4 || n == 8)) {
    if (n == 2) fold_linear_vectors<T, 2, 4>(dst, sh, nremote, nvec, elem0, f, rank, scalar);
    else if (n == 4) fold_linear_vectors<T, 4, 2>(dst, sh, nremote, nvec, elem0, f, rank, scalar);
    else fold_linear_vectors<T, 8, 1>(dst, sh, nremote, nvec, elem0, f, rank, scalar);
  } else {
    for (size_t v = t; v < nvec; v += nt) {
      Vec16<T> out;
      fold_vector_general<T>(out, sh, v, elem0 + v * V, f, rank, n, scalar);
      fold_store<T>(dst, sh, nremote, v, out, f);
    }
  }

  // whatever the vector loop did not cover, element by element
  const size_t first = (nvec << 4) / sizeof(T), total = nbytes / sizeof(T);
  for (size_t e = first + t; e < total; e += nt) {
    T x[kMaxRanks];
    for (int i = 0; i < n; ++i) x[i] = reinterpret_cast<const T*>(sh.src[i])[e];
    if (f.premul) x[rank] = scale(x[rank], scalar);
    const int b = (f.kind == kFoldLinear && f.ring) ? ring_block_of(sh, elem0 + e, n) : 0;
    T r = fold_one(x, n, rank, f, b);
    if (f.postdiv) r = div_trunc(r, f.postdiv);
    reinterpret_cast<T*>(dst)[e] = r;
    for (int q = 0; q < nremote; ++q) reinterpret_cast<T*>(sh.remote[q])[e] = r;
  }
}

// dst = src * scalar, element-wise (pre-scaled pushes)
template <typename T>
__device__ inline void cta_scale_copy(char* dst, const char* src, size_t nbytes, T scalar) {
  constexpr int V = 16 / sizeof(T);
  const int t = threadIdx.x, nt = blockDim.x;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  const size_t nvec = aligned ? nbytes >> 4 : 0;
  for (size_t v = t; v < nvec; v += nt) {
    Vec16<T> x;
    x.raw = ld16(src + (v << 4));
    st16(dst + (v << 4), apply_lanes(x, splat(scalar), kProd).raw);
  }
  const size_t first = (nvec << 4) / sizeof(T), total = nbytes / sizeof(T);
  for (size_t e = first + t; e < total; e += nt)
    reinterpret_cast<T*>(dst)[e] = scale(reinterpret_cast<const T*>(src)[e], scalar);
}

// ---- fp32 buffers with a narrow type on the wire (gradient buckets) --------------------------------
// dst[i] = scale(narrow(src[i]), scalar): rounds fp32 values to T (nearest even, the library's
// overflow and NaN rules) and applies the pre-scale in T's rule, as a cast followed by the
// ordinary pre-scaled push would. `nbytes` counts bytes of T.
template <typename T>
__device__ inline void cta_narrow_scale_copy(char* dst, const float* src, size_t nbytes, T scalar, bool premul) {
  constexpr int V = 16 / sizeof(T);
  const int t = threadIdx.x, nt = blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  const size_t nvec = aligned ? nbytes >> 4 : 0;
  for (size_t v = t; v < nvec; v += nt) {
    Vec16<T> x;
    const float4* in = reinterpret_cast<const float4*>(src + v * V);
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const float4 f = in[q];
      from_f32(f.x, &x.e[4 * q]);
      from_f32(f.y, &x.e[4 * q + 1]);
      from_f32(f.z, &x.e[4 * q + 2]);
      from_f32(f.w, &x.e[4 * q + 3]);
    }
    if (premul) x = apply_lanes(x, splat(scalar), kProd);
    st16(dst + (v << 4), x.raw);
  }
  const size_t first = (nvec << 4) / sizeof(T), total = nbytes / sizeof(T);
  for (size_t e = first + t; e < total; e += nt) {
    T x;
    from_f32(src[e], &x);
    reinterpret_cast<T*>(dst)[e] = premul ? scale(x, scalar) : x;
  }
}
// dst[i] = float(src[i]) (exact). `nbytes` counts bytes of T.
template <typename T>
__device__ inline void cta_widen_copy(float* dst, const char* src, size_t nbytes) {
  constexpr int V = 16 / sizeof(T);
  const int t = threadIdx.x, nt = blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  const size_t nvec = aligned ? nbytes >> 4 : 0;
  for (size_t v = t; v < nvec; v += nt) {
    Vec16<T> x;
    x.raw = ld16(src + (v << 4));
    float4* out = reinterpret_cast<float4*>(dst + v * V);
#pragma unroll
    for (int q = 0; q < V / 4; ++q)
      out[q] = make_float4(to_f32(x.e[4 * q]), to_f32(x.e[4 * q + 1]), to_f32(x.e[4 * q + 2]), to_f32(x.e[4 * q + 3]));
  }
  const size_t first = (nvec << 4) / sizeof(T), total = nbytes / sizeof(T);
  for (size_t e = first + t; e < total; e += nt) dst[e] = to_f32(reinterpret_cast<const T*>(src)[e]);
}

}  // namespace hx
