// Kernel entry points for one element type; included by one .cu file per type so the types
// compile in parallel.
#pragma once
#include "kernels/coll_body.cuh"
#include "kernels/roles_body.cuh"
#include "kernels/ring_body.cuh"
#include "kernels/ll_body.cuh"
#include "kernels/launch.h"

namespace hx {

template <typename T>
__global__ void __launch_bounds__(512) k_xchg_fold(const __grid_constant__ XchgArgs a) {
  __shared__ FoldShared sh;
  xchg_body<T, true>(a, blockIdx.x, gridDim.x, sh);
}
template <typename T>
__global__ void __launch_bounds__(512) k_xchg_fold_world(const XchgArgs* a) {
  __shared__ FoldShared sh;
  xchg_body<T, true>(a[blockIdx.y], blockIdx.x, gridDim.x, sh);
}
template <typename T>
__global__ void __launch_bounds__(512) k_twoshot(const __grid_constant__ TwoShotArgs a) {
  __shared__ FoldShared sh;
  twoshot_body<T>(a, blockIdx.x, gridDim.x, sh);
}
template <typename T>
__global__ void __launch_bounds__(512) k_twoshot_world(const TwoShotArgs* a) {
  __shared__ FoldShared sh;
  twoshot_body<T>(a[blockIdx.y], blockIdx.x, gridDim.x, sh);
}

// fp32 buffers, T on the wire (instantiated for fp16 and bf16 only)
template <typename T>
__global__ void __launch_bounds__(512) k_twoshot_cast(const __grid_constant__ TwoShotArgs a) {
  __shared__ FoldShared sh;
  twoshot_body<T, true>(a, blockIdx.x, gridDim.x, sh);
}
template <typename T>
__global__ void __launch_bounds__(512) k_twoshot_cast_world(const TwoShotArgs* a) {
  __shared__ FoldShared sh;
  twoshot_body<T, true>(a[blockIdx.y], blockIdx.x, gridDim.x, sh);
}

template <typename T>
__global__ void __launch_bounds__(512) k_twoshot_roles(const __grid_constant__ TwoShotArgs a) {
  __shared__ FoldShared sh;
  twoshot_roles_body<T>(a, blockIdx.x, gridDim.x, sh);
}
template <typename T>
__global__ void __launch_bounds__(512) k_twoshot_roles_world(const TwoShotArgs* a) {
  __shared__ FoldShared sh;
  twoshot_roles_body<T>(a[blockIdx.y], blockIdx.x, gridDim.x, sh);
}

template <typename T>
__global__ void __launch_bounds__(512) k_ring(const __grid_constant__ TwoShotArgs a) {
  __shared__ FoldShared sh;
  ring_body<T>(a, blockIdx.x, gridDim.x, sh);
}
template <typename T>
__global__ void __launch_bounds__(512) k_ring_world(const TwoShotArgs* a) {
  __shared__ FoldShared sh;
  ring_body<T>(a[blockIdx.y], blockIdx.x, gridDim.x, sh);
}

template <typename T>
__global__ void __launch_bounds__(256, 1) k_ll(const __grid_constant__ LLArgs a) {
  __shared__ FoldShared sh;
  ll_body<T>(a, blockIdx.x, gridDim.x, sh);
}
template <typename T>
__global__ void __launch_bounds__(256, 1) k_ll_world(const LLArgs* a) {
  __shared__ FoldShared sh;
  ll_body<T>(a[blockIdx.y], blockIdx.x, gridDim.x, sh);
}

template <typename Args>
cudaError_t launch_world(const void* kernel, const Args* dev_args, LaunchShape s, cudaStream_t st) {
  void* params[] = {const_cast<Args**>(&dev_args)};
  return cudaLaunchCooperativeKernel(kernel, dim3(s.ctas, s.world), dim3(s.threads), params, 0, st);
}

template <typename T>
cudaError_t launch_xchg_fold_t(const XchgArgs* args, LaunchShape s, cudaStream_t st) {
  if (s.world)
    return launch_world(reinterpret_cast<const void*>(&k_xchg_fold_world<T>), args, s, st);
  k_xchg_fold<T><<<s.ctas, s.threads, 0, st>>>(*args);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_twoshot_t(const TwoShotArgs* args, LaunchShape s, cudaStream_t st) {
  if (s.world)
    return launch_world(reinterpret_cast<const void*>(&k_twoshot_world<T>), args, s, st);
  k_twoshot<T><<<s.ctas, s.threads, 0, st>>>(*args);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_twoshot_cast_t(const TwoShotArgs* args, LaunchShape s, cudaStream_t st) {
  if (s.world)
    return launch_world(reinterpret_cast<const void*>(&k_twoshot_cast_world<T>), args, s, st);
  k_twoshot_cast<T><<<s.ctas, s.threads, 0, st>>>(*args);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_twoshot_roles_t(const TwoShotArgs* args, LaunchShape s, cudaStream_t st) {
  if (s.world)
    return launch_world(reinterpret_cast<const void*>(&k_twoshot_roles_world<T>), args, s, st);
  k_twoshot_roles<T><<<s.ctas, s.threads, 0, st>>>(*args);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_ring_t(const TwoShotArgs* args, LaunchShape s, cudaStream_t st) {
  if (s.world) return launch_world(reinterpret_cast<const void*>(&k_ring_world<T>), args, s, st);
  k_ring<T><<<s.ctas, s.threads, 0, st>>>(*args);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_ll_t(const LLArgs* args, LaunchShape s, cudaStream_t st) {
  if (s.world) return launch_world(reinterpret_cast<const void*>(&k_ll_world<T>), args, s, st);
  k_ll<T><<<s.ctas, s.threads, 0, st>>>(*args);
  return cudaGetLastError();
}

// ---- standalone elementwise kernels --------------------------------------------------------
template <typename T>
__global__ void k_reduce(T* dst, const T* src, size_t n, int op) {
  constexpr int V = 16 / sizeof(T);
  const size_t tid = blockIdx.x * size_t(blockDim.x) + threadIdx.x, nth = size_t(gridDim.x) * blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  const size_t nvec = aligned ? n / V : 0;
  for (size_t v = tid; v < nvec; v += nth) {
    Vec16<T> a, b;
    a.raw = ld16(reinterpret_cast<const char*>(dst) + (v << 4));
    b.raw = ld16(reinterpret_cast<const char*>(src) + (v << 4));
    st16(reinterpret_cast<char*>(dst) + (v << 4), apply_lanes(a, b, op).raw);
  }
  for (size_t e = nvec * V + tid; e < n; e += nth) dst[e] = apply(dst[e], src[e], op);
}
template <typename T>
__global__ void k_scale(T* dst, const T* src, size_t n, unsigned long long scalar_bits) {
  T k;
  memcpy(&k, &scalar_bits, sizeof(T));
  constexpr int V = 16 / sizeof(T);
  const size_t tid = blockIdx.x * size_t(blockDim.x) + threadIdx.x, nth = size_t(gridDim.x) * blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  const size_t nvec = aligned ? n / V : 0;
  for (size_t v = tid; v < nvec; v += nth) {
    Vec16<T> a;
    a.raw = ld16(reinterpret_cast<const char*>(src) + (v << 4));
    st16(reinterpret_cast<char*>(dst) + (v << 4), apply_lanes(a, splat(k), kProd).raw);
  }
  for (size_t e = nvec * V + tid; e < n; e += nth) dst[e] = scale(src[e], k);
}
template <typename T>
__global__ void k_divide(T* buf, size_t n, int divisor) {
  const size_t tid = blockIdx.x * size_t(blockDim.x) + threadIdx.x, nth = size_t(gridDim.x) * blockDim.x;
  for (size_t e = tid; e < n; e += nth) buf[e] = div_trunc(buf[e], divisor);
}

inline int elementwise_grid(size_t count, int per_thread) {
  size_t blocks = (count / per_thread + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;  // persistent-style: 16 CTAs per SM, grid-stride
  return static_cast<int>(blocks);
}
template <typename T>
cudaError_t launch_reduce_t(void* dst, const void* src, size_t count, int op, cudaStream_t st) {
  k_reduce<T><<<elementwise_grid(count, 16 / sizeof(T)), 256, 0, st>>>(
      static_cast<T*>(dst), static_cast<const T*>(src), count, op);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_scale_t(void* dst, const void* src, size_t count, unsigned long long bits,
                           cudaStream_t st) {
  k_scale<T><<<elementwise_grid(count, 16 / sizeof(T)), 256, 0, st>>>(
      static_cast<T*>(dst), static_cast<const T*>(src), count, bits);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_divide_t(void* buf, size_t count, int divisor, cudaStream_t st) {
  k_divide<T><<<elementwise_grid(count, 1), 256, 0, st>>>(static_cast<T*>(buf), count, divisor);
  return cudaGetLastError();
}

#define HX_INSTANTIATE_TYPE(T)                                                               \
  template cudaError_t launch_xchg_fold_t<T>(const XchgArgs*, LaunchShape, cudaStream_t);    \
  template cudaError_t launch_twoshot_t<T>(const TwoShotArgs*, LaunchShape, cudaStream_t);   \
  template cudaError_t launch_twoshot_roles_t<T>(const TwoShotArgs*, LaunchShape, cudaStream_t); \
  template cudaError_t launch_ring_t<T>(const TwoShotArgs*, LaunchShape, cudaStream_t);      \
  template cudaError_t launch_ll_t<T>(const LLArgs*, LaunchShape, cudaStream_t);             \
  template cudaError_t launch_reduce_t<T>(void*, const void*, size_t, int, cudaStream_t);    \
  template cudaError_t launch_scale_t<T>(void*, const void*, size_t, unsigned long long,     \
                                         cudaStream_t);                                      \
  template cudaError_t launch_divide_t<T>(void*, size_t, int, cudaStream_t);

}  // namespace hx
