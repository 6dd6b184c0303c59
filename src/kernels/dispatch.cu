// Type-independent kernels (byte exchange, Send/Recv lanes, NVLS) and the run-time dispatch
// from hxcclDataType_t to the per-type launchers.
#include <algorithm>

#include "kernels/inst.cuh"
#include "kernels/nvls_body.cuh"
#include "kernels/p2p_body.cuh"
#include "math/dtypes.h"

namespace hx {

__global__ void __launch_bounds__(512) k_xchg_copy(const __grid_constant__ XchgArgs a) {
  __shared__ FoldShared sh;
  xchg_body<uint8_t, false>(a, blockIdx.x, gridDim.x, sh);
}
__global__ void __launch_bounds__(512) k_xchg_copy_world(const XchgArgs* a) {
  __shared__ FoldShared sh;
  xchg_body<uint8_t, false>(a[blockIdx.y], blockIdx.x, gridDim.x, sh);
}
// CTA (lane, group): the group's workers one after the other (see P2pArgs::workers_per_cta)
__device__ inline void p2p_cta(const P2pArgs& a, int* fail, unsigned long long* word, BulkPipe* pipe = nullptr) {
  const int wpc = a.workers_per_cta, groups = kP2pWorkers / wpc;
  const int lane = blockIdx.x / groups, first = (blockIdx.x % groups) * wpc;
  if (lane >= a.nlanes) return;
  for (int k = 0; k < wpc; ++k) {
    if (!p2p_body(a, lane, first + k, fail, word, pipe)) return;
    __syncthreads();
  }
}
__global__ void __launch_bounds__(512) k_p2p(const __grid_constant__ P2pArgs a) {
  __shared__ int fail;
  __shared__ unsigned long long word;
  p2p_cta(a, &fail, &word);
}
// The same with the senders' pieces moved by bulk asynchronous copies through kBulkSmemBytes of
// dynamic shared memory (production form only).
__global__ void __launch_bounds__(512) k_p2p_bulk(const __grid_constant__ P2pArgs a) {
  extern __shared__ __align__(128) unsigned char staging[];
  __shared__ __align__(8) unsigned long long bars[kBulkStages];
  __shared__ int fail;
  __shared__ unsigned long long word;
  BulkPipe pipe;
  bulk_pipe_init(pipe, staging, bars);
  p2p_cta(a, &fail, &word, &pipe);
}
__global__ void __launch_bounds__(512) k_p2p_world(const P2pArgs* a) {
  __shared__ int fail;
  __shared__ unsigned long long word;
  p2p_cta(a[blockIdx.y], &fail, &word);
}
template <typename T, int kMode>
__global__ void __launch_bounds__(512) k_nvls(const __grid_constant__ NvlsArgs a) {
  __shared__ FoldShared sh;
  nvls_body<T, kMode>(a, blockIdx.x, gridDim.x, sh);
}
template <typename T, int kMode>
__global__ void __launch_bounds__(512) k_nvls_roles(const __grid_constant__ NvlsArgs a) {
  __shared__ FoldShared sh;
  nvls_roles_body<T, kMode>(a, blockIdx.x, gridDim.x, sh);
}

// ---- local copy (single-rank collectives, a rank's Send to itself) -------------------------------
// The general form: every CTA copies one contiguous share, any alignment.
__global__ void __launch_bounds__(512) k_copy(char* dst, const char* src, size_t bytes, size_t share) {
  const size_t lo = size_t(blockIdx.x) * share;
  if (lo < bytes) cta_copy(dst + lo, src + lo, min_sz(share, bytes - lo));
}
// The streaming form for 16-byte aligned, non-overlapping buffers: tiles of kCopyUnroll vectors
// per thread walked grid-stride by many small CTAs, loads that bypass L1 and evict-first
// stores (every byte is touched once). Measured on a B200 at 256 MiB against other shapes
// (share-per-CTA, 256-bit accesses, bulk-async copies through shared memory, one tile per CTA):
// 256 threads x 4 vectors with about 48 CTAs per SM was the fastest, 5 % above cudaMemcpyAsync.
constexpr int kCopyThreads = 256, kCopyUnroll = 4, kCopyCtasPerSm = 48;
__device__ __forceinline__ void st16_stream(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__global__ void __launch_bounds__(kCopyThreads) k_copy_stream(char* dst, const char* src, size_t bytes) {
  const size_t nv = bytes >> 4, nt = kCopyThreads, tile = nt * kCopyUnroll;
  for (size_t base = size_t(blockIdx.x) * tile; base < nv; base += size_t(gridDim.x) * tile) {
    uint4 r[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const size_t i = base + u * nt + threadIdx.x;
      if (i < nv) r[u] = ld16_stream(src + (i << 4));
    }
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const size_t i = base + u * nt + threadIdx.x;
      if (i < nv) st16_stream(dst + (i << 4), r[u]);
    }
  }
  if (blockIdx.x == 0)  // the last bytes of a size that is not a multiple of 16
    for (size_t k = (nv << 4) + threadIdx.x; k < bytes; k += nt) dst[k] = src[k];
}
cudaError_t launch_copy(void* dst, const void* src, size_t bytes, cudaStream_t st) {
  if (bytes == 0 || dst == src) return cudaSuccess;
  const uintptr_t d = reinterpret_cast<uintptr_t>(dst), s = reinterpret_cast<uintptr_t>(src);
  const bool apart = d + bytes <= s || s + bytes <= d;  // the read-only load path needs this
  if (((d | s) & 15u) == 0 && apart) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t tiles = ((bytes >> 4) + size_t(kCopyThreads) * kCopyUnroll - 1) / (size_t(kCopyThreads) * kCopyUnroll);
    const int grid = int(std::max<size_t>(1, std::min<size_t>(tiles, size_t(std::max(sms, 1)) * kCopyCtasPerSm)));
    k_copy_stream<<<grid, kCopyThreads, 0, st>>>(static_cast<char*>(dst), static_cast<const char*>(src), bytes);
    return cudaGetLastError();
  }
  const int grid = int(std::min<size_t>(size_t(max_resident_ctas(512)) * 2, (bytes + 65535) / 65536));
  const size_t share = ((bytes + grid - 1) / grid + 15) & ~size_t(15);
  k_copy<<<grid, 512, 0, st>>>(static_cast<char*>(dst), static_cast<const char*>(src), bytes, share);
  return cudaGetLastError();
}

cudaError_t launch_xchg_copy(const XchgArgs* args, LaunchShape s, cudaStream_t st) {
  if (s.world) return launch_world(reinterpret_cast<const void*>(&k_xchg_copy_world), args, s, st);
  k_xchg_copy<<<s.ctas, s.threads, 0, st>>>(*args);
  return cudaGetLastError();
}

cudaError_t launch_p2p(const P2pArgs* args, LaunchShape s, cudaStream_t st) {
  if (s.world) return launch_world(reinterpret_cast<const void*>(&k_p2p_world), args, s, st);
  if (args->bulk) {
    static const cudaError_t opted = cudaFuncSetAttribute(k_p2p_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kBulkSmemBytes));
    if (opted != cudaSuccess) return opted;
    k_p2p_bulk<<<s.ctas, s.threads, kBulkSmemBytes, st>>>(*args);
    return cudaGetLastError();
  }
  k_p2p<<<s.ctas, s.threads, 0, st>>>(*args);
  return cudaGetLastError();
}

#define HX_EXTERN_TYPE(T)                                                                       \
  extern template cudaError_t launch_xchg_fold_t<T>(const XchgArgs*, LaunchShape, cudaStream_t); \
  extern template cudaError_t launch_twoshot_t<T>(const TwoShotArgs*, LaunchShape, cudaStream_t); \
  extern template cudaError_t launch_twoshot_roles_t<T>(const TwoShotArgs*, LaunchShape, cudaStream_t); \
  extern template cudaError_t launch_ring_t<T>(const TwoShotArgs*, LaunchShape, cudaStream_t);  \
  extern template cudaError_t launch_ll_t<T>(const LLArgs*, LaunchShape, cudaStream_t);         \
  extern template cudaError_t launch_reduce_t<T>(void*, const void*, size_t, int, cudaStream_t); \
  extern template cudaError_t launch_scale_t<T>(void*, const void*, size_t, unsigned long long, \
                                                cudaStream_t);                                  \
  extern template cudaError_t launch_divide_t<T>(void*, size_t, int, cudaStream_t);
HX_EXTERN_TYPE(int8_t)
HX_EXTERN_TYPE(uint8_t)
HX_EXTERN_TYPE(int32_t)
HX_EXTERN_TYPE(uint32_t)
HX_EXTERN_TYPE(int64_t)
HX_EXTERN_TYPE(uint64_t)
HX_EXTERN_TYPE(float)
HX_EXTERN_TYPE(double)
HX_EXTERN_TYPE(f16)
HX_EXTERN_TYPE(bf16)
HX_EXTERN_TYPE(e4m3)
HX_EXTERN_TYPE(e5m2)

cudaError_t launch_xchg_fold(int dt, const XchgArgs* args, LaunchShape s, cudaStream_t st) {
  cudaError_t rc = cudaErrorInvalidValue;
  HX_DISPATCH_DTYPE(dt, rc = launch_xchg_fold_t<T>(args, s, st))
  return rc;
}
cudaError_t launch_twoshot(int dt, const TwoShotArgs* args, LaunchShape s, cudaStream_t st) {
  cudaError_t rc = cudaErrorInvalidValue;
  HX_DISPATCH_DTYPE(dt, rc = launch_twoshot_t<T>(args, s, st))
  return rc;
}
cudaError_t launch_twoshot_roles(int dt, const TwoShotArgs* args, LaunchShape s, cudaStream_t st) {
  cudaError_t rc = cudaErrorInvalidValue;
  HX_DISPATCH_DTYPE(dt, rc = launch_twoshot_roles_t<T>(args, s, st))
  return rc;
}
cudaError_t launch_ring(int dt, const TwoShotArgs* args, LaunchShape s, cudaStream_t st) {
  cudaError_t rc = cudaErrorInvalidValue;
  HX_DISPATCH_DTYPE(dt, rc = launch_ring_t<T>(args, s, st))
  return rc;
}
extern template cudaError_t launch_twoshot_cast_t<f16>(const TwoShotArgs*, LaunchShape, cudaStream_t);
extern template cudaError_t launch_twoshot_cast_t<bf16>(const TwoShotArgs*, LaunchShape, cudaStream_t);
cudaError_t launch_twoshot_cast(int wire_dt, const TwoShotArgs* args, LaunchShape s, cudaStream_t st) {
  if (wire_dt == hxcclFloat16) return launch_twoshot_cast_t<f16>(args, s, st);
  if (wire_dt == hxcclBfloat16) return launch_twoshot_cast_t<bf16>(args, s, st);
  return cudaErrorInvalidValue;
}
cudaError_t launch_ll(int dt, const LLArgs* args, LaunchShape s, cudaStream_t st) {
  cudaError_t rc = cudaErrorInvalidValue;
  HX_DISPATCH_DTYPE(dt, rc = launch_ll_t<T>(args, s, st))
  return rc;
}
cudaError_t launch_reduce(void* dst, const void* src, size_t count, int dt, int op, cudaStream_t st) {
  cudaError_t rc = cudaErrorInvalidValue;
  HX_DISPATCH_DTYPE(dt, rc = launch_reduce_t<T>(dst, src, count, op, st))
  return rc;
}
cudaError_t launch_scale(void* dst, const void* src, size_t count, int dt, const void* scalar_host,
                         cudaStream_t st) {
  unsigned long long bits = 0;
  memcpy(&bits, scalar_host, dtype_size(dt));
  cudaError_t rc = cudaErrorInvalidValue;
  HX_DISPATCH_DTYPE(dt, rc = launch_scale_t<T>(dst, src, count, bits, st))
  return rc;
}
cudaError_t launch_divide(void* buf, size_t count, int dt, int divisor, cudaStream_t st) {
  cudaError_t rc = cudaErrorInvalidValue;
  HX_DISPATCH_DTYPE(dt, rc = launch_divide_t<T>(buf, count, divisor, st))
  return rc;
}

#define HX_NVLS_CASE(MODE, T)                                         \
  case MODE:                                                          \
    if (roles)                                                        \
      k_nvls_roles<T, MODE><<<s.ctas, s.threads, 0, st>>>(*args);     \
    else                                                              \
      k_nvls<T, MODE><<<s.ctas, s.threads, 0, st>>>(*args);           \
    break;
cudaError_t launch_nvls(const NvlsArgs* args, LaunchShape s, cudaStream_t st, bool roles) {
  switch (nvls_mode(args->dt, args->op)) {
    HX_NVLS_CASE(kNvF32Add, float)
    HX_NVLS_CASE(kNvF64Add, double)
    HX_NVLS_CASE(kNvF16Add, f16)
    HX_NVLS_CASE(kNvF16Min, f16)
    HX_NVLS_CASE(kNvF16Max, f16)
    HX_NVLS_CASE(kNvBf16Add, bf16)
    HX_NVLS_CASE(kNvBf16Min, bf16)
    HX_NVLS_CASE(kNvBf16Max, bf16)
    HX_NVLS_CASE(kNvS32Add, int32_t)  // wrapping add: the same bits for signed and unsigned
    HX_NVLS_CASE(kNvS32Min, int32_t)
    HX_NVLS_CASE(kNvS32Max, int32_t)
    HX_NVLS_CASE(kNvU32Min, uint32_t)
    HX_NVLS_CASE(kNvU32Max, uint32_t)
    HX_NVLS_CASE(kNvU64Add, uint64_t)
    HX_NVLS_CASE(kNvS64Min, int64_t)
    HX_NVLS_CASE(kNvS64Max, int64_t)
    HX_NVLS_CASE(kNvU64Min, uint64_t)
    HX_NVLS_CASE(kNvU64Max, uint64_t)
    HX_NVLS_CASE(kNvE4m3Add, e4m3)
    HX_NVLS_CASE(kNvE4m3Min, e4m3)
    HX_NVLS_CASE(kNvE4m3Max, e4m3)
    HX_NVLS_CASE(kNvE5m2Add, e5m2)
    HX_NVLS_CASE(kNvE5m2Min, e5m2)
    HX_NVLS_CASE(kNvE5m2Max, e5m2)
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

int max_resident_ctas(int threads) {
  // The collective kernels differ in register use from type to type; every one of them fits
  // one 512-thread CTA per SM (__launch_bounds__(512) caps them at 128 registers per thread),
  // hence also two CTAs of 256 threads. That is what is promised, whatever the type.
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 1;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms < 1) sms = 1;
  return threads <= 256 ? 2 * sms : sms;
}

}  // namespace hx
