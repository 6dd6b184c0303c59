// Device self-checks of the narrow-float converters: the fast device paths (hardware cvt plus
// fix-ups, fpconv.h) against the bit-manipulation reference for EVERY input, 2^32 floats for
// encode and all codes for decode. Used by the GPU tests; has no part in the data path.
#include <cuda_runtime.h>

#include "hxccl_ext.h"
#include "math/dtypes.h"

namespace hx {
namespace {

template <typename S, typename Fmt>
__global__ void k_check_encode(unsigned long long* bad, unsigned int* first_bad) {
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  unsigned long long mism = 0;
  for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x; i < (1ull << 32);
       i += stride) {
    const float x = bits_f32(static_cast<uint32_t>(i));
    S fast;
    from_f32(x, &fast);
    if (static_cast<uint32_t>(fast.b) != Fmt::encode(x)) {
      if (mism++ == 0) atomicMin(first_bad, static_cast<unsigned int>(i));
    }
  }
  if (mism) atomicAdd(bad, mism);
}

template <typename S, typename Fmt, int kBits>
__global__ void k_check_decode(unsigned long long* bad) {
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (1u << kBits)) return;
  S v;
  v.b = static_cast<decltype(v.b)>(i);
  const float fast = to_f32(v), ref = Fmt::decode(i);
  const bool same = is_nan(ref) ? is_nan(fast) : f32_bits(fast) == f32_bits(ref);
  if (!same) atomicAdd(bad, 1ull);
}

}  // namespace
}  // namespace hx

extern "C" hxcclResult_t hxcclTestNarrowConvert(hxcclDataType_t dt, unsigned long long* mismatches,
                                                unsigned int* first_bad_bits) {
  using namespace hx;
  if (!mismatches || !first_bad_bits) return hxcclInvalidArgument;
  unsigned long long* d_bad = nullptr;
  unsigned int* d_first = nullptr;
  if (cudaMalloc(&d_bad, 8) != cudaSuccess || cudaMalloc(&d_first, 4) != cudaSuccess) return hxcclUnhandledCudaError;
  cudaMemset(d_bad, 0, 8);
  cudaMemset(d_first, 0xff, 4);
  const int grid = 148 * 8, block = 256;
  switch (dt) {
    case hxcclFloat16:
      k_check_encode<f16, FmtF16><<<grid, block>>>(d_bad, d_first);
      k_check_decode<f16, FmtF16, 16><<<256, 256>>>(d_bad);
      break;
    case hxcclBfloat16:
      k_check_encode<bf16, NarrowFmt<8, 7, true>><<<grid, block>>>(d_bad, d_first);
      k_check_decode<bf16, NarrowFmt<8, 7, true>, 16><<<256, 256>>>(d_bad);
      break;
    case hxcclFloat8e4m3:
      k_check_encode<e4m3, FmtE4M3><<<grid, block>>>(d_bad, d_first);
      k_check_decode<e4m3, FmtE4M3, 8><<<1, 256>>>(d_bad);
      break;
    case hxcclFloat8e5m2:
      k_check_encode<e5m2, FmtE5M2><<<grid, block>>>(d_bad, d_first);
      k_check_decode<e5m2, FmtE5M2, 8><<<1, 256>>>(d_bad);
      break;
    default:
      cudaFree(d_bad);
      cudaFree(d_first);
      return hxcclInvalidArgument;
  }
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(mismatches, d_bad, 8, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(first_bad_bits, d_first, 4, cudaMemcpyDeviceToHost);
  cudaFree(d_bad);
  cudaFree(d_first);
  return e == cudaSuccess ? hxcclSuccess : hxcclUnhandledCudaError;
}
