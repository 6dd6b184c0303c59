// hxcclAllReduceNoAlloc: the one-shot AllReduce of the world-on-one-GPU harness with every
// byte of scratch in a static device array (see noalloc.h for who needs that and the rules).
#include "kernels/noalloc.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <string>

#include "device/planner.h"
#include "kernels/launch.h"
#include "math/dtypes.h"
#include "math/reduce_host.h"

namespace {
using namespace hx;

// window of one rank: flag pages, then two staging halves
constexpr size_t kHalf = 512 * 1024;
constexpr size_t kWindow = 256 * 1024 + 2 * kHalf;
static_assert(kOffFlagsB + size_t(kMaxCtas) * kMaxRanks * 8 <= 256 * 1024, "flag pages must fit the header");
constexpr size_t kArgsOff = HXCCL_NOALLOC_MAX_RANKS * kWindow;
constexpr size_t kStatusOff = kArgsOff + 8192;  // 2 words per rank
static_assert(HXCCL_NOALLOC_MAX_RANKS * sizeof(XchgArgs) <= 8192, "argument blocks must fit");
constexpr size_t kScratchBytes = kStatusOff + 256;

// The scratch. In host code this name is only a handle for cudaGetSymbolAddress: it is not a
// device address and must never be handed to a kernel as one.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
  unsigned char* base = nullptr;  // device address of g_scratch on this device, as last looked up
  unsigned long long epoch = 2;
  bool dirty = false;             // flags are in an unknown state (failed call, or a new context)
};
PerDevice g_dev[kMaxDevices];
char g_error[256] = "";

hxcclResult_t fail(hxcclResult_t r, const char* msg, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess)
    std::snprintf(g_error, sizeof g_error, "%s: %s", msg, cudaGetErrorString(e));
  else
    std::snprintf(g_error, sizeof g_error, "%s", msg);
  return r;
}
}  // namespace

extern "C" const char* hxcclNoAllocLastError(void) { return g_error; }

extern "C" hxcclResult_t hxcclAllReduceNoAlloc(int nranks, const void* const* send, void* const* recv,
                                               size_t count, hxcclDataType_t dt, hxcclRedOp_t op,
                                               hxcclStream_t stream) {
  const size_t es = dtype_size(dt);
  if (nranks < 1 || nranks > HXCCL_NOALLOC_MAX_RANKS)
    return fail(hxcclInvalidArgument, "nranks must be between 1 and HXCCL_NOALLOC_MAX_RANKS");
  if (es == 0) return fail(hxcclInvalidArgument, "unknown datatype");
  if (!is_builtin_op(op) && op != hxcclAvg) return fail(hxcclInvalidArgument, "unsupported operator");
  if (count > HXCCL_NOALLOC_MAX_BYTES / es)
    return fail(hxcclInvalidArgument, "count * sizeof(datatype) exceeds HXCCL_NOALLOC_MAX_BYTES");
  if (count == 0) return hxcclSuccess;
  if (!send || !recv) return fail(hxcclInvalidArgument, "null buffer list");
  for (int r = 0; r < nranks; ++r)
    if (!send[r] || !recv[r]) return fail(hxcclInvalidArgument, "null buffer");

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(hxcclUnhandledCudaError, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(hxcclInvalidArgument, "device ordinal out of range");
  PerDevice& pd = g_dev[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {  // The array's device address, with this device current. The first call on a device is
     // the set-up; later calls repeat the (cheap) look-up instead of trusting a cached pointer,
     // which a cudaDeviceReset or another context on the same ordinal would leave stale. A
     // changed address means a fresh array image: start over from cleared flags.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess || !p) return fail(hxcclUnhandledCudaError, "cudaGetSymbolAddress", e);
    if (p != pd.base) {
      pd.base = static_cast<unsigned char*>(p);
      pd.dirty = true;
    }
  }
  if (pd.dirty) {  // start over from zeroed flags
    e = cudaMemsetAsync(pd.base, 0, kScratchBytes, st);
    if (e != cudaSuccess) return fail(hxcclUnhandledCudaError, "clearing the scratch", e);
    pd.epoch = 2;
    pd.dirty = false;
  }
  // status and abort words must start at zero in every call
  e = cudaMemsetAsync(pd.base + kStatusOff, 0, 256, st);
  for (int r = 0; e == cudaSuccess && r < nranks; ++r)
    e = cudaMemsetAsync(pd.base + size_t(r) * kWindow + kOffAbort, 0, 8, st);
  if (e != cudaSuccess) return fail(hxcclUnhandledCudaError, "clearing the status words", e);

  // the operator, resolved as hxcclAllReduce resolves it
  OpPlan plan;
  if (is_builtin_op(op)) {
    plan.base = op;
  } else if (is_integer(dt)) {
    plan.postdiv = true;
    plan.divisor = nranks;
  } else {
    plan.premul = true;
    store_scalar(1.0 / nranks, dt, plan.scalar);
  }
  const size_t bytes = count * es;
  const int order = bytes < kDoublingMaxBytes ? kOrderDoubling : kOrderRing;
  Tuning tune;
  tune.max_ctas = 16;
  const Geometry g = plan_xchg(bytes, nranks, kHalf, tune);
  // the host-side bounds check every other launch of this library gets
  const std::string bad_shape = check_geometry(kPlanXchg, g, bytes, nranks, kHalf);
  if (!bad_shape.empty() || size_t(g.ctas) * nranks > size_t(max_resident_ctas(g.threads)))
    return fail(hxcclInternalError, bad_shape.empty() ? "grid too large for a cooperative launch" : bad_shape.c_str());

  XchgArgs args[HXCCL_NOALLOC_MAX_RANKS];
  for (int r = 0; r < nranks; ++r) {
    WinView w{};
    for (int p = 0; p < nranks; ++p) w.win[p] = reinterpret_cast<char*>(pd.base + size_t(p) * kWindow);
    w.status = reinterpret_cast<unsigned long long*>(pd.base + kStatusOff) + 2 * r;
    w.soft = w.status + 1;
    w.half_off[0] = 256 * 1024;
    w.half_off[1] = 256 * 1024 + kHalf;
    w.half_bytes = kHalf;
    w.wait_ns = 5ull * 1000 * 1000 * 1000;
    w.rank = r;
    w.n = nranks;
    build_allreduce_oneshot(&args[r], w, pd.epoch, g, send[r], recv[r], count, dt, plan, order);
  }
  pd.epoch += g.epochs;
  const XchgArgs* dev_args = reinterpret_cast<const XchgArgs*>(pd.base + kArgsOff);
  e = cudaMemcpyAsync(pd.base + kArgsOff, args, sizeof(XchgArgs) * nranks, cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) return fail(hxcclUnhandledCudaError, "staging the arguments", e);
  // `args` lives on this stack frame: the copy of pageable memory has read it by now, and the
  // function does not return before the stream is idle anyway
  e = launch_xchg_fold(dt, dev_args, LaunchShape{g.ctas, g.threads, nranks}, st);
  if (e != cudaSuccess) {
    pd.dirty = true;
    return fail(hxcclUnhandledCudaError, "launching the AllReduce kernel", e);
  }
  unsigned long long status[2 * HXCCL_NOALLOC_MAX_RANKS] = {};
  e = cudaMemcpyAsync(status, pd.base + kStatusOff, sizeof status, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    pd.dirty = true;
    return fail(hxcclUnhandledCudaError, "waiting for the AllReduce kernel", e);
  }
  for (int r = 0; r < nranks; ++r)
    if (status[2 * r]) {
      pd.dirty = true;
      return fail(hxcclTimeout, "a device-side wait ran out of time");
    }
  return hxcclSuccess;
}
