// A whole communicator on one GPU (include/hxccl_ext.h: hxcclWorld*). Every rank gets a
// window in the same device's memory and the kernels run for all ranks in one cooperative
// launch, so ranks really are concurrent. It exists for testing the kernels where only one GPU
// is available; separate launches that wait on each other on one GPU must never be used
// instead, since nothing makes them run at the same time.
#include <cuda_runtime.h>

#include <cstring>
#include <string>
#include <vector>

#include "device/engine.h"
#include "hxccl_ext.h"
#include "math/dtypes.h"
#include "math/reduce_host.h"

struct hxcclWorld {
  int n = 0;
  std::vector<void*> windows;
  void* dummy = nullptr;
  unsigned long long* status = nullptr;  // pinned: [2*r] sticky, [2*r+1] soft
  hx::Engine eng;
};

namespace {
using namespace hx;

size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

// the plan hxcclAllReduce would make for (op, scalar) on n ranks
bool make_plan(int n, int dt, int op, const void* scalar, OpPlan* p) {
  *p = OpPlan{};
  if (scalar) {
    p->premul = true;
    std::memcpy(p->scalar, scalar, dtype_size(dt));
    return op == hxcclSum;
  }
  if (is_builtin_op(op)) {
    p->base = op;
    return true;
  }
  if (op != hxcclAvg) return false;
  if (is_integer(dt)) {
    p->postdiv = true;
    p->divisor = n;
  } else {
    p->premul = true;
    store_scalar(1.0 / n, dt, p->scalar);
  }
  return true;
}

// CTAs the whole world may use together. Kept well below the co-residency bound of the
// heaviest kernel: a cooperative launch is refused outright when it does not fit, and other
// work on the device can take SMs away.
int world_cta_budget() { return std::max(1, max_resident_ctas(512) * 3 / 4); }

std::vector<RankBufs> bufs(hxcclWorld* w, const void* const* send, void* const* recv) {
  std::vector<RankBufs> b(w->n);
  for (int r = 0; r < w->n; ++r) b[r] = RankBufs{send ? send[r] : nullptr, recv ? recv[r] : nullptr};
  return b;
}
std::string g_last_error;
hxcclResult_t rc_of(cudaError_t e) {
  if (e == cudaSuccess) return hxcclSuccess;
  g_last_error = cudaGetErrorString(e);
  return hxcclUnhandledCudaError;
}
}  // namespace

extern "C" {

hxcclResult_t hxcclWorldCreate(hxcclWorld_t* out, int n, int window_mb, int wait_ms) {
  if (!out || n < 1 || n > kMaxRanks || window_mb < 1 || wait_ms < 1) return hxcclInvalidArgument;
  auto* w = new hxcclWorld;
  w->n = n;
  const size_t p2p = round_up(p2p_region_bytes(n), 1u << 20);
  const size_t half = (size_t(window_mb) << 20) / 2;
  const size_t total = kHeaderBytes + p2p + 2 * half;
  bool ok = cudaHostAlloc(reinterpret_cast<void**>(&w->status), 16 * size_t(n), cudaHostAllocMapped) == cudaSuccess;
  if (ok) std::memset(w->status, 0, 16 * size_t(n));
  for (int r = 0; ok && r < n; ++r) {
    void* p = nullptr;
    ok = cudaMalloc(&p, total) == cudaSuccess && cudaMemset(p, 0, kHeaderBytes) == cudaSuccess;
    w->windows.push_back(p);
  }
  ok = ok && cudaMalloc(&w->dummy, total) == cudaSuccess && cudaMemset(w->dummy, 0, kHeaderBytes) == cudaSuccess;
  if (!ok) {
    hxcclWorldDestroy(w);
    return hxcclUnhandledCudaError;
  }
  for (int r = 0; r < n; ++r) {
    WinView v{};
    for (int p = 0; p < n; ++p) v.win[p] = static_cast<char*>(w->windows[p]);
    v.status = w->status + 2 * r;
    v.soft = w->status + 2 * r + 1;
    v.half_off[0] = kHeaderBytes + p2p;
    v.half_off[1] = v.half_off[0] + half;
    v.half_bytes = half;
    v.p2p_slot = kP2pSlotBytes;
    v.wait_ns = uint64_t(wait_ms) * 1000000ull;
    v.rank = r;
    v.n = n;
    w->eng.views.push_back(v);
  }
  // the whole world must be co-resident: a cooperative launch refuses anything larger
  w->eng.tune.max_ctas = std::max(1, std::min(64, world_cta_budget() / n));
  w->eng.tune.threads = 512;  // one CTA per SM: the budget above counts on it
  w->eng.tune.roles_min_ranks = 2;
  *out = w;
  return cudaDeviceSynchronize() == cudaSuccess ? hxcclSuccess : hxcclUnhandledCudaError;
}

hxcclResult_t hxcclWorldDestroy(hxcclWorld_t w) {
  if (!w) return hxcclInvalidArgument;
  cudaDeviceSynchronize();
  for (void* p : w->windows)
    if (p) cudaFree(p);
  if (w->dummy) cudaFree(w->dummy);
  if (w->status) cudaFreeHost(w->status);
  delete w;
  return hxcclSuccess;
}

hxcclResult_t hxcclWorldTune(hxcclWorld_t w, int variant, int exact, int max_ctas) {
  if (!w) return hxcclInvalidArgument;
  w->eng.forced_variant = variant;
  w->eng.tune.exact = exact != 0;
  if (max_ctas > 0) w->eng.tune.max_ctas = std::min(max_ctas, std::max(1, world_cta_budget() / w->n));
  return hxcclSuccess;
}

hxcclResult_t hxcclWorldTuneKnob(hxcclWorld_t w, const char* name, long value) {
  if (!w) return hxcclInvalidArgument;
  if (!set_knob(&w->eng.tune, name, value)) return hxcclInvalidArgument;
  w->eng.tune.max_ctas = std::min(w->eng.tune.max_ctas, std::max(1, world_cta_budget() / w->n));
  return hxcclSuccess;
}

hxcclResult_t hxcclWorldAllReduce(hxcclWorld_t w, const void* const* send, void* const* recv,
                                  size_t count, hxcclDataType_t dt, hxcclRedOp_t op,
                                  const void* scalar, int order, hxcclStream_t stream) {
  OpPlan plan;
  if (!w || !make_plan(w->n, dt, op, scalar, &plan) || dtype_size(dt) == 0) return hxcclInvalidArgument;
  if (count == 0) return hxcclSuccess;
  if (order < 0) order = count * dtype_size(dt) < kDoublingMaxBytes ? kOrderDoubling : kOrderRing;
  auto b = bufs(w, send, recv);
  return rc_of(w->eng.allreduce(b.data(), count, dt, plan, order, static_cast<cudaStream_t>(stream)));
}

hxcclResult_t hxcclWorldAllReduceCast(hxcclWorld_t w, const void* const* send, void* const* recv,
                                      size_t count, hxcclDataType_t wire_dt, hxcclRedOp_t op,
                                      hxcclStream_t stream) {
  OpPlan plan;
  if (!w || (wire_dt != hxcclFloat16 && wire_dt != hxcclBfloat16) || !make_plan(w->n, wire_dt, op, nullptr, &plan))
    return hxcclInvalidArgument;
  if (count == 0) return hxcclSuccess;
  if (w->n < 2) return hxcclInvalidUsage;
  auto b = bufs(w, send, recv);
  return rc_of(w->eng.allreduce_cast(b.data(), count, wire_dt, plan, static_cast<cudaStream_t>(stream)));
}

hxcclResult_t hxcclWorldReduceScatter(hxcclWorld_t w, const void* const* send, void* const* recv,
                                      size_t recvcount, hxcclDataType_t dt, hxcclRedOp_t op,
                                      const void* scalar, hxcclStream_t stream) {
  OpPlan plan;
  if (!w || !make_plan(w->n, dt, op, scalar, &plan) || dtype_size(dt) == 0) return hxcclInvalidArgument;
  if (recvcount == 0) return hxcclSuccess;
  auto b = bufs(w, send, recv);
  return rc_of(w->eng.reducescatter(b.data(), recvcount, dt, plan, static_cast<cudaStream_t>(stream)));
}

hxcclResult_t hxcclWorldReduce(hxcclWorld_t w, const void* const* send, void* const* recv,
                               size_t count, hxcclDataType_t dt, hxcclRedOp_t op,
                               const void* scalar, int root, hxcclStream_t stream) {
  OpPlan plan;
  if (!w || !make_plan(w->n, dt, op, scalar, &plan) || dtype_size(dt) == 0 || root < 0 || root >= w->n)
    return hxcclInvalidArgument;
  if (count == 0) return hxcclSuccess;
  auto b = bufs(w, send, recv);
  return rc_of(w->eng.reduce(b.data(), count, dt, plan, root, static_cast<cudaStream_t>(stream)));
}

hxcclResult_t hxcclWorldAllGather(hxcclWorld_t w, const void* const* send, void* const* recv,
                                  size_t bytes, hxcclStream_t stream) {
  if (!w) return hxcclInvalidArgument;
  if (bytes == 0) return hxcclSuccess;
  auto b = bufs(w, send, recv);
  return rc_of(w->eng.allgather(b.data(), bytes, static_cast<cudaStream_t>(stream)));
}
hxcclResult_t hxcclWorldBroadcast(hxcclWorld_t w, const void* const* send, void* const* recv,
                                  size_t bytes, int root, hxcclStream_t stream) {
  if (!w || root < 0 || root >= w->n) return hxcclInvalidArgument;
  if (bytes == 0) return hxcclSuccess;
  auto b = bufs(w, send, recv);
  return rc_of(w->eng.broadcast(b.data(), bytes, root, static_cast<cudaStream_t>(stream)));
}
hxcclResult_t hxcclWorldGather(hxcclWorld_t w, const void* const* send, void* const* recv,
                               size_t bytes, int root, hxcclStream_t stream) {
  if (!w || root < 0 || root >= w->n) return hxcclInvalidArgument;
  if (bytes == 0) return hxcclSuccess;
  auto b = bufs(w, send, recv);
  return rc_of(w->eng.gather(b.data(), bytes, root, static_cast<cudaStream_t>(stream)));
}
hxcclResult_t hxcclWorldScatter(hxcclWorld_t w, const void* const* send, void* const* recv,
                                size_t bytes, int root, hxcclStream_t stream) {
  if (!w || root < 0 || root >= w->n) return hxcclInvalidArgument;
  if (bytes == 0) return hxcclSuccess;
  auto b = bufs(w, send, recv);
  return rc_of(w->eng.scatter(b.data(), bytes, root, static_cast<cudaStream_t>(stream)));
}

hxcclResult_t hxcclWorldAllToAllv(hxcclWorld_t w, const void* const* send, void* const* recv,
                                  const size_t* bytes, const size_t* soff, const size_t* roff,
                                  hxcclStream_t stream) {
  if (!w || !bytes || !soff || !roff) return hxcclInvalidArgument;
  const int n = w->n;
  std::vector<size_t> rbytes(size_t(n) * n);
  size_t max_pair = 0;
  for (int r = 0; r < n; ++r)
    for (int i = 0; i < n; ++i) {
      rbytes[size_t(r) * n + i] = bytes[size_t(i) * n + r];
      max_pair = std::max(max_pair, bytes[size_t(r) * n + i]);
    }
  if (max_pair == 0) return hxcclSuccess;
  std::vector<RankV> v(n);
  for (int r = 0; r < n; ++r)
    v[r] = RankV{static_cast<const char*>(send[r]), bytes + size_t(r) * n, soff + size_t(r) * n,
                 static_cast<char*>(recv[r]), rbytes.data() + size_t(r) * n, roff + size_t(r) * n};
  return rc_of(w->eng.alltoallv(v.data(), max_pair, static_cast<cudaStream_t>(stream)));
}

hxcclResult_t hxcclWorldSendRecv(hxcclWorld_t w, int nops, const int* from, const int* to,
                                 const void* const* src, const size_t* sbytes, void* const* dst,
                                 const size_t* rbytes, hxcclStream_t stream) {
  if (!w || nops < 0) return hxcclInvalidArgument;
  std::vector<RankP2p> per(w->n);
  for (int k = 0; k < nops; ++k) {
    if (from[k] < 0 || from[k] >= w->n || to[k] < 0 || to[k] >= w->n) return hxcclInvalidArgument;
    per[from[k]].ops.push_back(P2pOp{true, to[k], const_cast<void*>(src[k]), sbytes[k]});
    per[to[k]].ops.push_back(P2pOp{false, from[k], dst[k], rbytes[k]});
  }
  return rc_of(w->eng.p2p(per.data(), static_cast<cudaStream_t>(stream)));
}

hxcclResult_t hxcclWorldStatus(hxcclWorld_t w, int rank, unsigned long long* sticky,
                               unsigned long long* soft) {
  if (!w || rank < 0 || rank >= w->n || !sticky || !soft) return hxcclInvalidArgument;
  volatile unsigned long long* s = w->status + 2 * rank;
  *sticky = s[0];
  *soft = s[1];
  s[1] = 0;
  return hxcclSuccess;
}

hxcclResult_t hxcclWorldInfo(hxcclWorld_t w, int* variant, unsigned long long* launches) {
  if (!w) return hxcclInvalidArgument;
  if (variant) *variant = w->eng.last_variant;
  if (launches) *launches = w->eng.launches;
  return hxcclSuccess;
}

const char* hxcclWorldLastError(void) { return g_last_error.c_str(); }

hxcclResult_t hxcclWorldMute(hxcclWorld_t w, int rank) {
  if (!w || rank < 0 || rank >= w->n) return hxcclInvalidArgument;
  for (int p = 0; p < w->n; ++p)
    if (p != rank) w->eng.views[rank].win[p] = static_cast<char*>(w->dummy);
  return hxcclSuccess;
}

}  // extern "C"
