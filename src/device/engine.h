// Plans and launches the collective kernels for one rank (production: one process per GPU)
// or for every rank of a small world that lives on a single GPU (tests): the same planner
// output and the same kernel bodies either way.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "device/planner.h"
#include "kernels/launch.h"

namespace hx {

struct RankBufs {
  const void* send;
  void* recv;
};
struct RankV {  // AlltoAllv arguments of one rank, in bytes
  const char* send;
  const size_t* sbytes;
  const size_t* soff;
  char* recv;
  const size_t* rbytes;
  const size_t* roff;
};
struct RankP2p {
  std::vector<P2pOp> ops;
};

class Engine {
 public:
  // views.size() == 1: production. Otherwise views[r] is rank r of a single-GPU world.
  std::vector<WinView> views;
  Tuning tune;
  uint64_t epoch = 2;  // flags start at zero; the first step must be able to tell
  int forced_variant = kVarAuto;
  int last_variant = kVarAuto;  // what the latest AllReduce used
  unsigned long long launches = 0;  // kernels launched so far
  std::string error;

  ~Engine();
  bool world() const { return views.size() > 1; }
  int n() const { return views[0].n; }

  cudaError_t allreduce(const RankBufs* b, size_t count, int dt, const OpPlan& plan, int order,
                        cudaStream_t st);
  // fp32 buffers, `wire_dt` (fp16 / bf16) carried and summed; ring order only (count * 2 bytes
  // must be at least the size from which the API takes the ring order)
  cudaError_t allreduce_cast(const RankBufs* b, size_t count, int wire_dt, const OpPlan& plan,
                             cudaStream_t st);
  cudaError_t reducescatter(const RankBufs* b, size_t per, int dt, const OpPlan& plan,
                            cudaStream_t st);
  cudaError_t reduce(const RankBufs* b, size_t count, int dt, const OpPlan& plan, int root,
                     cudaStream_t st);
  cudaError_t allgather(const RankBufs* b, size_t block, cudaStream_t st);
  cudaError_t broadcast(const RankBufs* b, size_t bytes, int root, cudaStream_t st);
  cudaError_t gather(const RankBufs* b, size_t block, int root, cudaStream_t st);
  cudaError_t scatter(const RankBufs* b, size_t block, int root, cudaStream_t st);
  cudaError_t alltoallv(const RankV* v, size_t max_pair, cudaStream_t st);
  // ops[r]: the Send/Recv list of rank r, in call order
  cudaError_t p2p(const RankP2p* ops, cudaStream_t st);

 private:
  template <typename Args>
  const Args* stage(const std::vector<Args>& args, cudaStream_t st, cudaError_t* rc);
  LaunchShape shape(const Geometry& g) const;
  uint64_t ll_era_ = 0;  // upper half of the epoch the line region was last cleared for
  void* dev_args_ = nullptr;
  size_t dev_args_bytes_ = 0;
};

}  // namespace hx
