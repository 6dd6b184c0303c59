// What the front end needs from the device data path. Two implementations exist
// (src/device): the peer-window path that launches the sm_100a kernels, and the staged path
// that bounces device buffers through host memory and the host algorithms when peer mapping is
// not possible (the reference's IPC / staged split: src/transport_ipc.cc:91-166, :224-325).
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "hxccl.h"

struct hxcclComm;

namespace hx {

// A reduction operator resolved at call time (reference: src/checks.h:15-21). Kernels take
// the pre-scale and the post-divide as launch parameters, so neither is a separate pass.
struct OpPlan {
  int base = hxcclSum;             // kSum / kProd / kMax / kMin
  bool premul = false;             // multiply each local input element by the scalar first
  unsigned char scalar[8] = {};    // the scalar's bits when known on the host
  const void* scalar_dev = nullptr;  // else: device address the kernel reads in stream order
  bool postdiv = false;            // integer Avg: divide the result by `divisor`
  int divisor = 1;
};

struct P2pOp {
  bool is_send;
  int peer;
  void* buf;
  size_t bytes;
};

class DevicePath {
 public:
  virtual ~DevicePath() = default;
  // hxcclSuccess while usable; after a failed transfer (here or on a peer) the path stays
  // failed and every later device call returns the same code.
  virtual hxcclResult_t broken(std::string* why) = 0;
  virtual const char* kind() const = 0;  // "window", "window+nvls" or "staged"
  // The CUDA device whose memory this path's kernels can address, or -1 when buffers of any
  // device will do (the staged path copies through the host).
  virtual int device() const { return -1; }

  virtual hxcclResult_t allreduce(const void* send, void* recv, size_t count, int dt,
                                  const OpPlan& plan, int order, void* stream) = 0;
  // fp32 buffers reduced with `wire_dt` (fp16 / bf16) on the wire; paths without a fused
  // kernel answer hxcclInvalidUsage and the caller casts for itself
  virtual hxcclResult_t allreduce_cast(const void*, void*, size_t, int /*wire_dt*/, const OpPlan&, void* /*stream*/) {
    error = "this device path has no fused cast AllReduce";
    return hxcclInvalidUsage;
  }
  virtual hxcclResult_t allgather(const void* send, void* recv, size_t block_bytes,
                                  void* stream) = 0;
  virtual hxcclResult_t reducescatter(const void* send, void* recv, size_t per, int dt,
                                      const OpPlan& plan, void* stream) = 0;
  virtual hxcclResult_t broadcast(const void* send, void* recv, size_t bytes, int root,
                                  void* stream) = 0;
  virtual hxcclResult_t reduce(const void* send, void* recv, size_t count, int dt,
                               const OpPlan& plan, int root, void* stream) = 0;
  virtual hxcclResult_t gather(const void* send, void* recv, size_t block_bytes, int root,
                               void* stream) = 0;
  virtual hxcclResult_t scatter(const void* send, void* recv, size_t block_bytes, int root,
                                void* stream) = 0;
  // max_pair_bytes: the largest block any rank sends to any rank, agreed over the control mesh
  virtual hxcclResult_t alltoallv(const char* send, const size_t* sbytes, const size_t* soff,
                                  char* recv, const size_t* rbytes, const size_t* roff,
                                  size_t max_pair_bytes, void* stream) = 0;
  // every Send/Recv of a group on this communicator, in call order
  virtual hxcclResult_t p2p_batch(const std::vector<P2pOp>& ops, void* stream) = 0;
  // waits for the work enqueued so far (used by Finalize/Destroy and blocking fallbacks)
  virtual hxcclResult_t drain() = 0;

  std::string error;
};

enum class MemKind { Null, Host, Device };
// Where `p` lives, asked of the driver without creating a CUDA context.
MemKind classify(const void* p);
// The same with the CUDA device the memory belongs to (*ordinal, -1 for host memory), in one
// driver call.
MemKind classify_on(const void* p, int* ordinal);
// CUDA device a device pointer belongs to, or -1 (host memory, unknown).
int device_ordinal_of(const void* p);
// True when this process already has a CUDA context (again without creating one).
bool cuda_context_exists();
// Collective over the communicator's ranks. Returns null with *rc/*why set on failure.
std::unique_ptr<DevicePath> start_device_path(hxcclComm* c, hxcclResult_t* rc, std::string* why);

}  // namespace hx
