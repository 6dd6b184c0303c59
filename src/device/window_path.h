// The production device path: one window per rank allocated with the CUDA virtual-memory API,
// exported as a file descriptor, mapped by every peer, and (where every GPU supports it) bound
// to one NVSwitch multicast object. Set-up is collective: every step runs on every rank and
// the ranks agree on its outcome before the next one, so that a failure on one rank turns into
// the same fallback everywhere instead of a hang (the discipline of the reference's
// IpcTransport::init, src/transport_ipc.cc:83-166).
#pragma once
#include <cuda.h>

#include <memory>
#include <vector>

#include "core/comm.h"
#include "device/engine.h"

namespace hx {

class WindowPath : public DevicePath {
 public:
  explicit WindowPath(hxcclComm* c);
  ~WindowPath() override;
  // collective; hxcclSuccess, or a code with `error` set (then the caller falls back)
  hxcclResult_t init();

  hxcclResult_t broken(std::string* why) override;
  const char* kind() const override { return nvls_ ? "window+nvls" : "window"; }
  int device() const override { return dev_; }
  hxcclResult_t allreduce(const void* send, void* recv, size_t count, int dt, const OpPlan& plan,
                          int order, void* stream) override;
  hxcclResult_t allreduce_cast(const void* send, void* recv, size_t count, int wire_dt, const OpPlan& plan,
                               void* stream) override;
  hxcclResult_t allgather(const void* send, void* recv, size_t block, void* stream) override;
  hxcclResult_t reducescatter(const void* send, void* recv, size_t per, int dt,
                              const OpPlan& plan, void* stream) override;
  hxcclResult_t broadcast(const void* send, void* recv, size_t bytes, int root,
                          void* stream) override;
  hxcclResult_t reduce(const void* send, void* recv, size_t count, int dt, const OpPlan& plan,
                       int root, void* stream) override;
  hxcclResult_t gather(const void* send, void* recv, size_t block, int root,
                       void* stream) override;
  hxcclResult_t scatter(const void* send, void* recv, size_t block, int root,
                        void* stream) override;
  hxcclResult_t alltoallv(const char* send, const size_t* sbytes, const size_t* soff, char* recv,
                          const size_t* rbytes, const size_t* roff, size_t max_pair,
                          void* stream) override;
  hxcclResult_t p2p_batch(const std::vector<P2pOp>& ops, void* stream) override;
  hxcclResult_t drain() override;

  Engine& engine() { return eng_; }
  // Phase timers (HXCCL_TRACE=1): copies kTraceSlots nanosecond sums per CTA to `out` (up to
  // `max_ctas` rows) after draining the stream, and clears them. Returns the rows copied.
  int read_trace(unsigned long long* out, int max_ctas);

 private:
  hxcclResult_t fail(hxcclResult_t r, const std::string& why);
  bool agree(bool ok);  // true when every rank reports ok
  hxcclResult_t setup_local();
  hxcclResult_t setup_windows();
  void setup_multicast();
  void release();
  cudaStream_t enter(void* stream);  // orders this launch after earlier ones on other streams
  hxcclResult_t done(cudaError_t e, const char* what);

  hxcclComm* c_;
  int rank_, n_;
  int dev_ = 0;
  CUdevice cudev_ = 0;
  size_t win_bytes_ = 0;
  size_t p2p_slot_ = kP2pSlotBytes;  // Send/Recv slot size of this communicator
  bool vmm_ = false;  // windows came from cuMemCreate (else one cudaMalloc, n == 1)
  CUmemGenericAllocationHandle own_h_ = 0;
  std::vector<CUmemGenericAllocationHandle> peer_h_;
  std::vector<CUdeviceptr> va_;
  CUmemGenericAllocationHandle mc_h_ = 0;
  CUdeviceptr mc_va_ = 0;
  bool mc_bound_ = false;
  bool nvls_ = false;
  unsigned long long* status_ = nullptr;  // pinned host: [0] sticky, [1] soft
  Engine eng_;
  int caller_dev_ = -1;  // the caller's current device while a launch switched to dev_
  cudaStream_t last_stream_ = nullptr;
  bool used_ = false;
  cudaEvent_t order_event_ = nullptr;
  unsigned long long* trace_ = nullptr;
  void* scratch_ = nullptr;  // private copy of an overlapping AlltoAll send side
  size_t scratch_bytes_ = 0;
  hxcclResult_t broken_ = hxcclSuccess;
  std::string broken_why_;
};

}  // namespace hx
