// torch.distributed backend "hxccl" over the hxccl C API.
//
// The reference's backend (python/hxccl_torch/csrc/backend.cpp:70-161) runs every call to
// completion on the caller's stream and returns an already-finished Work. Here device
// collectives are asynchronous: each call makes the backend's communication stream wait for
// the caller's current stream, enqueues the kernel there and returns a Work whose wait() makes
// the caller's stream wait for the kernel (no host blocking) and whose Future completes in
// stream order, which is what DistributedDataParallel needs to overlap gradient buckets with
// the rest of backward. The tensor's own device is made current for every call. CPU tensors go
// through the host path and complete before the call returns.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/chrono.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/python.h>

#include <cstdlib>
#include <cstring>
#include <optional>

#include "hxccl.h"
#include "hxccl_ext.h"

namespace {
using namespace c10d;

hxcclDataType_t to_dt(at::ScalarType t) {
  switch (t) {
    case at::kChar: return hxcclInt8;
    case at::kByte: return hxcclUint8;
    case at::kBool: return hxcclUint8;
    case at::kInt: return hxcclInt32;
    case at::kUInt32: return hxcclUint32;
    case at::kLong: return hxcclInt64;
    case at::kUInt64: return hxcclUint64;
    case at::kHalf: return hxcclFloat16;
    case at::kFloat: return hxcclFloat32;
    case at::kDouble: return hxcclFloat64;
    case at::kBFloat16: return hxcclBfloat16;
    case at::kFloat8_e4m3fn: return hxcclFloat8e4m3;
    case at::kFloat8_e5m2: return hxcclFloat8e5m2;
    default: TORCH_CHECK_TYPE(false, "hxccl: unsupported dtype ", t);
  }
}
hxcclRedOp_t to_op(const ReduceOp& op) {
  switch (op.op_) {
    case ReduceOp::SUM: return hxcclSum;
    case ReduceOp::PRODUCT: return hxcclProd;
    case ReduceOp::MIN: return hxcclMin;
    case ReduceOp::MAX: return hxcclMax;
    case ReduceOp::AVG: return hxcclAvg;
    default: TORCH_CHECK_VALUE(false, "hxccl: unsupported reduce op");
  }
}
void check_tensor(const at::Tensor& t) {
  TORCH_CHECK_VALUE(t.is_contiguous(), "hxccl: tensors must be contiguous");
  TORCH_CHECK_VALUE(t.is_cuda() || t.is_cpu(), "hxccl: tensors must be on a CUDA device or the CPU");
}

// Finished before it is returned (host path).
class DoneWork : public Work {
 public:
  DoneWork(OpType t, std::vector<at::Tensor> out) : Work(-1, t), out_(std::move(out)) {
    fut_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
    fut_->markCompleted(c10::IValue(out_));
  }
  bool isCompleted() override { return true; }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds) override { return true; }
  std::vector<at::Tensor> result() override { return out_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return fut_; }

 private:
  std::vector<at::Tensor> out_;
  c10::intrusive_ptr<c10::ivalue::Future> fut_;
};

// A kernel in flight on the communication stream.
class StreamWork : public Work {
 public:
  StreamWork(OpType t, std::vector<at::Tensor> out, c10::cuda::CUDAStream comm_stream)
      : Work(-1, t), out_(std::move(out)), device_(comm_stream.device()) {
    done_.record(comm_stream);
    fut_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                    std::vector<c10::Device>{device_});
    // completing the future under the communication stream ties its value to that stream:
    // callbacks and wait() synchronize with the kernel, not with the host
    c10::cuda::CUDAStreamGuard g(comm_stream);
    fut_->markCompleted(c10::IValue(out_));
  }
  bool isCompleted() override { return done_.query(); }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds) override {
    done_.block(c10::cuda::getCurrentCUDAStream(device_.index()));
    return true;
  }
  void synchronize() override { done_.block(c10::cuda::getCurrentCUDAStream(device_.index())); }
  std::vector<at::Tensor> result() override { return out_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return fut_; }

 private:
  std::vector<at::Tensor> out_;
  c10::Device device_;
  at::cuda::CUDAEvent done_;
  c10::intrusive_ptr<c10::ivalue::Future> fut_;
};

class HxcclBackend : public Backend {
 public:
  HxcclBackend(const c10::intrusive_ptr<Store>& store, int rank, int size) : Backend(rank, size) {
    // A CUDA context on every rank before the communicator exists lets the library set its
    // device path up collectively right away.
    if (at::cuda::is_available()) {
      device_ = c10::cuda::current_device();
      cudaFree(nullptr);
    }
    hxcclUniqueId id;
    if (rank == 0) {
      ok(hxcclGetUniqueId(&id), "GetUniqueId");
      store->set("hxccl_uid", std::vector<uint8_t>(reinterpret_cast<uint8_t*>(&id),
                                                   reinterpret_cast<uint8_t*>(&id) + sizeof id));
    }
    auto v = store->get("hxccl_uid");
    TORCH_CHECK(v.size() == sizeof id, "hxccl: bad unique id in the store");
    std::memcpy(&id, v.data(), sizeof id);
    ok(hxcclCommInitRank(&comm_, size, id, rank), "CommInitRank");
  }
  ~HxcclBackend() override { shutdown(); }
  void shutdown() override {
    if (comm_) hxcclCommDestroy(comm_);
    comm_ = nullptr;
  }
  void abort() override {
    if (comm_) hxcclCommAbort(comm_);
    comm_ = nullptr;
  }
  const std::string getBackendName() const override { return "hxccl"; }
  hxcclComm_t comm() const { return comm_; }

  // ---- the one pattern every device op follows ------------------------------------------
  template <typename F>
  c10::intrusive_ptr<Work> run(OpType type, const at::Tensor& probe, std::vector<at::Tensor> keep,
                               std::vector<at::Tensor> out, F enqueue) {
    if (!probe.is_cuda()) {
      enqueue(nullptr);
      return c10::make_intrusive<DoneWork>(type, std::move(out));
    }
    c10::cuda::CUDAGuard guard(probe.device());
    auto cur = c10::cuda::getCurrentCUDAStream(probe.device().index());
    auto cs = comm_stream(probe.device().index());
    at::cuda::CUDAEvent ready;
    ready.record(cur);
    ready.block(cs);
    for (const at::Tensor& t : keep)  // the allocator must not hand the memory out while the kernel runs
      c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), cs);
    enqueue(cs.stream());
    if (coalescing_) coalesced_device_ = probe.device().index();  // the batch's Work comes from endCoalescing
    return c10::make_intrusive<StreamWork>(type, std::move(out), cs);
  }

  // ---- collectives ------------------------------------------------------------------------
  c10::intrusive_ptr<Work> allreduce(std::vector<at::Tensor>& ts, const AllreduceOptions& o) override {
    TORCH_CHECK_VALUE(!ts.empty(), "hxccl: no tensor");
    for (auto& t : ts) check_tensor(t);
    const hxcclRedOp_t op = to_op(o.reduceOp);
    return run(OpType::ALLREDUCE, ts[0], ts, ts, [&](hxcclStream_t s) {
      for (auto& t : ts)
        ok(hxcclAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), to_dt(t.scalar_type()), op, comm_, s), "AllReduce");
    });
  }
  // fp32 CUDA tensor reduced in place with fp16 / bf16 on the wire, one kernel (hxcclAllReduceCast)
  c10::intrusive_ptr<Work> allreduce_cast(at::Tensor& t, hxcclDataType_t wire, hxcclRedOp_t op) {
    check_tensor(t);
    TORCH_CHECK_VALUE(t.is_cuda() && t.scalar_type() == at::kFloat, "hxccl: allreduce_cast takes an fp32 CUDA tensor");
    std::vector<at::Tensor> ts{t};
    return run(OpType::ALLREDUCE, t, ts, ts, [&](hxcclStream_t s) {
      ok(hxcclAllReduceCast(t.data_ptr(), t.data_ptr(), t.numel(), wire, op, comm_, s), "AllReduceCast");
    });
  }
  c10::intrusive_ptr<Work> allreduce_coalesced(std::vector<at::Tensor>& ts,
                                               const AllreduceCoalescedOptions& o) override {
    AllreduceOptions ao;
    ao.reduceOp = o.reduceOp;
    return allreduce(ts, ao);
  }
  c10::intrusive_ptr<Work> broadcast(std::vector<at::Tensor>& ts, const BroadcastOptions& o) override {
    TORCH_CHECK_VALUE(!ts.empty(), "hxccl: no tensor");
    for (auto& t : ts) check_tensor(t);
    return run(OpType::BROADCAST, ts[0], ts, ts, [&](hxcclStream_t s) {
      for (auto& t : ts)
        ok(hxcclBroadcast(t.data_ptr(), t.data_ptr(), t.numel(), to_dt(t.scalar_type()), int(o.rootRank), comm_, s),
           "Broadcast");
    });
  }
  c10::intrusive_ptr<Work> reduce(std::vector<at::Tensor>& ts, const ReduceOptions& o) override {
    TORCH_CHECK_VALUE(ts.size() == 1, "hxccl: reduce takes one tensor");
    check_tensor(ts[0]);
    auto& t = ts[0];
    return run(OpType::REDUCE, t, ts, ts, [&](hxcclStream_t s) {
      ok(hxcclReduce(t.data_ptr(), t.data_ptr(), t.numel(), to_dt(t.scalar_type()), to_op(o.reduceOp),
                     int(o.rootRank), comm_, s),
         "Reduce");
    });
  }
  c10::intrusive_ptr<Work> _allgather_base(at::Tensor& out, at::Tensor& in, const AllgatherOptions&) override {
    check_tensor(in);
    check_tensor(out);
    TORCH_CHECK_VALUE(out.numel() == in.numel() * getSize(), "hxccl: output must hold world_size * input elements");
    return run(OpType::_ALLGATHER_BASE, in, {in, out}, {out}, [&](hxcclStream_t s) {
      ok(hxcclAllGather(in.data_ptr(), out.data_ptr(), in.numel(), to_dt(in.scalar_type()), comm_, s), "AllGather");
    });
  }
  c10::intrusive_ptr<Work> allgather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins,
                                     const AllgatherOptions& o) override {
    TORCH_CHECK_VALUE(ins.size() == 1 && outs.size() == 1, "hxccl: allgather takes one input tensor");
    TORCH_CHECK_VALUE(int(outs[0].size()) == getSize(), "hxccl: allgather needs world_size outputs");
    at::Tensor in = ins[0].contiguous();
    at::Tensor flat = at::empty({getSize(), in.numel()}, in.options());
    auto w = _allgather_base(flat, in, o);
    if (in.is_cuda()) {  // the copies below must follow the kernel; they run on the caller's stream
      w->wait();
    }
    for (int r = 0; r < getSize(); ++r) outs[0][r].copy_(flat[r].view_as(outs[0][r]));
    return w;
  }
  c10::intrusive_ptr<Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outs,
                                                           std::vector<at::Tensor>& ins,
                                                           const AllgatherOptions& o) override {
    TORCH_CHECK_VALUE(outs.size() == ins.size() && !ins.empty(), "hxccl: mismatched tensor lists");
    c10::intrusive_ptr<Work> last;
    for (size_t i = 0; i < ins.size(); ++i) last = _allgather_base(outs[i], ins[i], o);
    return last;
  }
  c10::intrusive_ptr<Work> _reduce_scatter_base(at::Tensor& out, at::Tensor& in,
                                                const ReduceScatterOptions& o) override {
    check_tensor(in);
    check_tensor(out);
    TORCH_CHECK_VALUE(in.numel() == out.numel() * getSize(), "hxccl: input must hold world_size * output elements");
    return run(OpType::_REDUCE_SCATTER_BASE, in, {in, out}, {out}, [&](hxcclStream_t s) {
      ok(hxcclReduceScatter(in.data_ptr(), out.data_ptr(), out.numel(), to_dt(in.scalar_type()), to_op(o.reduceOp),
                            comm_, s),
         "ReduceScatter");
    });
  }
  c10::intrusive_ptr<Work> reduce_scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins,
                                          const ReduceScatterOptions& o) override {
    TORCH_CHECK_VALUE(outs.size() == 1 && ins.size() == 1 && int(ins[0].size()) == getSize(),
                      "hxccl: reduce_scatter takes one output and world_size inputs");
    std::vector<at::Tensor> flat_parts;
    for (auto& t : ins[0]) flat_parts.push_back(t.reshape({-1}));
    at::Tensor flat = at::cat(flat_parts).contiguous();
    return _reduce_scatter_base(outs[0], flat, o);
  }
  c10::intrusive_ptr<Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outs,
                                                           std::vector<at::Tensor>& ins,
                                                           const ReduceScatterOptions& o) override {
    TORCH_CHECK_VALUE(outs.size() == ins.size() && !ins.empty(), "hxccl: mismatched tensor lists");
    c10::intrusive_ptr<Work> last;
    for (size_t i = 0; i < ins.size(); ++i) last = _reduce_scatter_base(outs[i], ins[i], o);
    return last;
  }
  c10::intrusive_ptr<Work> alltoall_base(at::Tensor& out, at::Tensor& in, std::vector<int64_t>& out_split,
                                         std::vector<int64_t>& in_split, const AllToAllOptions&) override {
    check_tensor(in);
    check_tensor(out);
    const int n = getSize();
    if (out_split.empty() && in_split.empty()) {
      TORCH_CHECK_VALUE(in.numel() % n == 0 && in.numel() == out.numel(), "hxccl: alltoall sizes must divide evenly");
      return run(OpType::ALLTOALL_BASE, in, {in, out}, {out}, [&](hxcclStream_t s) {
        ok(hxcclAlltoAll(in.data_ptr(), out.data_ptr(), in.numel() / n, to_dt(in.scalar_type()), comm_, s), "AlltoAll");
      });
    }
    TORCH_CHECK_VALUE(int(out_split.size()) == n && int(in_split.size()) == n, "hxccl: split sizes need one entry per rank");
    // splits count rows of dimension 0
    const size_t in_row = in.numel() ? in.numel() / in.size(0) : 0, out_row = out.numel() ? out.numel() / out.size(0) : 0;
    std::vector<size_t> sc(n), sd(n), rc(n), rd(n);
    size_t so = 0, ro = 0;
    for (int r = 0; r < n; ++r) {
      sc[r] = size_t(in_split[r]) * in_row;
      rc[r] = size_t(out_split[r]) * out_row;
      sd[r] = so;
      rd[r] = ro;
      so += sc[r];
      ro += rc[r];
    }
    return run(OpType::ALLTOALL_BASE, in, {in, out}, {out}, [&](hxcclStream_t s) {
      ok(hxcclAllToAllv(in.data_ptr(), sc.data(), sd.data(), out.data_ptr(), rc.data(), rd.data(),
                        to_dt(in.scalar_type()), comm_, s),
         "AllToAllv");
    });
  }
  c10::intrusive_ptr<Work> alltoall(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins,
                                    const AllToAllOptions&) override {
    const int n = getSize();
    TORCH_CHECK_VALUE(int(outs.size()) == n && int(ins.size()) == n, "hxccl: alltoall needs world_size tensors");
    for (auto& t : ins) check_tensor(t);
    for (auto& t : outs) check_tensor(t);
    std::vector<at::Tensor> keep = ins;
    keep.insert(keep.end(), outs.begin(), outs.end());
    return run(OpType::ALLTOALL, ins[0], keep, outs, [&](hxcclStream_t s) {
      ok(hxcclGroupStart(), "GroupStart");
      for (int r = 0; r < n; ++r) {
        ok(hxcclSend(ins[r].data_ptr(), ins[r].numel(), to_dt(ins[r].scalar_type()), r, comm_, s), "Send");
        ok(hxcclRecv(outs[r].data_ptr(), outs[r].numel(), to_dt(outs[r].scalar_type()), r, comm_, s), "Recv");
      }
      ok(hxcclGroupEnd(), "GroupEnd");
    });
  }
  c10::intrusive_ptr<Work> gather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins,
                                  const GatherOptions& o) override {
    TORCH_CHECK_VALUE(ins.size() == 1, "hxccl: gather takes one input tensor");
    at::Tensor in = ins[0].contiguous();
    const bool root = getRank() == int(o.rootRank);
    at::Tensor flat = root ? at::empty({getSize(), in.numel()}, in.options()) : at::Tensor();
    auto w = run(OpType::GATHER, in, root ? std::vector<at::Tensor>{in, flat} : std::vector<at::Tensor>{in},
                 root ? outs[0] : std::vector<at::Tensor>{}, [&](hxcclStream_t s) {
                   ok(hxcclGather(in.data_ptr(), root ? flat.data_ptr() : nullptr, in.numel(), to_dt(in.scalar_type()),
                                  int(o.rootRank), comm_, s),
                      "Gather");
                 });
    if (root) {
      if (in.is_cuda()) w->wait();
      for (int r = 0; r < getSize(); ++r) outs[0][r].copy_(flat[r].view_as(outs[0][r]));
    }
    return w;
  }
  c10::intrusive_ptr<Work> scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins,
                                   const ScatterOptions& o) override {
    TORCH_CHECK_VALUE(outs.size() == 1, "hxccl: scatter takes one output tensor");
    at::Tensor& out = outs[0];
    check_tensor(out);
    const bool root = getRank() == int(o.rootRank);
    at::Tensor flat;
    if (root) {
      std::vector<at::Tensor> parts;
      for (auto& t : ins[0]) parts.push_back(t.reshape({-1}));
      flat = at::cat(parts).contiguous();
    }
    return run(OpType::SCATTER, out, root ? std::vector<at::Tensor>{out, flat} : std::vector<at::Tensor>{out}, {out},
               [&](hxcclStream_t s) {
                 ok(hxcclScatter(root ? flat.data_ptr() : nullptr, out.data_ptr(), out.numel(),
                                 to_dt(out.scalar_type()), int(o.rootRank), comm_, s),
                    "Scatter");
               });
  }
  // The C API has no message tags (neither has NCCL's); Send/Recv toward one peer match in order.
  c10::intrusive_ptr<Work> send(std::vector<at::Tensor>& ts, int dst, int) override {
    check_tensor(ts[0]);
    return run(OpType::SEND, ts[0], ts, ts, [&](hxcclStream_t s) {
      ok(hxcclSend(ts[0].data_ptr(), ts[0].numel(), to_dt(ts[0].scalar_type()), dst, comm_, s), "Send");
    });
  }
  c10::intrusive_ptr<Work> recv(std::vector<at::Tensor>& ts, int src, int) override {
    check_tensor(ts[0]);
    return run(OpType::RECV, ts[0], ts, ts, [&](hxcclStream_t s) {
      ok(hxcclRecv(ts[0].data_ptr(), ts[0].numel(), to_dt(ts[0].scalar_type()), src, comm_, s), "Recv");
    });
  }
  c10::intrusive_ptr<Work> barrier(const BarrierOptions&) override {
    auto opts = at::TensorOptions().dtype(at::kInt);
    auto t = at::zeros({1}, device_ >= 0 ? opts.device(at::Device(at::kCUDA, device_)) : opts);
    std::vector<at::Tensor> v{t};
    auto w = allreduce(v, AllreduceOptions());
    if (t.is_cuda()) {  // a barrier holds the host too
      w->wait();
      c10::cuda::getCurrentCUDAStream(device_).synchronize();
    }
    return w;
  }
  // Coalescing = one hxccl group: the calls between start and end are queued and run at the
  // end, collectives first, then all Send/Recv together (on GPUs in one kernel, so that
  // dist.batch_isend_irecv cannot stall on its own order). The Work of the whole batch is
  // recorded on the communication stream after the group has been launched.
  void startCoalescing() override {
    ok(hxcclGroupStart(), "GroupStart");
    coalescing_ = true;
    coalesced_device_ = -1;
  }
  c10::intrusive_ptr<Work> endCoalescing() override {
    coalescing_ = false;
    ok(hxcclGroupEnd(), "GroupEnd");
    if (coalesced_device_ >= 0)
      return c10::make_intrusive<StreamWork>(OpType::COALESCED, std::vector<at::Tensor>{},
                                             comm_stream(coalesced_device_));
    return c10::make_intrusive<DoneWork>(OpType::COALESCED, std::vector<at::Tensor>{});
  }
  // Advertised where it has been exercised: process groups without a GPU always, with a GPU
  // when HXCCL_TORCH_COALESCE=1 asks for it.
  bool supportsCoalescing() const override {
    if (device_ < 0) return true;
    const char* e = std::getenv("HXCCL_TORCH_COALESCE");
    return e && *e == '1';
  }

 private:
  void ok(hxcclResult_t r, const char* what) const {
    TORCH_CHECK(r == hxcclSuccess, "hxccl ", what, " failed (", int(r), ", ", hxcclGetErrorString(r),
                "): ", comm_ ? hxcclGetLastError(comm_) : "");
  }
  c10::cuda::CUDAStream comm_stream(c10::DeviceIndex dev) {
    if (!stream_ || stream_->device_index() != dev)
      stream_ = c10::cuda::getStreamFromPool(/*isHighPriority=*/true, dev);
    return *stream_;
  }
  hxcclComm_t comm_ = nullptr;
  c10::DeviceIndex device_ = -1;
  bool coalescing_ = false;
  c10::DeviceIndex coalesced_device_ = -1;
  std::optional<c10::cuda::CUDAStream> stream_;
};

c10::intrusive_ptr<Backend> create_backend(const c10::intrusive_ptr<Store>& store, int rank, int size,
                                           const std::chrono::duration<float>&) {
  return c10::make_intrusive<HxcclBackend>(store, rank, size);
}

// hxcclCommTune / hxcclCommDeviceInfo for the communicator behind a backend object
void tune(const c10::intrusive_ptr<Backend>& b, int variant, int exact, int max_ctas) {
  auto* h = dynamic_cast<HxcclBackend*>(b.get());
  TORCH_CHECK(h, "not an hxccl backend");
  hxcclCommTune(h->comm(), variant, exact, max_ctas);
}
std::tuple<std::string, int, unsigned long long> device_info(const c10::intrusive_ptr<Backend>& b) {
  auto* h = dynamic_cast<HxcclBackend*>(b.get());
  TORCH_CHECK(h, "not an hxccl backend");
  char kind[32];
  int variant = 0;
  unsigned long long launches = 0;
  hxcclCommDeviceInfo(h->comm(), kind, sizeof kind, &variant, &launches);
  return {kind, variant, launches};
}
c10::intrusive_ptr<Work> allreduce_cast(const c10::intrusive_ptr<Backend>& b, at::Tensor t, bool bf16, bool average) {
  auto* h = dynamic_cast<HxcclBackend*>(b.get());
  TORCH_CHECK(h, "not an hxccl backend");
  return h->allreduce_cast(t, bf16 ? hxcclBfloat16 : hxcclFloat16, average ? hxcclAvg : hxcclSum);
}
}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("allreduce_cast", &allreduce_cast);
  m.def("create_backend", &create_backend);
  m.def("tune", &tune);
  m.def("device_info", &device_info);
}
