// Fallback device path: device buffers are copied to host memory, the host algorithms run over
// the control mesh, and the result is copied back. Slow, but it needs nothing from the GPUs
// beyond cudaMemcpy, so it works when windows cannot be shared (ranks on several machines or
// on one GPU, no file-descriptor handles, HXCCL_DEVICE_TRANSPORT=staged). It mirrors the
// reference's staged transport (src/transport_ipc.cc:224-325), at the granularity of whole
// collectives instead of single messages. Calls complete before they return.
#include <cuda_runtime.h>

#include <cstring>
#include <vector>

#include "core/comm.h"
#include "host/algos.h"
#include "math/reduce_host.h"

namespace hx {
namespace {

// The host wire counts what the staged path sends, and the API layer books the same call on
// the device counters; this puts the host counters back when a call ends.
struct KeepHostCounters {
  explicit KeepHostCounters(hxcclComm* c) : w(*c->wire), b(w.bytes_sent), m(w.msgs_sent) {}
  ~KeepHostCounters() {
    w.bytes_sent = b;
    w.msgs_sent = m;
  }
  HostWire& w;
  uint64_t b, m;
};

class StagedPath : public DevicePath {
 public:
  explicit StagedPath(hxcclComm* c) : c_(c) { cudaGetDevice(&dev_); }
  hxcclResult_t broken(std::string* why) override {
    if (broken_ != hxcclSuccess && why) *why = error;
    return broken_;
  }
  const char* kind() const override { return "staged"; }

  hxcclResult_t allreduce(const void* send, void* recv, size_t count, int dt, const OpPlan& plan,
                          int order, void* stream) override {
    KeepHostCounters keep(c_);
    const size_t bytes = count * dtype_size(dt);
    std::vector<char> in, out(bytes);
    HostPlan hp;
    if (hxcclResult_t r = fetch(send, bytes, stream, &in)) return r;
    if (hxcclResult_t r = resolve(plan, dt, stream, &hp)) return r;
    premul(hp, in, count, dt);
    hxcclResult_t r = order == kOrderRing ? host_allreduce_ring(ctx(), in.data(), out.data(), count, dt, hp.base)
                                          : host_allreduce_doubling(ctx(), in.data(), out.data(), count, dt, hp.base);
    if (r == hxcclSuccess && hp.postdiv && count) divide_trunc(out.data(), count, dt, hp.divisor);
    return finish(r, recv, out, bytes, stream);
  }
  hxcclResult_t allgather(const void* send, void* recv, size_t block, void* stream) override {
    KeepHostCounters keep(c_);
    std::vector<char> in, out(block * c_->nranks);
    if (hxcclResult_t r = fetch(send, block, stream, &in)) return r;
    return finish(host_allgather(ctx(), in.data(), out.data(), block), recv, out, out.size(), stream);
  }
  hxcclResult_t reducescatter(const void* send, void* recv, size_t per, int dt, const OpPlan& plan,
                              void* stream) override {
    KeepHostCounters keep(c_);
    const size_t block = per * dtype_size(dt);
    std::vector<char> in, out(block);
    HostPlan hp;
    if (hxcclResult_t r = fetch(send, block * c_->nranks, stream, &in)) return r;
    if (hxcclResult_t r = resolve(plan, dt, stream, &hp)) return r;
    premul(hp, in, per * c_->nranks, dt);
    hxcclResult_t r = host_reducescatter(ctx(), in.data(), out.data(), per, dt, hp.base);
    if (r == hxcclSuccess && hp.postdiv && per) divide_trunc(out.data(), per, dt, hp.divisor);
    return finish(r, recv, out, block, stream);
  }
  hxcclResult_t broadcast(const void* send, void* recv, size_t bytes, int root, void* stream) override {
    KeepHostCounters keep(c_);
    std::vector<char> buf(bytes);
    if (c_->rank == root)
      if (hxcclResult_t r = fetch(send, bytes, stream, &buf)) return r;
    return finish(host_broadcast(ctx(), buf.data(), buf.data(), bytes, root), recv, buf, bytes, stream);
  }
  hxcclResult_t reduce(const void* send, void* recv, size_t count, int dt, const OpPlan& plan,
                       int root, void* stream) override {
    KeepHostCounters keep(c_);
    const size_t bytes = count * dtype_size(dt);
    std::vector<char> in, out(bytes);
    HostPlan hp;
    if (hxcclResult_t r = fetch(send, bytes, stream, &in)) return r;
    if (hxcclResult_t r = resolve(plan, dt, stream, &hp)) return r;
    premul(hp, in, count, dt);
    hxcclResult_t r = host_reduce(ctx(), in.data(), out.data(), count, dt, hp.base, root);
    if (c_->rank != root) return finish(r, nullptr, out, 0, stream);
    if (r == hxcclSuccess && hp.postdiv && count) divide_trunc(out.data(), count, dt, hp.divisor);
    return finish(r, recv, out, bytes, stream);
  }
  hxcclResult_t gather(const void* send, void* recv, size_t block, int root, void* stream) override {
    KeepHostCounters keep(c_);
    std::vector<char> in, out(c_->rank == root ? block * c_->nranks : 0);
    if (hxcclResult_t r = fetch(send, block, stream, &in)) return r;
    return finish(host_gather(ctx(), in.data(), out.data(), block, root), c_->rank == root ? recv : nullptr, out,
                  out.size(), stream);
  }
  hxcclResult_t scatter(const void* send, void* recv, size_t block, int root, void* stream) override {
    KeepHostCounters keep(c_);
    std::vector<char> in, out(block);
    if (c_->rank == root)
      if (hxcclResult_t r = fetch(send, block * c_->nranks, stream, &in)) return r;
    return finish(host_scatter(ctx(), in.data(), out.data(), block, root), recv, out, block, stream);
  }
  hxcclResult_t alltoallv(const char* send, const size_t* sbytes, const size_t* soff, char* recv,
                          const size_t* rbytes, const size_t* roff, size_t, void* stream) override {
    KeepHostCounters keep(c_);
    size_t send_end = 0, recv_end = 0;
    for (int j = 0; j < c_->nranks; ++j) {
      if (sbytes[j]) send_end = std::max(send_end, soff[j] + sbytes[j]);
      if (rbytes[j]) recv_end = std::max(recv_end, roff[j] + rbytes[j]);
    }
    std::vector<char> in, out;
    if (hxcclResult_t r = fetch(send, send_end, stream, &in)) return r;
    if (hxcclResult_t r = fetch(recv, recv_end, stream, &out)) return r;  // gaps keep their contents
    return finish(host_alltoallv(ctx(), in.data(), sbytes, soff, out.data(), rbytes, roff), recv, out, recv_end, stream);
  }
  hxcclResult_t p2p_batch(const std::vector<P2pOp>& ops, void* stream) override {
    KeepHostCounters keep(c_);
    std::vector<std::vector<char>> bufs(ops.size());
    for (size_t i = 0; i < ops.size(); ++i) {
      if (ops[i].is_send) {
        if (hxcclResult_t r = fetch(ops[i].buf, ops[i].bytes, stream, &bufs[i])) return r;
        if (hxcclResult_t r = c_->wire->post_send(ops[i].peer, bufs[i].data(), ops[i].bytes, kTagP2p)) {
          c_->wire->cancel_all();
          return lose(r, c_->wire->error);
        }
      } else {
        bufs[i].resize(ops[i].bytes);
        c_->wire->post_recv(ops[i].peer, bufs[i].data(), ops[i].bytes, kTagP2p);
      }
    }
    const hxcclResult_t r = c_->wire->finish_all();
    // deliver what arrived even when some transfer failed (a truncated receive keeps its prefix)
    for (size_t i = 0; i < ops.size(); ++i)
      if (!ops[i].is_send && ops[i].bytes)
        cudaMemcpy(ops[i].buf, bufs[i].data(), ops[i].bytes, cudaMemcpyHostToDevice);
    if (r != hxcclSuccess) {
      error = c_->wire->error;
      return r;  // a failed message does not break the path
    }
    return hxcclSuccess;
  }
  hxcclResult_t drain() override { return hxcclSuccess; }

 private:
  struct HostPlan {
    int base;
    bool premul, postdiv;
    int divisor;
    unsigned char scalar[8];
  };
  HostCtx ctx() { return HostCtx{*c_->wire, c_->rank, c_->nranks}; }
  hxcclResult_t lose(hxcclResult_t r, const std::string& why) {
    error = why;
    if (r == hxcclUnhandledCudaError) broken_ = r;
    return r;
  }
  hxcclResult_t fetch(const void* dev, size_t bytes, void* stream, std::vector<char>* out) {
    out->resize(bytes);
    cudaSetDevice(dev_);
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess && bytes) e = cudaMemcpy(out->data(), dev, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess || std::getenv("HXCCL_TEST_FAIL_DEVICE_COPY"))
      return lose(hxcclUnhandledCudaError, std::string("copying device data to the host: ") +
                                               (e ? cudaGetErrorString(e) : "injected failure"));
    return hxcclSuccess;
  }
  hxcclResult_t resolve(const OpPlan& p, int dt, void* stream, HostPlan* hp) {
    hp->base = p.base;
    hp->premul = p.premul;
    hp->postdiv = p.postdiv;
    hp->divisor = p.divisor;
    std::memcpy(hp->scalar, p.scalar, 8);
    if (p.premul && p.scalar_dev) {
      std::vector<char> tmp;
      if (hxcclResult_t r = fetch(p.scalar_dev, dtype_size(dt), stream, &tmp)) return r;
      std::memcpy(hp->scalar, tmp.data(), tmp.size());
    }
    return hxcclSuccess;
  }
  static void premul(const HostPlan& hp, std::vector<char>& buf, size_t count, int dt) {
    if (hp.premul && count) scale_into(buf.data(), buf.data(), count, dt, hp.scalar);
  }
  hxcclResult_t finish(hxcclResult_t r, void* recv, const std::vector<char>& out, size_t bytes, void*) {
    if (r != hxcclSuccess) {
      error = c_->wire->error;
      if (r != hxcclInvalidArgument) broken_ = r;
      return r;
    }
    if (recv && bytes && cudaMemcpy(recv, out.data(), bytes, cudaMemcpyHostToDevice) != cudaSuccess)
      return lose(hxcclUnhandledCudaError, "copying the result to the device failed");
    return hxcclSuccess;
  }

  hxcclComm* c_;
  int dev_ = 0;
  hxcclResult_t broken_ = hxcclSuccess;
};

}  // namespace

std::unique_ptr<DevicePath> make_staged_path(hxcclComm* c) { return std::make_unique<StagedPath>(c); }

}  // namespace hx
