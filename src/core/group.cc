#include "core/group.h"

#include <algorithm>
#include <utility>

#include "core/trace.h"

namespace hx {
namespace {

struct QueuedP2p {
  hxcclComm* c;
  Path path;
  P2pOp op;
  void* stream;
};
struct OpenGroup {
  int depth = 0;
  std::vector<Deferred> collectives;
  std::vector<QueuedP2p> p2p;
};
thread_local OpenGroup tl_group;

// Host Send/Recv: post every transfer before waiting for any, then advance all communicators
// involved in one loop; blocking on one while a peer blocks on another would deadlock.
hxcclResult_t run_host_p2p(const std::vector<QueuedP2p>& ops) {
  std::vector<hxcclComm*> comms;
  for (const QueuedP2p& q : ops) {
    if (std::find(comms.begin(), comms.end(), q.c) == comms.end()) comms.push_back(q.c);
    HostWire& w = *q.c->wire;
    const hxcclResult_t r = q.op.is_send ? w.post_send(q.op.peer, q.op.buf, q.op.bytes, kTagP2p)
                                         : w.post_recv(q.op.peer, q.op.buf, q.op.bytes, kTagP2p);
    if (r != hxcclSuccess) {
      for (hxcclComm* c : comms) c->wire->cancel_all();
      return comm_fail(q.c, r, w.error);
    }
  }
  hxcclResult_t first = hxcclSuccess;
  std::vector<bool> fin(comms.size(), false);
  for (size_t left = comms.size(); left > 0;) {
    for (size_t i = 0; i < comms.size(); ++i) {
      if (fin[i]) continue;
      bool done = false;
      const hxcclResult_t r = comms[i]->wire->step(&done);
      if (!done) continue;
      fin[i] = true;
      --left;
      // a failure on one communicator must not strand the transfers of the others
      if (r != hxcclSuccess && first == hxcclSuccess)
        first = comm_fail(comms[i], r, comms[i]->wire->error);
    }
  }
  return first;
}

// Device Send/Recv: one fused peer-copy launch per communicator. The launches of a group are
// serialised on a stream and each one waits for its peers' kernels, so every rank must issue
// them in the same order whatever order its calls named the communicators in (rank 0: Send on
// c1, Recv on c2; rank 1: Send on c2, Recv on c1 - the crossed case of the reference's
// tests/repro_two_comm_group.cc). The channel id is the same on every member of a communicator,
// which makes it a rank-independent sort key.
hxcclResult_t run_device_p2p(const std::vector<QueuedP2p>& ops) {
  std::vector<hxcclComm*> comms;
  for (const QueuedP2p& q : ops)
    if (std::find(comms.begin(), comms.end(), q.c) == comms.end()) comms.push_back(q.c);
  std::stable_sort(comms.begin(), comms.end(),
                   [](const hxcclComm* a, const hxcclComm* b) { return a->chan->id() < b->chan->id(); });
  hxcclResult_t first = hxcclSuccess;
  for (hxcclComm* c : comms) {
    std::vector<P2pOp> mine;
    void* stream = nullptr;
    bool have_stream = false;
    for (const QueuedP2p& q : ops)
      if (q.c == c) {
        mine.push_back(q.op);
        if (!have_stream) stream = q.stream, have_stream = true;
        if (q.op.is_send) {
          c->device.bytes += q.op.bytes;
          ++c->device.msgs;
        }
      }
    const hxcclResult_t r = c->device.path->p2p_batch(mine, stream);
    if (r != hxcclSuccess && first == hxcclSuccess) first = comm_fail(c, r, c->device.path->error);
  }
  return first;
}

hxcclResult_t run_p2p(const std::vector<QueuedP2p>& ops) {
  const bool any_host =
      std::any_of(ops.begin(), ops.end(), [](const QueuedP2p& q) { return q.path == Path::Host; });
  const bool any_dev = std::any_of(ops.begin(), ops.end(),
                                   [](const QueuedP2p& q) { return q.path == Path::Device; });
  if (any_host && any_dev)
    return comm_fail(ops.front().c, hxcclInvalidUsage,
                     "a group cannot mix host and device Send/Recv buffers");
  TraceRange range("hxccl:p2p");
  return any_dev ? run_device_p2p(ops) : run_host_p2p(ops);
}

}  // namespace

hxcclResult_t dispatch(hxcclComm*, Deferred work) {
  if (tl_group.depth == 0) return work();
  tl_group.collectives.push_back(std::move(work));
  return hxcclSuccess;
}

hxcclResult_t submit_p2p(hxcclComm* c, Path path, bool is_send, int peer, void* buf,
                         size_t bytes, void* stream) {
  QueuedP2p q{c, path, P2pOp{is_send, peer, buf, bytes}, stream};
  if (tl_group.depth == 0) return run_p2p({q});
  tl_group.p2p.push_back(q);
  return hxcclSuccess;
}

}  // namespace hx

extern "C" {

hxcclResult_t hxcclGroupStart(void) {
  ++hx::tl_group.depth;
  return hxcclSuccess;
}

hxcclResult_t hxcclGroupEnd(void) {
  hx::OpenGroup& g = hx::tl_group;
  if (g.depth == 0) return hxcclInvalidUsage;
  if (--g.depth > 0) return hxcclSuccess;
  std::vector<hx::Deferred> colls;
  std::vector<hx::QueuedP2p> p2p;
  colls.swap(g.collectives);
  p2p.swap(g.p2p);
  for (hx::Deferred& work : colls)  // collectives first, in call order
    if (hxcclResult_t r = work()) return r;
  return p2p.empty() ? hxcclSuccess : hx::run_p2p(p2p);
}

}  // extern "C"
