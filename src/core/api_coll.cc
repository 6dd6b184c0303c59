// Collective entry points: argument checks, operator planning, data-path choice, then either
// the host algorithm (runs to completion) or one kernel launch on the caller's stream.
// (Reference entry points: src/api.cc:15-81, src/api_rooted.cc:21-79, src/api_alltoall.cc:15-112.)
#include <algorithm>
#include <climits>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <vector>

#include "core/comm.h"
#include "core/group.h"
#include "core/trace.h"
#include "core/traffic.h"
#include "host/algos.h"
#include "math/reduce_host.h"

namespace hx {

// Which reduction order an AllReduce of `bytes` uses: recursive doubling below 64 KiB, ring
// from there on; HXCCL_ALGO=ring|rd forces one (reference: src/select.cc:10-16). The device
// path replays the same order whatever kernel variant moves the data.
int choose_order(size_t bytes) {
  if (const char* e = std::getenv("HXCCL_ALGO")) {
    if (std::strcmp(e, "ring") == 0) return kOrderRing;
    if (std::strcmp(e, "rd") == 0) return kOrderDoubling;
  }
  return bytes < kDoublingMaxBytes ? kOrderDoubling : kOrderRing;
}

namespace {

hxcclResult_t host_done(hxcclComm* c, hxcclResult_t r) {
  return r == hxcclSuccess ? r : comm_fail(c, r, c->wire->error);
}
hxcclResult_t dev_done(hxcclComm* c, hxcclResult_t r, Traffic t) {
  if (r != hxcclSuccess) return comm_fail(c, r, c->device.path->error);
  c->device.bytes += t.bytes;
  c->device.msgs += t.msgs;
  return r;
}
HostCtx ctx(hxcclComm* c) { return HostCtx{*c->wire, c->rank, c->nranks}; }

// input * scalar into `tmp` when the plan asks for it; returns the buffer to reduce from.
// `tmp` is written before it is read, so it is not cleared.
using HostTmp = std::unique_ptr<char[]>;
const void* host_premul(const OpPlan& p, const void* send, size_t count, int dt, HostTmp& tmp) {
  if (!p.premul || count == 0) return send;
  tmp.reset(new char[count * dtype_size(dt)]);
  scale_into(tmp.get(), send, count, dt, p.scalar);
  return tmp.get();
}
void host_finish(const OpPlan& p, void* buf, size_t count, int dt) {
  if (p.postdiv && count) divide_trunc(buf, count, dt, p.divisor);
}

hxcclResult_t check_root(hxcclComm* c, int root) {
  return root >= 0 && root < c->nranks ? hxcclSuccess
                                       : comm_fail(c, hxcclInvalidArgument, "root out of range");
}

// 0 fine, 1 invalid argument, 2 a block beyond the host transport's message limit
int alltoallv_local_status(const hxcclComm* c, const void* send, const size_t* sc,
                           const size_t* sd, const void* recv, const size_t* rc,
                           const size_t* rd, size_t es) {
  if (es == 0 || !sc || !sd || !rc || !rd) return 1;
  int status = 0;
  for (int j = 0; j < c->nranks; ++j) {
    if (sc[j] > SIZE_MAX / es || rc[j] > SIZE_MAX / es) return 1;
    if (sc[j] * es > size_t(INT_MAX) || rc[j] * es > size_t(INT_MAX)) status = 2;
    if (sd[j] > SIZE_MAX / es - sc[j] || rd[j] > SIZE_MAX / es - rc[j]) return 1;
    if ((sc[j] && !send) || (rc[j] && !recv)) return 1;
  }
  return status;
}

size_t reach(const std::vector<size_t>& bytes, const std::vector<size_t>& off) {
  size_t end = 0;
  for (size_t j = 0; j < bytes.size(); ++j)
    if (bytes[j]) end = std::max(end, off[j] + bytes[j]);
  return end;
}

hxcclResult_t run_alltoallv(hxcclComm* c, Path path, void* stream, const char* send,
                            const std::vector<size_t>& sb, const std::vector<size_t>& so,
                            char* recv, const std::vector<size_t>& rb,
                            const std::vector<size_t>& ro, size_t max_pair) {
  TraceRange range("hxccl:alltoall");
  if (path == Path::Device)  // the kernel stages through the windows, so overlap is harmless
    return dev_done(c,
                    c->device.path->alltoallv(send, sb.data(), so.data(), recv, rb.data(), ro.data(),
                                      max_pair, stream),
                    traffic_alltoallv(c->rank, c->nranks, sb.data()));
  // in-place or overlapping buffers: the exchange would overwrite blocks not yet sent
  const size_t send_end = reach(sb, so), recv_end = reach(rb, ro);
  const bool overlap = send_end && recv_end && send < recv + recv_end && recv < send + send_end;
  std::vector<char> stage;
  if (overlap) {
    stage.assign(send, send + send_end);
    send = stage.data();
  }
  return host_done(c, host_alltoallv(ctx(c), send, sb.data(), so.data(), recv, rb.data(), ro.data()));
}

}  // namespace
}  // namespace hx

using namespace hx;

extern "C" {

hxcclResult_t hxcclAllReduce(const void* send, void* recv, size_t count, hxcclDataType_t dt,
                             hxcclRedOp_t op, hxcclComm_t c, hxcclStream_t stream) {
  if (hxcclResult_t r = check_args(c, send, recv, count, 1, dt)) return r;
  OpPlan plan;
  if (hxcclResult_t r = plan_op(c, op, dt, &plan)) return r;
  const size_t es = dtype_size(dt);
  const int order = choose_order(count * es);
  Path path;
  if (hxcclResult_t r = pick_path(c, send, recv, &path)) return r;
  if (path == Path::Host) {
    const size_t largest =
        order == kOrderRing ? ring_block(count, c->nranks, 0).len * es : count * es;
    if (hxcclResult_t r = check_message(c, largest)) return r;
  }
  return dispatch(c, [=] {
    TraceRange range("hxccl:allreduce");
    if (path == Path::Device)
      return dev_done(c, c->device.path->allreduce(send, recv, count, dt, plan, order, stream),
                      traffic_allreduce(order, c->rank, c->nranks, count, es));
    // the scaled input of an AllReduce can live in the result buffer: the algorithms work in
    // place (unless the two buffers overlap without being equal)
    HostTmp tmp;
    const void* in = send;
    const char* s0 = static_cast<const char*>(send);
    char* r0 = static_cast<char*>(recv);
    const bool apart = s0 == r0 || s0 + count * es <= r0 || r0 + count * es <= s0;
    if (plan.premul && count && apart) {
      scale_into(recv, send, count, dt, plan.scalar);
      in = recv;
    } else {
      in = host_premul(plan, send, count, dt, tmp);
    }
    hxcclResult_t r = order == kOrderRing
                          ? host_allreduce_ring(ctx(c), in, recv, count, dt, plan.base)
                          : host_allreduce_doubling(ctx(c), in, recv, count, dt, plan.base);
    if (r == hxcclSuccess) host_finish(plan, recv, count, dt);
    return host_done(c, r);
  });
}

// An extension (include/hxccl_ext.h): fp32 device buffers, a 16-bit float type on the wire.
hxcclResult_t hxcclAllReduceCast(const void* send, void* recv, size_t count, hxcclDataType_t wire_dt,
                                 hxcclRedOp_t op, hxcclComm_t c, hxcclStream_t stream) {
  if (hxcclResult_t r = check_args(c, send, recv, count, 1, hxcclFloat32)) return r;
  if (wire_dt != hxcclFloat16 && wire_dt != hxcclBfloat16)
    return comm_fail(c, hxcclInvalidArgument, "the wire type must be hxcclFloat16 or hxcclBfloat16");
  OpPlan plan;
  if (hxcclResult_t r = plan_op(c, op, wire_dt, &plan)) return r;
  const size_t es = dtype_size(wire_dt);
  if (choose_order(count * es) != kOrderRing)
    return comm_fail(c, hxcclInvalidUsage, "the fused cast AllReduce needs a message that takes the ring order");
  Path path;
  if (hxcclResult_t r = pick_path(c, send, recv, &path)) return r;
  if (path != Path::Device) return comm_fail(c, hxcclInvalidUsage, "the fused cast AllReduce is for device buffers");
  return dispatch(c, [=] {
    TraceRange range("hxccl:allreduce_cast");
    const hxcclResult_t r = c->device.path->allreduce_cast(send, recv, count, wire_dt, plan, stream);
    if (r == hxcclInvalidUsage) return comm_fail(c, r, c->device.path->error);  // not offered here: no failure state
    return dev_done(c, r, traffic_allreduce(kOrderRing, c->rank, c->nranks, count, es));
  });
}

hxcclResult_t hxcclAllGather(const void* send, void* recv, size_t sendcount, hxcclDataType_t dt,
                             hxcclComm_t c, hxcclStream_t stream) {
  if (hxcclResult_t r = check_args(c, send, recv, sendcount, c ? c->nranks : 1, dt)) return r;
  const size_t block = sendcount * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, send, recv, &path)) return r;
  if (path == Path::Host)
    if (hxcclResult_t r = check_message(c, block)) return r;
  return dispatch(c, [=] {
    TraceRange range("hxccl:allgather");
    if (path == Path::Device)
      return dev_done(c, c->device.path->allgather(send, recv, block, stream),
                      traffic_ring_blocks(c->nranks, block));
    return host_done(c, host_allgather(ctx(c), send, recv, block));
  });
}

hxcclResult_t hxcclReduceScatter(const void* send, void* recv, size_t recvcount,
                                 hxcclDataType_t dt, hxcclRedOp_t op, hxcclComm_t c,
                                 hxcclStream_t stream) {
  if (hxcclResult_t r = check_args(c, send, recv, recvcount, c ? c->nranks : 1, dt)) return r;
  OpPlan plan;
  if (hxcclResult_t r = plan_op(c, op, dt, &plan)) return r;
  const size_t block = recvcount * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, send, recv, &path)) return r;
  if (path == Path::Host)
    if (hxcclResult_t r = check_message(c, block)) return r;
  return dispatch(c, [=] {
    TraceRange range("hxccl:reducescatter");
    if (path == Path::Device)
      return dev_done(c, c->device.path->reducescatter(send, recv, recvcount, dt, plan, stream),
                      traffic_ring_blocks(c->nranks, block));
    HostTmp tmp;
    const void* in = host_premul(plan, send, recvcount * c->nranks, dt, tmp);
    hxcclResult_t r = host_reducescatter(ctx(c), in, recv, recvcount, dt, plan.base);
    if (r == hxcclSuccess) host_finish(plan, recv, recvcount, dt);
    return host_done(c, r);
  });
}

hxcclResult_t hxcclBroadcast(const void* send, void* recv, size_t count, hxcclDataType_t dt,
                             int root, hxcclComm_t c, hxcclStream_t stream) {
  // only the root reads `send`
  if (hxcclResult_t r = check_args(c, c && c->rank == root ? send : recv, recv, count, 1, dt))
    return r;
  if (hxcclResult_t r = check_root(c, root)) return r;
  const size_t bytes = count * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, c->rank == root ? send : nullptr, recv, &path)) return r;
  return dispatch(c, [=] {
    TraceRange range("hxccl:broadcast");
    if (path == Path::Device)
      return dev_done(c, c->device.path->broadcast(send, recv, bytes, root, stream),
                      traffic_broadcast(c->rank, c->nranks, bytes, root));
    return host_done(c, host_broadcast(ctx(c), send, recv, bytes, root));
  });
}

hxcclResult_t hxcclBcast(void* buff, size_t count, hxcclDataType_t dt, int root, hxcclComm_t c,
                         hxcclStream_t stream) {
  return hxcclBroadcast(buff, buff, count, dt, root, c, stream);
}

hxcclResult_t hxcclReduce(const void* send, void* recv, size_t count, hxcclDataType_t dt,
                          hxcclRedOp_t op, int root, hxcclComm_t c, hxcclStream_t stream) {
  if (!c) return hxcclInvalidArgument;
  if (hxcclResult_t r = check_root(c, root)) return r;
  const bool is_root = c->rank == root;
  if (hxcclResult_t r = check_args(c, send, is_root ? recv : send, count, 1, dt)) return r;
  OpPlan plan;
  if (hxcclResult_t r = plan_op(c, op, dt, &plan)) return r;
  const size_t bytes = count * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, send, is_root ? recv : nullptr, &path)) return r;
  if (path == Path::Host)
    if (hxcclResult_t r = check_message(c, bytes < kTreeMaxBytes ? bytes : kChainPiece)) return r;
  return dispatch(c, [=] {
    TraceRange range("hxccl:reduce");
    if (path == Path::Device)
      return dev_done(c, c->device.path->reduce(send, recv, count, dt, plan, root, stream),
                      traffic_reduce(c->rank, c->nranks, bytes, root));
    HostTmp tmp;
    const void* in = host_premul(plan, send, count, dt, tmp);
    hxcclResult_t r = host_reduce(ctx(c), in, recv, count, dt, plan.base, root);
    if (r == hxcclSuccess && is_root) host_finish(plan, recv, count, dt);  // divide once
    return host_done(c, r);
  });
}

hxcclResult_t hxcclGather(const void* send, void* recv, size_t count, hxcclDataType_t dt,
                          int root, hxcclComm_t c, hxcclStream_t stream) {
  if (!c) return hxcclInvalidArgument;
  if (hxcclResult_t r = check_root(c, root)) return r;
  const bool is_root = c->rank == root;
  if (hxcclResult_t r = check_args(c, send, is_root ? recv : send, count, c->nranks, dt))
    return r;
  const size_t block = count * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, send, is_root ? recv : nullptr, &path)) return r;
  if (path == Path::Host)
    if (hxcclResult_t r = check_message(c, block)) return r;
  return dispatch(c, [=] {
    TraceRange range("hxccl:gather");
    if (path == Path::Device)
      return dev_done(c, c->device.path->gather(send, recv, block, root, stream),
                      traffic_gather(c->rank, c->nranks, block, root));
    return host_done(c, host_gather(ctx(c), send, recv, block, root));
  });
}

hxcclResult_t hxcclScatter(const void* send, void* recv, size_t count, hxcclDataType_t dt,
                           int root, hxcclComm_t c, hxcclStream_t stream) {
  if (!c) return hxcclInvalidArgument;
  if (hxcclResult_t r = check_root(c, root)) return r;
  const bool is_root = c->rank == root;
  if (hxcclResult_t r = check_args(c, is_root ? send : recv, recv, count, c->nranks, dt))
    return r;
  const size_t block = count * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, is_root ? send : nullptr, recv, &path)) return r;
  if (path == Path::Host)
    if (hxcclResult_t r = check_message(c, block)) return r;
  return dispatch(c, [=] {
    TraceRange range("hxccl:scatter");
    if (path == Path::Device)
      return dev_done(c, c->device.path->scatter(send, recv, block, root, stream),
                      traffic_scatter(c->rank, c->nranks, block, root));
    return host_done(c, host_scatter(ctx(c), send, recv, block, root));
  });
}

// Block sizes differ per rank, so one rank cannot see another's bad block: every rank shares
// its local verdict (and its largest block, which sizes the device launch) first and all of
// them accept or reject together.
hxcclResult_t hxcclAllToAllv(const void* send, const size_t sc[], const size_t sd[], void* recv,
                             const size_t rc[], const size_t rd[], hxcclDataType_t dt,
                             hxcclComm_t c, hxcclStream_t stream) {
  if (!c) return hxcclInvalidArgument;
  if (c->closed) return comm_fail(c, hxcclInvalidUsage, "communicator was finalized");
  const size_t es = dtype_size(dt);
  struct Verdict {
    uint64_t status, largest;
  } mine{0, 0};
  mine.status = alltoallv_local_status(c, send, sc, sd, recv, rc, rd, es);
  if (mine.status != 1) {
    const MemKind ks = classify(send), kr = classify(recv);
    if (ks != MemKind::Null && kr != MemKind::Null && ks != kr) mine.status = 1;
  }
  if (mine.status != 1)
    for (int j = 0; j < c->nranks; ++j) mine.largest = std::max<uint64_t>(mine.largest, sc[j] * es);
  std::vector<Verdict> all(c->nranks);
  if (c->chan->allgather(&mine, all.data(), sizeof mine) != hxcclSuccess)
    return comm_fail(c, hxcclSystemError,
                     "the AllToAllv argument check failed: " + c->chan->error);
  uint64_t status = 0, largest = 0;
  for (const Verdict& v : all) {
    status = std::max(status, v.status == 1 ? uint64_t(3) : v.status);  // invalid beats too-big
    largest = std::max(largest, v.largest);
  }
  if (status == 3)
    return comm_fail(c, hxcclInvalidArgument, "invalid AllToAllv arguments on some rank");
  Path path;
  if (hxcclResult_t r = pick_path(c, send, recv, &path)) return r;
  if (status == 2 && path == Path::Host)
    return comm_fail(c, hxcclInvalidArgument,
                     "a single message would exceed INT_MAX bytes (host transport limit)");
  std::vector<size_t> sb(c->nranks), so(c->nranks), rb(c->nranks), ro(c->nranks);
  for (int j = 0; j < c->nranks; ++j) {
    sb[j] = sc[j] * es;
    so[j] = sd[j] * es;
    rb[j] = rc[j] * es;
    ro[j] = rd[j] * es;
  }
  return dispatch(c, [=] {
    return run_alltoallv(c, path, stream, static_cast<const char*>(send), sb, so,
                         static_cast<char*>(recv), rb, ro, largest);
  });
}

hxcclResult_t hxcclAlltoAll(const void* send, void* recv, size_t count, hxcclDataType_t dt,
                            hxcclComm_t c, hxcclStream_t stream) {
  if (hxcclResult_t r = check_args(c, send, recv, count, c ? c->nranks : 1, dt)) return r;
  const size_t block = count * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, send, recv, &path)) return r;
  if (path == Path::Host)
    if (hxcclResult_t r = check_message(c, block)) return r;
  if (count == 0) return hxcclSuccess;
  std::vector<size_t> b(c->nranks, block), off(c->nranks);
  for (int j = 0; j < c->nranks; ++j) off[j] = size_t(j) * block;
  return dispatch(c, [=] {
    return run_alltoallv(c, path, stream, static_cast<const char*>(send), b, off,
                         static_cast<char*>(recv), b, off, block);
  });
}

hxcclResult_t hxcclAllToAll(const void* send, void* recv, size_t count, hxcclDataType_t dt,
                            hxcclComm_t c, hxcclStream_t stream) {
  return hxcclAlltoAll(send, recv, count, dt, c, stream);
}

// ---- Send / Recv -------------------------------------------------------------------------

static hxcclResult_t check_p2p(hxcclComm* c, const void* buf, size_t count, hxcclDataType_t dt,
                               int peer) {
  if (hxcclResult_t r = check_args(c, buf, buf, count, 1, dt)) return r;
  if (peer < 0 || peer >= c->nranks) return comm_fail(c, hxcclInvalidArgument, "peer out of range");
  return hxcclSuccess;
}

hxcclResult_t hxcclSend(const void* buf, size_t count, hxcclDataType_t dt, int peer,
                        hxcclComm_t c, hxcclStream_t stream) {
  if (hxcclResult_t r = check_p2p(c, buf, count, dt, peer)) return r;
  const size_t bytes = count * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, buf, nullptr, &path)) return r;
  if (path == Path::Host)
    if (hxcclResult_t r = check_message(c, bytes)) return r;
  return submit_p2p(c, path, true, peer, const_cast<void*>(buf), bytes, stream);
}

hxcclResult_t hxcclRecv(void* buf, size_t count, hxcclDataType_t dt, int peer, hxcclComm_t c,
                        hxcclStream_t stream) {
  if (hxcclResult_t r = check_p2p(c, buf, count, dt, peer)) return r;
  const size_t bytes = count * dtype_size(dt);
  Path path;
  if (hxcclResult_t r = pick_path(c, buf, nullptr, &path)) return r;
  if (path == Path::Host)
    if (hxcclResult_t r = check_message(c, bytes)) return r;
  return submit_p2p(c, path, false, peer, buf, bytes, stream);
}

// ---- PreMulSum operators ---------------------------------------------------------------------

hxcclResult_t hxcclRedOpCreatePreMulSum(hxcclRedOp_t* op, void* scalar, hxcclDataType_t dt,
                                        hxcclScalarResidence_t residence, hxcclComm_t c) {
  if (!c || !op || !scalar) return hxcclInvalidArgument;
  if (dtype_size(dt) == 0) return comm_fail(c, hxcclInvalidArgument, "unknown datatype");
  if (residence != hxcclScalarDevice && residence != hxcclScalarHostImmediate)
    return comm_fail(c, hxcclInvalidArgument, "unknown scalar residence");
  if (residence == hxcclScalarHostImmediate && classify(scalar) == MemKind::Device)
    return comm_fail(c, hxcclInvalidArgument,
                     "hxcclScalarHostImmediate needs a scalar in host memory");
  const long slot = c->ops.claim();
  if (slot < 0)
    return comm_fail(c, hxcclInternalError, "too many live PreMulSum ops on this communicator");
  ScalarOp& u = c->ops.at(slot);
  u.dt = dt;
  if (residence == hxcclScalarDevice)
    u.deferred = scalar;
  else
    std::memcpy(u.bits, scalar, dtype_size(dt));
  *op = c->ops.handle(slot);
  return hxcclSuccess;
}

hxcclResult_t hxcclRedOpDestroy(hxcclRedOp_t op, hxcclComm_t c) {
  if (!c) return hxcclInvalidArgument;
  const long slot = c->ops.find(op);
  if (slot < 0)
    return comm_fail(c, hxcclInvalidArgument, "not a live PreMulSum op of this communicator");
  c->ops.release(slot);
  return hxcclSuccess;
}

}  // extern "C"
