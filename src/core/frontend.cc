// Checks, operator planning and data-path choice shared by every API entry point.
// (Reference behaviour: src/checks.cc:10-83, src/memspace_cuda.cc:74-119.)
#include <climits>
#include <cstdlib>
#include <cstring>

#include "core/comm.h"
#include "math/reduce_host.h"

namespace hx {

hxcclResult_t comm_fail(hxcclComm* c, hxcclResult_t r, const std::string& msg) {
  if (c) {
    c->fail.text = msg;
    if (r == hxcclSystemError || r == hxcclInternalError || r == hxcclRemoteError || r == hxcclTimeout)
      c->fail.sticky = r;
  }
  return r;
}

hxcclResult_t check_args(hxcclComm* c, const void* send, const void* recv, size_t count,
                         size_t multiplier, hxcclDataType_t dt) {
  if (!c) return hxcclInvalidArgument;
  if (c->closed) return comm_fail(c, hxcclInvalidUsage, "communicator was finalized");
  const size_t es = dtype_size(dt);
  if (es == 0) return comm_fail(c, hxcclInvalidArgument, "unknown datatype");
  if (count != 0 && count > SIZE_MAX / es / multiplier)
    return comm_fail(c, hxcclInvalidArgument, "count * sizeof(datatype) overflows size_t");
  if (count != 0 && (!send || !recv))
    return comm_fail(c, hxcclInvalidArgument, "null buffer with count > 0");
  return hxcclSuccess;
}

hxcclResult_t check_message(hxcclComm* c, size_t largest_bytes) {
  if (largest_bytes <= static_cast<size_t>(INT_MAX)) return hxcclSuccess;
  return comm_fail(c, hxcclInvalidArgument,
                   "a single message would exceed INT_MAX bytes (host transport limit)");
}

hxcclResult_t plan_op(hxcclComm* c, hxcclRedOp_t op, hxcclDataType_t dt, OpPlan* plan) {
  *plan = OpPlan{};
  if (is_builtin_op(op)) {
    plan->base = op;
    return hxcclSuccess;
  }
  if (op == hxcclAvg) {  // integers: sum, then divide; floats: scale by 1/n, then sum
    if (is_integer(dt)) {
      plan->postdiv = true;
      plan->divisor = c->nranks;
    } else {
      plan->premul = true;
      store_scalar(1.0 / c->nranks, dt, plan->scalar);
    }
    return hxcclSuccess;
  }
  const long slot = c->ops.find(op);
  if (slot < 0) return comm_fail(c, hxcclInvalidArgument, "unknown op for this communicator");
  const ScalarOp& u = c->ops.at(slot);
  if (u.dt != dt)
    return comm_fail(c, hxcclInvalidArgument, "PreMulSum op was created for another datatype");
  plan->premul = true;
  if (!u.deferred) {
    std::memcpy(plan->scalar, u.bits, dtype_size(dt));
  } else if (classify(u.deferred) == MemKind::Device) {
    plan->scalar_dev = u.deferred;  // the kernel loads it, ordered after earlier work on the stream
  } else {
    std::memcpy(plan->scalar, u.deferred, dtype_size(dt));
  }
  return hxcclSuccess;
}

void device_eager_start(hxcclComm* c) {
  const char* e = std::getenv("HXCCL_DEVICE");
  int want;
  if (e && std::strcmp(e, "0") == 0)
    want = 0;
  else if (e && *e)
    want = 1;
  else
    want = cuda_context_exists() ? 1 : 0;
  int no = want ? 0 : 1;
  if (c->chan->max_int(&no) != hxcclSuccess) {
    c->device.down = hxcclSystemError;
    c->device.down_why = "agreement on starting the device path failed: " + c->chan->error;
    return;
  }
  if (no) return;
  c->device.path = start_device_path(c, &c->device.down, &c->device.down_why);
}

hxcclResult_t pick_path(hxcclComm* c, const void* a, const void* b, Path* out) {
  int where_a = -1, where_b = -1;
  const MemKind ka = classify_on(a, &where_a), kb = classify_on(b, &where_b);
  if (ka != MemKind::Null && kb != MemKind::Null && ka != kb)
    return comm_fail(c, hxcclInvalidArgument,
                     "send and recv buffers must both be host or both be device memory");
  if (ka != MemKind::Device && kb != MemKind::Device) {
    *out = Path::Host;
    return hxcclSuccess;
  }
  if (!c->device.path && c->device.down == hxcclSuccess)
    c->device.path = start_device_path(c, &c->device.down, &c->device.down_why);
  if (c->device.path && c->device.down == hxcclSuccess) {
    std::string why;
    if (hxcclResult_t r = c->device.path->broken(&why)) {
      c->device.down = r;
      c->device.down_why = why;
    }
  }
  if (c->device.down != hxcclSuccess) return comm_fail(c, c->device.down, c->device.down_why);
  // The kernels address the memory of the communicator's own GPU (and its peers' windows): a
  // buffer that lives on another device of this process would fault them.
  const int home = c->device.path ? c->device.path->device() : -1;
  if (home >= 0) {
    const int wheres[2] = {where_a, where_b};
    for (int k = 0; k < 2; ++k) {
      const int where = wheres[k];
      if (where >= 0 && where != home)
        return comm_fail(c, hxcclInvalidArgument,
                         "the buffer lives on CUDA device " + std::to_string(where) +
                             " but the communicator was created on device " + std::to_string(home));
    }
  }
  *out = Path::Device;
  return hxcclSuccess;
}

}  // namespace hx
