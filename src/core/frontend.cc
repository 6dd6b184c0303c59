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
    c->last_error = msg;
    if (r == hxcclSystemError || r == hxcclInternalError || r == hxcclRemoteError || r == hxcclTimeout)
      c->async_error = r;
  }
  return r;
}

long user_op_slot(const hxcclComm* c, hxcclRedOp_t op) {
  const long v = static_cast<long>(op) - hxcclNumOps;
  if (v < 0 || (v >> kOpSlotBits) != c->op_tag) return -1;
  const long slot = v & ((1L << kOpSlotBits) - 1);
  if (slot >= static_cast<long>(c->user_ops.size()) || !c->user_ops[slot].live) return -1;
  return slot;
}

hxcclResult_t check_args(hxcclComm* c, const void* send, const void* recv, size_t count,
                         size_t multiplier, hxcclDataType_t dt) {
  if (!c) return hxcclInvalidArgument;
  if (c->finalized) return comm_fail(c, hxcclInvalidUsage, "communicator was finalized");
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
  const long slot = user_op_slot(c, op);
  if (slot < 0) return comm_fail(c, hxcclInvalidArgument, "unknown op for this communicator");
  const UserOp& u = c->user_ops[slot];
  if (u.dt != dt)
    return comm_fail(c, hxcclInvalidArgument, "PreMulSum op was created for another datatype");
  plan->premul = true;
  if (!u.by_pointer) {
    std::memcpy(plan->scalar, u.value, dtype_size(dt));
  } else if (classify(u.ptr) == MemKind::Device) {
    plan->scalar_dev = u.ptr;  // the kernel loads it, ordered after earlier work on the stream
  } else {
    std::memcpy(plan->scalar, u.ptr, dtype_size(dt));
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
    c->dev_error = hxcclSystemError;
    c->dev_error_msg = "agreement on starting the device path failed: " + c->chan->error;
    return;
  }
  if (no) return;
  c->dev = start_device_path(c, &c->dev_error, &c->dev_error_msg);
}

hxcclResult_t pick_path(hxcclComm* c, const void* a, const void* b, Path* out) {
  const MemKind ka = classify(a), kb = classify(b);
  if (ka != MemKind::Null && kb != MemKind::Null && ka != kb)
    return comm_fail(c, hxcclInvalidArgument,
                     "send and recv buffers must both be host or both be device memory");
  if (ka != MemKind::Device && kb != MemKind::Device) {
    *out = Path::Host;
    return hxcclSuccess;
  }
  if (!c->dev && c->dev_error == hxcclSuccess)
    c->dev = start_device_path(c, &c->dev_error, &c->dev_error_msg);
  if (c->dev && c->dev_error == hxcclSuccess) {
    std::string why;
    if (hxcclResult_t r = c->dev->broken(&why)) {
      c->dev_error = r;
      c->dev_error_msg = why;
    }
  }
  if (c->dev_error != hxcclSuccess) return comm_fail(c, c->dev_error, c->dev_error_msg);
  *out = Path::Device;
  return hxcclSuccess;
}

}  // namespace hx
