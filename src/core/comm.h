// The communicator object and the helpers of the API front end.
// (Reference: src/comm.h:11-42, src/checks.h:8-33.)
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "core/devpath.h"
#include "ctrl/fabric.h"
#include "host/wire.h"
#include "hxccl.h"

namespace hx {
// A live PreMulSum operator. Its handle is hxcclNumOps + (comm tag << 16) + slot, so a handle
// from another communicator never resolves here.
struct UserOp {
  bool live = false;
  int dt = hxcclFloat32;
  bool by_pointer = false;  // hxcclScalarDevice: dereference at call time
  unsigned char value[8] = {};
  const void* ptr = nullptr;
};
constexpr int kOpSlotBits = 16;
}  // namespace hx

struct hxcclComm {
  int rank = 0;
  int nranks = 1;
  std::shared_ptr<hx::Channel> chan;       // control + host payload
  std::unique_ptr<hx::HostWire> wire;      // host data path
  std::unique_ptr<hx::DevicePath> dev;     // device data path, once started
  hxcclResult_t dev_error = hxcclSuccess;  // sticky failure of the device path
  std::string dev_error_msg;
  std::string last_error;
  std::vector<hx::UserOp> user_ops;
  int op_tag = 0;        // 1..0x7ffe, per communicator of this process
  uint64_t derived = 0;  // Split calls so far; feeds the children's channel ids
  // Shrink calls so far per exclude list. Only the survivors of a list call Shrink, so a count
  // shared with Split would drift apart between ranks that were and were not excluded.
  std::map<uint64_t, uint64_t> shrunk;
  bool finalized = false;
  hxcclResult_t async_error = hxcclSuccess;
  uint64_t dev_bytes = 0, dev_msgs = 0;  // device-path traffic under the reference schedule
};

namespace hx {

// Records `msg` as the communicator's last error; System/Internal/Remote (and Timeout, which
// only the bounded device-side waits produce) also become the sticky asynchronous error.
// Returns r.
hxcclResult_t comm_fail(hxcclComm* c, hxcclResult_t r, const std::string& msg);
long user_op_slot(const hxcclComm* c, hxcclRedOp_t op);  // -1 when not a live op of c

// Argument checks shared by the collectives; nothing is sent when they fail.
hxcclResult_t check_args(hxcclComm* c, const void* send, const void* recv, size_t count,
                         size_t multiplier, hxcclDataType_t dt);
// The host transport's per-message limit (INT_MAX bytes); every rank computes the same value.
hxcclResult_t check_message(hxcclComm* c, size_t largest_bytes);
hxcclResult_t plan_op(hxcclComm* c, hxcclRedOp_t op, hxcclDataType_t dt, OpPlan* plan);

enum class Path { Host, Device };
// Chooses the data path from the buffers this rank uses (null ones are ignored); mixed host
// and device buffers are hxcclInvalidArgument. Starts or re-checks the device path as needed.
hxcclResult_t pick_path(hxcclComm* c, const void* a, const void* b, Path* out);
// Starts the device path when every rank wants it (a CUDA context exists, or HXCCL_DEVICE=1).
void device_eager_start(hxcclComm* c);

// Run now, or at the outermost hxcclGroupEnd when a group is open.
using Deferred = std::function<hxcclResult_t()>;

}  // namespace hx
