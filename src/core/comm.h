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

// The PreMulSum operators of one communicator. A handle packs hxcclNumOps + (tag << 16) + slot:
// the tag is drawn per communicator of this process, so a handle made for another communicator
// does not resolve here, and the lowest free slot is reused, so a destroyed operator's handle
// value comes back (the handle arithmetic is the reference's, src/api.cc:103-104).
constexpr int kOpSlotBits = 16;
struct ScalarOp {
  int dt = -1;                     // element type the scalar was given in; -1 marks a free slot
  const void* deferred = nullptr;  // hxcclScalarDevice: read at call time (host or device memory)
  unsigned char bits[8] = {};      // hxcclScalarHostImmediate: the value copied at creation
};
class OpTable {
 public:
  explicit OpTable(int tag = 0) : tag_(tag) {}
  // slot of a live handle of this table, or -1
  long find(hxcclRedOp_t handle) const {
    const long v = static_cast<long>(handle) - hxcclNumOps;
    if (v < 0 || (v >> kOpSlotBits) != tag_) return -1;
    const long slot = v & ((1L << kOpSlotBits) - 1);
    return slot < static_cast<long>(slots_.size()) && slots_[slot].dt >= 0 ? slot : -1;
  }
  // claims the lowest free slot; -1 when the handle space is used up
  long claim() {
    size_t slot = 0;
    while (slot < slots_.size() && slots_[slot].dt >= 0) ++slot;
    if (slot >> kOpSlotBits) return -1;
    if (slot == slots_.size()) slots_.emplace_back();
    slots_[slot] = ScalarOp{};
    return static_cast<long>(slot);
  }
  void release(long slot) { slots_[slot].dt = -1; }
  ScalarOp& at(long slot) { return slots_[slot]; }
  const ScalarOp& at(long slot) const { return slots_[slot]; }
  hxcclRedOp_t handle(long slot) const {
    return static_cast<hxcclRedOp_t>(hxcclNumOps + (tag_ << kOpSlotBits) + int(slot));
  }

 private:
  int tag_;  // 1..0x7ffe
  std::vector<ScalarOp> slots_;
};

// The device side of a communicator: the path object once it started (windows and kernels, or
// the staged fallback), why it cannot be used if set-up or a launch failed for good, and the
// traffic its calls stand for under the host schedule (what hxcclCommGetStats adds to the
// host wire's counters).
struct DeviceSide {
  std::unique_ptr<DevicePath> path;
  hxcclResult_t down = hxcclSuccess;  // not Success: every later device call returns this
  std::string down_why;
  uint64_t bytes = 0, msgs = 0;
  // true for communicators made by Split / Shrink: their windows are sized more modestly
  // (HXCCL_CHILD_WINDOW_MB, smaller Send/Recv slots) than a communicator made from scratch
  bool derived = false;
};

// What the caller can ask about failures: the text of the latest one, and the code that
// hxcclCommGetAsyncError keeps returning once a System / Internal / Remote / Timeout failure
// happened (argument errors never land there).
struct Failures {
  std::string text;
  hxcclResult_t sticky = hxcclSuccess;
};

// Numbering of the communicators derived from this one, which feeds their channel ids. Every
// member calls Split, so one counter serves; only the survivors of an exclude list call
// Shrink, so those are counted per list (a shared counter would drift between ranks).
struct Offspring {
  uint64_t splits = 0;
  std::map<uint64_t, uint64_t> shrinks;
};
}  // namespace hx

struct hxcclComm {
  int rank = 0;
  int nranks = 1;
  std::shared_ptr<hx::Channel> chan;   // control messages and host payload
  std::unique_ptr<hx::HostWire> wire;  // host data path
  hx::DeviceSide device;
  hx::OpTable ops;
  hx::Failures fail;
  hx::Offspring offspring;
  bool closed = false;  // hxcclCommFinalize was called: only Destroy is still allowed
};

namespace hx {

// Builds a communicator on a connected channel (collective: the device path may start).
hxcclResult_t comm_from_channel(hxcclComm_t* out, std::shared_ptr<Channel> chan, bool derived = false);

// Records `msg` as the communicator's last error; System/Internal/Remote (and Timeout, which
// only the bounded device-side waits produce) also become the sticky asynchronous error.
// Returns r.
hxcclResult_t comm_fail(hxcclComm* c, hxcclResult_t r, const std::string& msg);

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
