// Communicator lifecycle and the small query functions.
// (Reference behaviour: src/comm.cc:14-285.)
#include "core/comm.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace hx {
namespace {

int next_op_tag() {
  static std::mutex mu;
  static int tag = 0;  // wraps after 32766 communicators of one process
  std::lock_guard<std::mutex> g(mu);
  tag = tag % 0x7ffe + 1;
  return tag;
}

}  // namespace

hxcclResult_t comm_from_channel(hxcclComm_t* out, std::shared_ptr<Channel> chan, bool derived) {
  auto* c = new hxcclComm;
  c->rank = chan->rank();
  c->nranks = chan->size();
  c->chan = std::move(chan);
  c->wire = std::make_unique<HostWire>(c->chan);
  c->ops = OpTable(next_op_tag());
  c->device.derived = derived;
  device_eager_start(c);
  *out = c;
  return hxcclSuccess;
}

namespace {
hxcclResult_t make_comm(hxcclComm_t* out, std::shared_ptr<Channel> chan, bool derived = false) {
  return comm_from_channel(out, std::move(chan), derived);
}

hxcclResult_t check_config(const hxcclConfig_t* cfg) {
  if (!cfg) return hxcclSuccess;
  if (cfg->size != sizeof(hxcclConfig_t) || cfg->magic != HXCCL_CONFIG_MAGIC)
    return hxcclInvalidArgument;  // not made with HXCCL_CONFIG_INITIALIZER
  if (cfg->blocking == 0) return hxcclInvalidArgument;
  return hxcclSuccess;
}

void teardown(hxcclComm* c, bool orderly) {
  if (c->device.path) {
    c->device.path->drain();
    if (orderly && std::strstr(c->device.path->kind(), "nvls")) c->chan->barrier();
    c->device.path.reset();
  }
  c->wire.reset();
  delete c;
}

}  // namespace
}  // namespace hx

using namespace hx;

extern "C" {

hxcclResult_t hxcclGetVersion(int* version) {
  if (!version) return hxcclInvalidArgument;
  *version = HXCCL_VERSION_CODE;
  return hxcclSuccess;
}

hxcclResult_t hxcclGetUniqueId(hxcclUniqueId* id) {
  if (!id) return hxcclInvalidArgument;
  std::string why;
  return make_unique_id(id, &why);
}

hxcclResult_t hxcclCommInitRank(hxcclComm_t* comm, int nranks, hxcclUniqueId id, int rank) {
  if (!comm || nranks < 1 || rank < 0 || rank >= nranks) return hxcclInvalidArgument;
  std::shared_ptr<Channel> chan;
  std::string why;
  if (hxcclResult_t r = rendezvous(id, nranks, rank, &chan, &why)) return r;
  return make_comm(comm, std::move(chan));
}

hxcclResult_t hxcclCommInitRankConfig(hxcclComm_t* comm, int nranks, hxcclUniqueId id, int rank,
                                      hxcclConfig_t* config) {
  if (hxcclResult_t r = check_config(config)) return r;
  return hxcclCommInitRank(comm, nranks, id, rank);
}

hxcclResult_t hxcclCommSplit(hxcclComm_t comm, int color, int key, hxcclComm_t* newcomm,
                             hxcclConfig_t* config) {
  if (!comm || !newcomm || (color < 0 && color != HXCCL_SPLIT_NOCOLOR))
    return hxcclInvalidArgument;
  if (hxcclResult_t r = check_config(config)) return comm_fail(comm, r, "unsupported config");
  const uint64_t seq = comm->offspring.splits++;
  const int mine[2] = {color, key};
  std::vector<int> all(2 * size_t(comm->nranks));
  if (hxcclResult_t r = comm->chan->allgather(mine, all.data(), sizeof mine))
    return comm_fail(comm, r, "Split: " + comm->chan->error);
  // every rank takes part in the device-path agreement of the children below only with its
  // own colour, so a rank without colour is done here
  if (color == HXCCL_SPLIT_NOCOLOR) {
    *newcomm = nullptr;
    return hxcclSuccess;
  }
  std::vector<int> members;  // parent ranks of my colour, ordered by (key, parent rank)
  for (int i = 0; i < comm->nranks; ++i)
    if (all[2 * i] == color) members.push_back(i);
  std::stable_sort(members.begin(), members.end(),
                   [&](int a, int b) { return all[2 * a + 1] < all[2 * b + 1]; });
  const int me = int(std::find(members.begin(), members.end(), comm->rank) - members.begin());
  return make_comm(newcomm,
                   comm->chan->child(members, me, mix_id(comm->chan->id(), seq, uint32_t(color))), true);
}

hxcclResult_t hxcclCommShrink(hxcclComm_t comm, int* excl, int nexcl, hxcclComm_t* newcomm,
                              hxcclConfig_t* config, int flags) {
  if (!comm || !newcomm || nexcl < 0 || (nexcl > 0 && !excl)) return hxcclInvalidArgument;
  if (flags != 0) return comm_fail(comm, hxcclInvalidArgument, "shrinkFlags must be 0");
  if (hxcclResult_t r = check_config(config)) return comm_fail(comm, r, "unsupported config");
  std::vector<bool> out(comm->nranks, false);
  for (int i = 0; i < nexcl; ++i) {
    if (excl[i] < 0 || excl[i] >= comm->nranks || out[excl[i]])
      return comm_fail(comm, hxcclInvalidArgument, "excluded rank out of range or repeated");
    out[excl[i]] = true;
  }
  if (out[comm->rank])
    return comm_fail(comm, hxcclInvalidUsage, "excluded ranks must not call Shrink");
  // only the survivors call, all with the same list: the child's identity is computed, no
  // message goes to anyone (an excluded rank may be dead)
  uint64_t salt = 0x6b6e726873ull;
  std::vector<int> members;
  for (int i = 0; i < comm->nranks; ++i) {
    if (out[i])
      salt = mix_id(salt, uint64_t(i), 1);
    else
      members.push_back(i);
  }
  const int me = int(std::find(members.begin(), members.end(), comm->rank) - members.begin());
  return make_comm(newcomm,
                   comm->chan->child(members, me, mix_id(comm->chan->id(), comm->offspring.shrinks[salt]++, salt)), true);
}

hxcclResult_t hxcclCommAbort(hxcclComm_t comm) {
  if (!comm) return hxcclInvalidArgument;
  teardown(comm, /*orderly=*/false);
  return hxcclSuccess;
}

hxcclResult_t hxcclCommFinalize(hxcclComm_t comm) {
  if (!comm) return hxcclInvalidArgument;
  if (comm->device.path) comm->device.path->drain();
  comm->closed = true;
  return hxcclSuccess;
}

hxcclResult_t hxcclCommGetAsyncError(hxcclComm_t comm, hxcclResult_t* err) {
  if (!comm || !err) return hxcclInvalidArgument;
  if (comm->device.path && comm->fail.sticky == hxcclSuccess) {
    std::string why;
    if (hxcclResult_t r = comm->device.path->broken(&why)) comm_fail(comm, r, why);
  }
  *err = comm->fail.sticky;
  return hxcclSuccess;
}

hxcclResult_t hxcclCommDestroy(hxcclComm_t comm) {
  if (!comm) return hxcclInvalidArgument;
  teardown(comm, /*orderly=*/true);
  return hxcclSuccess;
}

hxcclResult_t hxcclCommCount(hxcclComm_t comm, int* count) {
  if (!comm || !count) return hxcclInvalidArgument;
  *count = comm->nranks;
  return hxcclSuccess;
}

hxcclResult_t hxcclCommUserRank(hxcclComm_t comm, int* rank) {
  if (!comm || !rank) return hxcclInvalidArgument;
  *rank = comm->rank;
  return hxcclSuccess;
}

const char* hxcclGetErrorString(hxcclResult_t r) {
  switch (r) {
    case hxcclSuccess: return "no error";
    case hxcclUnhandledCudaError: return "unhandled device error";
    case hxcclSystemError: return "system (network) error";
    case hxcclInternalError: return "internal error";
    case hxcclInvalidArgument: return "invalid argument";
    case hxcclInvalidUsage: return "invalid usage";
    case hxcclRemoteError: return "remote process error";
    case hxcclInProgress: return "operation in progress";
    case hxcclTimeout: return "timeout";
    default: return "unknown result";
  }
}

const char* hxcclGetLastError(hxcclComm_t comm) { return comm ? comm->fail.text.c_str() : ""; }

hxcclResult_t hxcclCommGetStats(hxcclComm_t comm, uint64_t* bytes, uint64_t* msgs) {
  if (!comm || !bytes || !msgs) return hxcclInvalidArgument;
  *bytes = comm->wire->bytes_sent + comm->device.bytes;
  *msgs = comm->wire->msgs_sent + comm->device.msgs;
  return hxcclSuccess;
}

hxcclResult_t hxcclCommResetStats(hxcclComm_t comm) {
  if (!comm) return hxcclInvalidArgument;
  comm->wire->bytes_sent = comm->wire->msgs_sent = 0;
  comm->device.bytes = comm->device.msgs = 0;
  return hxcclSuccess;
}

}  // extern "C"
