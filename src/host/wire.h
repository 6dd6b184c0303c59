// Point-to-point user payload for host buffers, over a communicator's control channel, with
// the traffic counters hxcclCommGetStats reports (user bytes and messages this rank sent;
// control traffic is not counted). Plays the role of the reference's Transport /
// NetTransport (src/transport.h:15-39, src/transport_net.cc:3-102).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "ctrl/fabric.h"

namespace hx {

class HostWire {
 public:
  explicit HostWire(std::shared_ptr<Channel> ch) : ch_(std::move(ch)) {}

  // blocking forms used by the collective algorithms (tag kTagColl)
  // `fragment`: the send continues a message that was counted already (bytes count, the
  // message does not)
  hxcclResult_t exchange(int to, const void* sbuf, size_t sbytes, int from, void* rbuf,
                         size_t rbytes, bool fragment = false);
  hxcclResult_t send(int to, const void* buf, size_t bytes);
  hxcclResult_t recv(int from, void* buf, size_t bytes);
  // non-blocking forms: post, then finish_all (blocking) or step (one pass)
  hxcclResult_t post_send(int to, const void* buf, size_t bytes, int tag, bool fragment = false);
  hxcclResult_t post_recv(int from, void* buf, size_t bytes, int tag);
  hxcclResult_t finish_all();
  // One non-blocking pass over everything posted. *done turns true when nothing is left; the
  // value returned then is the first failure (all transfers are driven to their end first).
  hxcclResult_t step(bool* done);
  void cancel_all();

  Channel& channel() { return *ch_; }

  uint64_t bytes_sent = 0, msgs_sent = 0;
  std::string error;
  // Test hook: when >= 0, the (fail_after+1)-th send from now fails with hxcclSystemError
  // without touching the network.
  long fail_after = -1;

 private:
  bool injected();
  std::shared_ptr<Channel> ch_;
  std::vector<int> open_;
  hxcclResult_t first_ = hxcclSuccess;
  std::string first_why_;
};

}  // namespace hx
