// Control fabric: one TCP connection per pair of processes of a bootstrap, shared by every
// communicator derived from it (Split / Shrink children differ only by their 64-bit channel
// id). It carries bootstrap traffic, argument agreement, memory-handle exchange and, for
// host buffers, the user payload. It is never on the device data path.
//
// Behaviour kept from the reference's socket layer (src/net_sock.h:12-131, described in
// docs/specs/2026-11-11-hxccl-e-socket-design.md): messages match receives per
// (sender, channel, tag) in posting order; a message that arrives before its receive is parked
// in memory; a message longer than its receive delivers the first bytes and fails the receive
// with hxcclSystemError; a lost connection fails only the requests that involve that peer;
// cancelling a send that is already partly on the wire keeps a private copy of the rest so the
// caller may free its buffer. New here: every entry point takes the fabric lock, so two threads
// may drive communicators that share a fabric, and waits can be bounded
// (HXCCL_NET_TIMEOUT_MS).
#pragma once
#include <poll.h>
#include <sys/types.h>

#include <cstdint>
#include <chrono>
#include <deque>
#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "hxccl.h"

struct iovec;

namespace hx {

constexpr const char* kTruncatedMsg =
    "message truncated: the receive buffer is smaller than the message";

// What a communicator needs from the layer that connects its processes: tagged messages
// between pairs, matched per (sender, channel, tag) in posting order, handed out as tickets.
// Two carriers exist: the TCP mesh below (Fabric) and, in builds with MPI, MpiCarrier
// (ctrl/mpi_carrier.cc), which stands where the reference has MpiNet and MpiTransport
// (src/net_mpi.cc:5-84, src/transport_mpi.cc:9-110).
class Carrier {
 public:
  virtual ~Carrier() = default;
  virtual int self() const = 0;
  virtual int nprocs() const = 0;
  // Post a transfer; the returned ticket is polled with poll_ticket. peer == self() pairs a
  // send with a receive of this process.
  virtual int post_send(int peer, uint64_t chan, int tag, const void* buf, size_t bytes) = 0;
  virtual int post_recv(int peer, uint64_t chan, int tag, void* buf, size_t bytes) = 0;
  // Non-blocking progress + completion check. When *done the ticket is released and the result
  // of the transfer returned (*why explains a failure).
  virtual hxcclResult_t poll_ticket(int ticket, bool* done, std::string* why) = 0;
  // Blocks (making progress) until the ticket completes or the optional limit runs out.
  virtual hxcclResult_t wait_ticket(int ticket, std::string* why) = 0;
  virtual void cancel(int ticket) = 0;
  // Test hook: treats the connection to `peer` as lost, as if the process had died.
  virtual void sever(int peer) = 0;
};

class Fabric : public Carrier {
 public:
  // socks[i] is a connected, non-blocking stream socket to process i; socks[self] is -1.
  Fabric(int self, std::vector<int> socks);
  ~Fabric() override;
  Fabric(const Fabric&) = delete;
  Fabric& operator=(const Fabric&) = delete;

  int self() const override { return self_; }
  int nprocs() const override { return static_cast<int>(links_.size()); }
  int post_send(int peer, uint64_t chan, int tag, const void* buf, size_t bytes) override;
  int post_recv(int peer, uint64_t chan, int tag, void* buf, size_t bytes) override;
  hxcclResult_t poll_ticket(int ticket, bool* done, std::string* why) override;
  hxcclResult_t wait_ticket(int ticket, std::string* why) override;  // polls the sockets
  void cancel(int ticket) override;
  void sever(int peer) override;  // shuts the connection down

 private:
  struct Wire {  // frame header on the socket
    uint32_t magic;
    int32_t tag;
    uint64_t chan;
    uint64_t bytes;
  };
  struct Ticket {
    bool live = false, finished = false;
    hxcclResult_t rc = hxcclSuccess;
    std::string why;
  };
  struct Outgoing {
    int ticket;  // -1 once cancelled
    Wire head;
    const char* body;
    size_t sent = 0;              // header + body bytes written
    std::vector<char> keepalive;  // body copy made when a started frame is cancelled
    int unsent(iovec v[2]) const;
  };
  struct Wanted {  // a posted receive
    int ticket;
    uint64_t chan;
    int tag;
    char* buf;
    size_t room;
  };
  struct Parked {  // a message with no receive yet
    uint64_t chan;
    int tag;
    std::vector<char> bytes;
    bool whole = false;
    int claimer = -1;  // receive posted while the body was still arriving
    char* claim_buf = nullptr;
    size_t claim_room = 0;
    bool discard = false;
  };
  struct Link {
    int fd = -1;
    bool down = false;
    std::string down_why;
    std::deque<Outgoing> out;
    std::list<Wanted> wanted;
    std::list<Parked> parked;
    // frame currently being read
    Wire in_head{};
    size_t head_got = 0;
    bool in_body = false;
    size_t body_got = 0;
    int in_ticket = -1;  // receive matched to the frame, -1 none
    char* in_buf = nullptr;
    size_t in_room = 0;
    bool in_orphan = false;  // matched receive was cancelled: swallow the body
    Parked* in_parked = nullptr;
    // The header of a large frame is in, nothing asks for it yet and nothing else is wanted from
    // this peer: its body stays in the socket for a moment, so that a receive posted right after
    // gets it straight into its buffer instead of through a parked copy.
    bool held = false;
    std::chrono::steady_clock::time_point held_since{};
    // read-ahead for headers and small bodies: [ahead_pos, ahead_end) is received but not consumed
    std::vector<char> ahead;
    size_t ahead_pos = 0, ahead_end = 0;
  };

  int new_ticket();
  void finish(int ticket, hxcclResult_t rc, const std::string& why = {});
  bool pump(int timeout_ms);
  void flush_out(int peer);
  void drain_in(int peer);
  ssize_t pull(Link& l, char* into, size_t want);
  void start_body(Link& l, int peer);
  void park_frame(Link& l);
  void end_body(Link& l);
  void link_down(int peer, const std::string& why);
  void pair_self();

  int self_;
  std::vector<Link> links_;
  std::vector<Ticket> tickets_;
  std::vector<int> spare_;
  std::vector<char> sink_;  // where surplus bytes of truncated messages go
  std::vector<struct pollfd> poll_set_;
  std::vector<int> poll_who_;
  // self traffic
  std::list<Wanted> self_wanted_;
  struct SelfSend { int ticket; uint64_t chan; int tag; const char* buf; size_t bytes; };
  std::list<SelfSend> self_sends_;
  std::recursive_mutex mu_;
  long wait_limit_ms_ = 0;  // 0 = wait forever
  long spin_us_ = 10000;    // HXCCL_SPIN_US: how long a wait polls without news before it sleeps
  long hold_us_ = 200;      // HXCCL_HOLD_US: how long an unclaimed large frame stays held (0: never)
};

// A communicator's view of the fabric: ranks are positions in `members` (fabric process
// numbers), traffic is tagged with the communicator's channel id.
class Channel {
 public:
  Channel(std::shared_ptr<Carrier> f, uint64_t id, std::vector<int> members, int rank)
      : fabric_(std::move(f)), id_(id), members_(std::move(members)), rank_(rank) {}
  int rank() const { return rank_; }
  int size() const { return static_cast<int>(members_.size()); }
  uint64_t id() const { return id_; }
  Carrier& fabric() { return *fabric_; }
  const std::vector<int>& members() const { return members_; }

  int post_send(int peer, int tag, const void* buf, size_t bytes) {
    return fabric_->post_send(members_[peer], id_, tag, buf, bytes);
  }
  int post_recv(int peer, int tag, void* buf, size_t bytes) {
    return fabric_->post_recv(members_[peer], id_, tag, buf, bytes);
  }
  hxcclResult_t poll_ticket(int t, bool* done) { return note(fabric_->poll_ticket(t, done, &why_)); }
  hxcclResult_t wait_ticket(int t) { return note(fabric_->wait_ticket(t, &why_)); }
  void cancel(int t) { fabric_->cancel(t); }

  // Small collectives on the control tag (never mixed with user traffic).
  hxcclResult_t allgather(const void* mine, void* all, size_t bytes);
  hxcclResult_t max_int(int* v);
  hxcclResult_t max_u64(uint64_t* v);
  hxcclResult_t barrier() { int z = 0; return max_int(&z); }

  // Child over `subset` (ranks of this channel, in their new order).
  std::shared_ptr<Channel> child(const std::vector<int>& subset, int new_rank, uint64_t id) const;

  std::string error;  // text of the last failure

 private:
  hxcclResult_t note(hxcclResult_t r) {
    if (r != hxcclSuccess) error = why_;
    return r;
  }
  std::shared_ptr<Carrier> fabric_;
  uint64_t id_;
  std::vector<int> members_;
  int rank_;
  std::string why_;
};

// Message tags. User payload: collectives 0, Send/Recv 1 (reference: src/transport.h:12).
constexpr int kTagColl = 0, kTagP2p = 1, kTagCtl = -1, kTagHandles = -2;

// splitmix64-style mixing for the channel ids of derived communicators
uint64_t mix_id(uint64_t parent, uint64_t seq, uint64_t salt);

// Bootstrap (reference behaviour: src/net_sock.cc:539-626). make_unique_id opens a listener
// in this process and writes its address and a random nonce into the id; rendezvous connects
// all ranks through it and returns the world channel.
hxcclResult_t make_unique_id(hxcclUniqueId* id, std::string* why);
hxcclResult_t rendezvous(const hxcclUniqueId& id, int nranks, int rank,
                         std::shared_ptr<Channel>* out, std::string* why);

}  // namespace hx
