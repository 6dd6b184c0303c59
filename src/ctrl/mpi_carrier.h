// A Carrier over an MPI communicator, for builds with MPI (-DHXCCL_HAVE_MPI): control messages
// and host payload travel as MPI point-to-point messages instead of over this library's TCP
// mesh. It stands where the reference has MpiNet (control: src/net_mpi.cc:5-84) and MpiTransport
// (host data: src/transport_mpi.cc:9-110); here one class serves both, because a communicator's
// control traffic and host payload share one Channel.
#pragma once
#ifdef HXCCL_HAVE_MPI
#include <mpi.h>

#include <deque>
#include <list>
#include <mutex>
#include <vector>

#include "ctrl/fabric.h"

namespace hx {

class MpiCarrier : public Carrier {
 public:
  // Duplicates `comm` so that the traffic here can never match the application's own messages.
  explicit MpiCarrier(MPI_Comm comm);
  ~MpiCarrier() override;
  bool ok() const { return comm_ != MPI_COMM_NULL; }

  int self() const override { return self_; }
  int nprocs() const override { return n_; }
  int post_send(int peer, uint64_t chan, int tag, const void* buf, size_t bytes) override;
  int post_recv(int peer, uint64_t chan, int tag, void* buf, size_t bytes) override;
  hxcclResult_t poll_ticket(int ticket, bool* done, std::string* why) override;
  hxcclResult_t wait_ticket(int ticket, std::string* why) override;
  void cancel(int ticket) override;
  void sever(int peer) override;

 private:
  // Every transfer is two MPI messages to the same peer: an envelope {channel, tag, bytes} on
  // kEnvelopeTag and the body on kBodyTag. MPI keeps messages of one (source, tag) pair in
  // order, so the k-th envelope from a peer describes the k-th body from it; matching by
  // (sender, channel, tag) in posting order, parking of early messages and truncation are done
  // here, exactly as the TCP carrier does them, because a 64-bit channel id does not fit an MPI
  // tag.
  struct Envelope {
    uint64_t chan;
    int64_t tag;
    uint64_t bytes;
  };
  struct Ticket {
    bool live = false, finished = false;
    hxcclResult_t rc = hxcclSuccess;
    std::string why;
  };
  struct Outgoing {
    int ticket;
    int peer;
    Envelope env;
    MPI_Request req[2];
  };
  struct Wanted {
    int ticket;
    uint64_t chan;
    int tag;
    char* buf;
    size_t room;
  };
  struct Arriving {  // a body receive in flight
    int ticket;      // -1: parked (nobody asked yet) or orphaned
    int peer;
    Envelope env;
    std::vector<char> stash;  // parked or truncated messages land here
    char* dst;                // where the bytes go directly, or null when stashed
    size_t room;
    MPI_Request req;
  };
  struct Parked {
    uint64_t chan;
    int tag;
    std::vector<char> bytes;
  };
  int new_ticket();
  void finish(int ticket, hxcclResult_t rc, const std::string& why = {});
  void progress();
  bool fail_mpi(int rc, const char* what, int peer);
  void deliver(Parked& p, const Wanted& w);

  MPI_Comm comm_ = MPI_COMM_NULL;
  int self_ = 0, n_ = 1;
  std::vector<Ticket> tickets_;
  std::vector<int> spare_;
  std::list<Outgoing> out_;
  std::vector<std::list<Wanted>> wanted_;    // per peer, posting order
  std::vector<std::list<Parked>> parked_;    // per peer, arrival order
  std::vector<std::deque<Arriving>> arriving_;  // per peer, envelope order
  std::vector<char> down_;
  std::recursive_mutex mu_;
  long wait_limit_ms_ = 0;
};

}  // namespace hx
#endif  // HXCCL_HAVE_MPI
