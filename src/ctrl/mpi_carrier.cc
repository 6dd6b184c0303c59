#ifdef HXCCL_HAVE_MPI
#include "ctrl/mpi_carrier.h"

#include <algorithm>
#include <chrono>
#include <climits>
#include <cstdlib>
#include <cstring>

namespace hx {
namespace {
constexpr int kEnvelopeTag = 7001, kBodyTag = 7002;
using Guard = std::lock_guard<std::recursive_mutex>;

std::string mpi_text(int rc) {
  char buf[MPI_MAX_ERROR_STRING + 1] = {};
  int len = 0;
  if (MPI_Error_string(rc, buf, &len) != MPI_SUCCESS) return "MPI error " + std::to_string(rc);
  return std::string(buf, size_t(std::max(0, len)));
}
}  // namespace

MpiCarrier::MpiCarrier(MPI_Comm comm) {
  if (MPI_Comm_dup(comm, &comm_) != MPI_SUCCESS) {
    comm_ = MPI_COMM_NULL;
    return;
  }
  MPI_Comm_set_errhandler(comm_, MPI_ERRORS_RETURN);  // failures become result codes, not aborts
  MPI_Comm_rank(comm_, &self_);
  MPI_Comm_size(comm_, &n_);
  wanted_.resize(size_t(n_));
  parked_.resize(size_t(n_));
  arriving_.resize(size_t(n_));
  down_.assign(size_t(n_), 0);
  if (const char* e = std::getenv("HXCCL_NET_TIMEOUT_MS")) wait_limit_ms_ = std::atol(e);
}

MpiCarrier::~MpiCarrier() {
  if (comm_ != MPI_COMM_NULL) MPI_Comm_free(&comm_);
}

int MpiCarrier::new_ticket() {
  int t;
  if (!spare_.empty()) {
    t = spare_.back();
    spare_.pop_back();
  } else {
    t = int(tickets_.size());
    tickets_.emplace_back();
  }
  tickets_[size_t(t)] = Ticket{};
  tickets_[size_t(t)].live = true;
  return t;
}

void MpiCarrier::finish(int ticket, hxcclResult_t rc, const std::string& why) {
  if (ticket < 0) return;
  Ticket& t = tickets_[size_t(ticket)];
  if (!t.live || t.finished) return;
  t.finished = true;
  t.rc = rc;
  t.why = why;
}

// A failed MPI call on the link to `peer` fails everything that involves that peer, and
// nothing else (the TCP carrier's rule for a lost connection).
bool MpiCarrier::fail_mpi(int rc, const char* what, int peer) {
  if (rc == MPI_SUCCESS) return false;
  const std::string why = std::string(what) + ": " + mpi_text(rc);
  down_[size_t(peer)] = 1;
  for (Outgoing& o : out_)
    if (o.peer == peer) finish(o.ticket, hxcclSystemError, why);
  for (Wanted& w : wanted_[size_t(peer)]) finish(w.ticket, hxcclSystemError, why);
  wanted_[size_t(peer)].clear();
  for (Arriving& a : arriving_[size_t(peer)]) finish(a.ticket, hxcclSystemError, why);
  return true;
}

int MpiCarrier::post_send(int peer, uint64_t chan, int tag, const void* buf, size_t bytes) {
  Guard g(mu_);
  const int t = new_ticket();
  if (down_[size_t(peer)]) {
    finish(t, hxcclSystemError, "the connection to that peer was lost");
    return t;
  }
  if (bytes > size_t(INT_MAX)) {  // one MPI message counts its bytes in an int
    finish(t, hxcclInvalidArgument, "a single message would exceed INT_MAX bytes (MPI limit)");
    return t;
  }
  out_.push_back(Outgoing{t, peer, Envelope{chan, tag, bytes}, {MPI_REQUEST_NULL, MPI_REQUEST_NULL}});
  Outgoing& o = out_.back();
  int rc = MPI_Isend(&o.env, int(sizeof o.env), MPI_BYTE, peer, kEnvelopeTag, comm_, &o.req[0]);
  if (rc == MPI_SUCCESS) rc = MPI_Isend(buf, int(bytes), MPI_BYTE, peer, kBodyTag, comm_, &o.req[1]);
  fail_mpi(rc, "MPI_Isend", peer);
  return t;
}

void MpiCarrier::deliver(Parked& p, const Wanted& w) {
  const size_t take = std::min(p.bytes.size(), w.room);
  if (take) std::memcpy(w.buf, p.bytes.data(), take);
  if (p.bytes.size() > w.room)
    finish(w.ticket, hxcclSystemError, kTruncatedMsg);
  else
    finish(w.ticket, hxcclSuccess);
}

int MpiCarrier::post_recv(int peer, uint64_t chan, int tag, void* buf, size_t bytes) {
  Guard g(mu_);
  const int t = new_ticket();
  const Wanted w{t, chan, tag, static_cast<char*>(buf), bytes};
  // a message that came before its receive waits in the parked list
  auto& parked = parked_[size_t(peer)];
  for (auto p = parked.begin(); p != parked.end(); ++p)
    if (p->chan == chan && p->tag == tag) {
      deliver(*p, w);
      parked.erase(p);
      return t;
    }
  // ... or is still arriving into a stash that nobody had claimed
  for (Arriving& a : arriving_[size_t(peer)])
    if (a.ticket == -1 && a.env.chan == chan && a.env.tag == tag && a.dst == nullptr && a.room == 0) {
      a.ticket = t;
      a.dst = static_cast<char*>(buf);  // copied out of the stash when the body is complete
      a.room = bytes;
      return t;
    }
  if (down_[size_t(peer)]) {
    finish(t, hxcclSystemError, "the connection to that peer was lost");
    return t;
  }
  wanted_[size_t(peer)].push_back(w);
  return t;
}

void MpiCarrier::progress() {
  // sends: both parts done
  for (auto o = out_.begin(); o != out_.end();) {
    int done = 0;
    const int rc = MPI_Testall(2, o->req, &done, MPI_STATUSES_IGNORE);
    if (rc != MPI_SUCCESS) {
      const int peer = o->peer;
      const int ticket = o->ticket;
      o = out_.erase(o);
      finish(ticket, hxcclSystemError, "MPI_Testall: " + mpi_text(rc));
      down_[size_t(peer)] = 1;
      continue;
    }
    if (done) {
      finish(o->ticket, hxcclSuccess);
      o = out_.erase(o);
    } else {
      ++o;
    }
  }
  // new envelopes: each one starts the receive of its body, into the matching buffer when one
  // was posted and is large enough, else into a stash
  for (;;) {
    int flag = 0;
    MPI_Status st;
    if (MPI_Iprobe(MPI_ANY_SOURCE, kEnvelopeTag, comm_, &flag, &st) != MPI_SUCCESS || !flag) break;
    const int peer = st.MPI_SOURCE;
    Envelope env{};
    if (fail_mpi(MPI_Recv(&env, int(sizeof env), MPI_BYTE, peer, kEnvelopeTag, comm_, MPI_STATUS_IGNORE),
                 "MPI_Recv", peer))
      continue;
    arriving_[size_t(peer)].emplace_back();
    Arriving& a = arriving_[size_t(peer)].back();
    a.ticket = -1;
    a.peer = peer;
    a.env = env;
    a.dst = nullptr;
    a.room = 0;
    auto& wanted = wanted_[size_t(peer)];
    auto w = std::find_if(wanted.begin(), wanted.end(),
                          [&](const Wanted& x) { return x.chan == env.chan && x.tag == int(env.tag); });
    void* into;
    if (w != wanted.end() && w->room >= env.bytes) {
      a.ticket = w->ticket;
      into = w->buf;
      a.dst = w->buf;
      a.room = w->room;
      wanted.erase(w);
    } else {
      a.stash.resize(size_t(env.bytes));
      into = a.stash.data();
      if (w != wanted.end()) {  // too small: the leading bytes are copied out at the end
        a.ticket = w->ticket;
        a.dst = w->buf;
        a.room = w->room;
        wanted.erase(w);
      }
    }
    if (fail_mpi(MPI_Irecv(into, int(env.bytes), MPI_BYTE, peer, kBodyTag, comm_, &a.req), "MPI_Irecv", peer))
      arriving_[size_t(peer)].pop_back();
  }
  // bodies, in order per peer
  for (int peer = 0; peer < n_; ++peer) {
    auto& q = arriving_[size_t(peer)];
    while (!q.empty()) {
      Arriving& a = q.front();
      int done = 0;
      if (fail_mpi(MPI_Test(&a.req, &done, MPI_STATUS_IGNORE), "MPI_Test", peer)) {
        q.clear();
        break;
      }
      if (!done) break;
      if (a.stash.empty() && a.env.bytes > 0) {  // went straight into the posted buffer
        finish(a.ticket, hxcclSuccess);
      } else if (a.dst || a.room || a.ticket >= 0) {  // claimed: copy what fits
        Parked p{a.env.chan, int(a.env.tag), std::move(a.stash)};
        deliver(p, Wanted{a.ticket, a.env.chan, int(a.env.tag), a.dst, a.room});
      } else {
        // nobody asked yet (or the receive was cancelled and the bytes are dropped)
        if (a.ticket != -2) parked_[size_t(peer)].push_back(Parked{a.env.chan, int(a.env.tag), std::move(a.stash)});
      }
      q.pop_front();
    }
  }
}

hxcclResult_t MpiCarrier::poll_ticket(int ticket, bool* done, std::string* why) {
  Guard g(mu_);
  progress();
  Ticket& t = tickets_[size_t(ticket)];
  *done = t.finished;
  if (!t.finished) return hxcclSuccess;
  const hxcclResult_t rc = t.rc;
  if (why) *why = t.why;
  t.live = false;
  spare_.push_back(ticket);
  return rc;
}

hxcclResult_t MpiCarrier::wait_ticket(int ticket, std::string* why) {
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    bool done = false;
    const hxcclResult_t rc = poll_ticket(ticket, &done, why);
    if (done) return rc;
    if (wait_limit_ms_ > 0 && std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(wait_limit_ms_)) {
      cancel(ticket);
      if (why) *why = "no answer from a peer within HXCCL_NET_TIMEOUT_MS";
      return hxcclSystemError;
    }
  }
}

// A receive that has not matched yet is simply withdrawn; one whose body is arriving lets the
// bytes land in the stash (or, if they go straight to the caller's buffer, is waited for, as
// the memory must stay valid). A send is never taken back - MPI cannot promise that and the
// reference does not try either (src/transport_mpi.cc:102-110): it is waited for.
void MpiCarrier::cancel(int ticket) {
  Guard g(mu_);
  if (ticket < 0 || !tickets_[size_t(ticket)].live) return;
  for (auto& wanted : wanted_)
    wanted.remove_if([&](const Wanted& w) { return w.ticket == ticket; });
  for (auto& q : arriving_)
    for (Arriving& a : q)
      if (a.ticket == ticket) {
        if (a.stash.empty() && a.env.bytes > 0) MPI_Wait(&a.req, MPI_STATUS_IGNORE);
        a.ticket = -2;
        a.dst = nullptr;
        a.room = 0;
      }
  for (auto o = out_.begin(); o != out_.end();)
    if (o->ticket == ticket) {
      MPI_Waitall(2, o->req, MPI_STATUSES_IGNORE);
      o = out_.erase(o);
    } else {
      ++o;
    }
  tickets_[size_t(ticket)].live = false;
  spare_.push_back(ticket);
}

void MpiCarrier::sever(int peer) {
  Guard g(mu_);
  fail_mpi(MPI_ERR_OTHER, "connection closed by a test", peer);
}

}  // namespace hx
#endif  // HXCCL_HAVE_MPI
