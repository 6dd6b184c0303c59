#include "fabric.h"

#include <errno.h>
#include <poll.h>
#include <sched.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>

namespace hx {
namespace {
constexpr uint32_t kWireMagic = 0x48784632u;        // "HxF2"
constexpr uint64_t kMaxFrame = uint64_t(1) << 40;    // larger sizes mean a corrupt stream
constexpr uint64_t kHoldMin = 64 * 1024;             // smaller early frames are parked at once
using Lock = std::lock_guard<std::recursive_mutex>;

std::string peer_gone(int peer) { return "rank " + std::to_string(peer) + " closed the connection"; }
}  // namespace

Fabric::Fabric(int self, std::vector<int> socks) : self_(self), links_(socks.size()) {
  for (size_t i = 0; i < socks.size(); ++i) links_[i].fd = socks[i];
  sink_.resize(64 * 1024);
  if (const char* e = std::getenv("HXCCL_NET_TIMEOUT_MS")) wait_limit_ms_ = std::atol(e);
  if (const char* e = std::getenv("HXCCL_SPIN_US")) spin_us_ = std::max(0L, std::atol(e));
  if (const char* e = std::getenv("HXCCL_HOLD_US")) hold_us_ = std::max(0L, std::atol(e));
}

Fabric::~Fabric() {
  for (Link& l : links_)
    if (l.fd >= 0) ::close(l.fd);
}

int Fabric::new_ticket() {
  int t;
  if (!spare_.empty()) {
    t = spare_.back();
    spare_.pop_back();
  } else {
    t = static_cast<int>(tickets_.size());
    tickets_.emplace_back();
  }
  tickets_[t] = Ticket{};
  tickets_[t].live = true;
  return t;
}

void Fabric::finish(int ticket, hxcclResult_t rc, const std::string& why) {
  if (ticket < 0) return;
  Ticket& t = tickets_[ticket];
  if (!t.live || t.finished) return;
  t.finished = true;
  t.rc = rc;
  t.why = why;
}

// ---- posting -------------------------------------------------------------------------------

void Fabric::pair_self() {
  for (auto s = self_sends_.begin(); s != self_sends_.end();) {
    auto w = std::find_if(self_wanted_.begin(), self_wanted_.end(), [&](const Wanted& x) {
      return x.chan == s->chan && x.tag == s->tag;
    });
    if (w == self_wanted_.end()) {
      ++s;
      continue;
    }
    const size_t n = std::min(s->bytes, w->room);
    if (n) std::memmove(w->buf, s->buf, n);
    finish(w->ticket, s->bytes > w->room ? hxcclSystemError : hxcclSuccess,
           s->bytes > w->room ? kTruncatedMsg : "");
    finish(s->ticket, hxcclSuccess);
    self_wanted_.erase(w);
    s = self_sends_.erase(s);
  }
}

int Fabric::post_send(int peer, uint64_t chan, int tag, const void* buf, size_t bytes) {
  Lock g(mu_);
  const int t = new_ticket();
  if (peer == self_) {
    self_sends_.push_back({t, chan, tag, static_cast<const char*>(buf), bytes});
    pair_self();
    return t;
  }
  Link& l = links_[peer];
  if (l.down) {
    finish(t, hxcclSystemError, l.down_why);
    return t;
  }
  Outgoing o;
  o.ticket = t;
  o.head = Wire{kWireMagic, tag, chan, bytes};
  o.body = static_cast<const char*>(buf);
  l.out.push_back(std::move(o));
  flush_out(peer);
  return t;
}

int Fabric::post_recv(int peer, uint64_t chan, int tag, void* buf, size_t bytes) {
  Lock g(mu_);
  const int t = new_ticket();
  char* dst = static_cast<char*>(buf);
  if (peer == self_) {
    self_wanted_.push_back({t, chan, tag, dst, bytes});
    pair_self();
    return t;
  }
  Link& l = links_[peer];
  for (auto p = l.parked.begin(); p != l.parked.end(); ++p) {
    if (p->chan != chan || p->tag != tag || p->claimer >= 0 || p->discard) continue;
    if (p->whole) {
      const size_t n = std::min(p->bytes.size(), bytes);
      if (n) std::memcpy(dst, p->bytes.data(), n);
      const bool cut = p->bytes.size() > bytes;
      finish(t, cut ? hxcclSystemError : hxcclSuccess, cut ? kTruncatedMsg : "");
      l.parked.erase(p);
    } else {
      p->claimer = t;
      p->claim_buf = dst;
      p->claim_room = bytes;
    }
    return t;
  }
  if (l.down) {
    finish(t, hxcclSystemError, l.down_why);
    return t;
  }
  if (l.held) {
    if (l.in_head.chan == chan && l.in_head.tag == tag) {  // the held frame is the one
      l.held = false;
      l.in_ticket = t;
      l.in_buf = dst;
      l.in_room = bytes;
      drain_in(peer);
      return t;
    }
    park_frame(l);  // what this receive wants is behind the held frame
    l.wanted.push_back({t, chan, tag, dst, bytes});
    drain_in(peer);
    return t;
  }
  l.wanted.push_back({t, chan, tag, dst, bytes});
  return t;
}

// ---- socket progress -------------------------------------------------------------------------

// What of a frame has not left yet, as at most two pieces (rest of the header, rest of the body).
int Fabric::Outgoing::unsent(iovec v[2]) const {
  const struct {
    const char* at;
    size_t len;
  } piece[2] = {{reinterpret_cast<const char*>(&head), sizeof(Wire)}, {body, head.bytes}};
  size_t skip = sent;
  int k = 0;
  for (const auto& p : piece) {
    if (skip >= p.len) {
      skip -= p.len;
      continue;
    }
    v[k].iov_base = const_cast<char*>(p.at) + skip;
    v[k++].iov_len = p.len - skip;
    skip = 0;
  }
  return k;
}

void Fabric::flush_out(int peer) {
  Link& l = links_[peer];
  while (!l.down && !l.out.empty()) {
    Outgoing& o = l.out.front();
    iovec v[2];
    msghdr m{};
    m.msg_iov = v;
    // header and body leave in one system call
    while ((m.msg_iovlen = o.unsent(v)) > 0) {
      const ssize_t w = ::sendmsg(l.fd, &m, MSG_NOSIGNAL);
      if (w > 0) {
        o.sent += static_cast<size_t>(w);
        continue;
      }
      if (w < 0 && errno == EINTR) continue;
      if (w < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) return;
      link_down(peer, peer_gone(peer));
      return;
    }
    finish(o.ticket, hxcclSuccess);
    l.out.pop_front();
  }
}

void Fabric::start_body(Link& l, int peer) {
  if (l.in_head.magic != kWireMagic || l.in_head.bytes > kMaxFrame) {
    link_down(peer, "corrupt frame from rank " + std::to_string(peer));
    return;
  }
  l.in_body = true;
  l.body_got = 0;
  l.in_ticket = -1;
  l.in_buf = nullptr;
  l.in_room = 0;
  l.in_orphan = false;
  l.in_parked = nullptr;
  auto w = std::find_if(l.wanted.begin(), l.wanted.end(), [&](const Wanted& x) {
    return x.chan == l.in_head.chan && x.tag == l.in_head.tag;
  });
  if (w != l.wanted.end()) {
    l.in_ticket = w->ticket;
    l.in_buf = w->buf;
    l.in_room = w->room;
    l.wanted.erase(w);
  } else if (hold_us_ > 0 && l.in_head.bytes >= kHoldMin && l.wanted.empty()) {
    l.held = true;
    l.held_since = std::chrono::steady_clock::now();
    return;
  } else {
    park_frame(l);
  }
  if (l.in_head.bytes == 0) end_body(l);
}

// The frame whose header is in l.in_head gets a private buffer until a receive asks for it.
void Fabric::park_frame(Link& l) {
  l.held = false;
  l.parked.emplace_back();
  Parked& p = l.parked.back();
  p.chan = l.in_head.chan;
  p.tag = l.in_head.tag;
  p.bytes.resize(l.in_head.bytes);
  l.in_parked = &p;
}

void Fabric::end_body(Link& l) {
  const size_t n = l.in_head.bytes;
  if (l.in_parked) {
    Parked* p = l.in_parked;
    p->whole = true;
    if (p->claimer >= 0) {
      const size_t c = std::min(n, p->claim_room);
      if (c) std::memcpy(p->claim_buf, p->bytes.data(), c);
      finish(p->claimer, n > p->claim_room ? hxcclSystemError : hxcclSuccess,
             n > p->claim_room ? kTruncatedMsg : "");
    }
    if (p->claimer >= 0 || p->discard)
      l.parked.remove_if([p](const Parked& x) { return &x == p; });
  } else if (l.in_ticket >= 0) {
    finish(l.in_ticket, n > l.in_room ? hxcclSystemError : hxcclSuccess,
           n > l.in_room ? kTruncatedMsg : "");
  }
  l.in_body = false;
  l.head_got = 0;
  l.in_parked = nullptr;
  l.in_ticket = -1;
}

// Bytes from the connection: frame headers and small bodies come through a read-ahead buffer
// (one system call then usually delivers a whole small message, header and body, or several
// of them), larger bodies go straight from the socket into their destination. The buffer is
// small so that the head of a large body, which arrives in it with the header, costs little to
// copy on.
ssize_t Fabric::pull(Link& l, char* into, size_t want) {
  constexpr size_t kAhead = 8 * 1024, kDirect = 4 * 1024;
  if (l.ahead_pos == l.ahead_end) {
    if (want >= kDirect) return ::recv(l.fd, into, want, 0);
    if (l.ahead.empty()) l.ahead.resize(kAhead);
    const ssize_t r = ::recv(l.fd, l.ahead.data(), l.ahead.size(), 0);
    if (r <= 0) return r;
    l.ahead_pos = 0;
    l.ahead_end = static_cast<size_t>(r);
  }
  const size_t n = std::min(want, l.ahead_end - l.ahead_pos);
  std::memcpy(into, l.ahead.data() + l.ahead_pos, n);
  l.ahead_pos += n;
  return static_cast<ssize_t>(n);
}

void Fabric::drain_in(int peer) {
  Link& l = links_[peer];
  while (!l.down && !l.held) {
    char* into;
    size_t want;
    if (!l.in_body) {
      into = reinterpret_cast<char*>(&l.in_head) + l.head_got;
      want = sizeof(Wire) - l.head_got;
    } else {
      const size_t left = l.in_head.bytes - l.body_got;
      if (l.in_parked) {
        into = l.in_parked->bytes.data() + l.body_got;
        want = left;
      } else if (l.body_got < l.in_room) {
        into = l.in_buf + l.body_got;
        want = std::min(left, l.in_room - l.body_got);
      } else {  // beyond the receive buffer (or the receive was cancelled): swallow
        into = sink_.data();
        want = std::min(left, sink_.size());
      }
    }
    const ssize_t r = pull(l, into, want);
    if (r < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) return;
      link_down(peer, peer_gone(peer));
      return;
    }
    if (r == 0) {
      link_down(peer, peer_gone(peer));
      return;
    }
    if (!l.in_body) {
      l.head_got += static_cast<size_t>(r);
      if (l.head_got == sizeof(Wire)) start_body(l, peer);
    } else {
      l.body_got += static_cast<size_t>(r);
      if (l.body_got == l.in_head.bytes) end_body(l);
    }
  }
}

void Fabric::link_down(int peer, const std::string& why) {
  Link& l = links_[peer];
  if (l.down) return;
  l.down = true;
  l.down_why = why;
  if (l.fd >= 0) {
    ::close(l.fd);
    l.fd = -1;
  }
  for (Outgoing& o : l.out) finish(o.ticket, hxcclSystemError, why);
  l.out.clear();
  for (Wanted& w : l.wanted) finish(w.ticket, hxcclSystemError, why);
  l.wanted.clear();
  if (l.in_body && l.in_ticket >= 0) finish(l.in_ticket, hxcclSystemError, why);
  for (auto p = l.parked.begin(); p != l.parked.end();) {
    if (!p->whole) {
      finish(p->claimer, hxcclSystemError, why);
      p = l.parked.erase(p);
    } else {
      ++p;
    }
  }
  l.in_body = false;
  l.held = false;
  l.in_parked = nullptr;
  l.in_ticket = -1;
}

// One round of socket progress; true when a connection had something to do.
bool Fabric::pump(int timeout_ms) {
  std::vector<pollfd>& pf = poll_set_;  // kept between calls: this runs once per wait
  std::vector<int>& who = poll_who_;
  pf.clear();
  who.clear();
  bool took_in = false;
  for (int i = 0; i < nprocs(); ++i) {
    Link& l = links_[i];
    if (i == self_ || l.down || l.fd < 0) continue;
    if (l.held) {
      const auto age = std::chrono::duration_cast<std::chrono::microseconds>(
                           std::chrono::steady_clock::now() - l.held_since).count();
      if (age > hold_us_) {
        park_frame(l);  // nobody came for it: take it in as any early message
        drain_in(i);
        took_in = true;
        if (l.down) continue;
      } else if (timeout_ms > 0) {  // a sleep must not outlast the hold
        timeout_ms = std::min<long>(timeout_ms, 1 + (hold_us_ - age) / 1000);
      }
    }
    pollfd p{};
    p.fd = l.fd;
    p.events = l.held ? 0 : POLLIN;  // a held frame's bytes wait in the socket
    if (!l.out.empty()) p.events |= POLLOUT;
    pf.push_back(p);
    who.push_back(i);
  }
  if (pf.empty()) return took_in;
  const int rc = ::poll(pf.data(), pf.size(), took_in ? 0 : timeout_ms);
  if (rc <= 0) return took_in;
  for (size_t k = 0; k < pf.size(); ++k) {
    if (pf[k].revents & POLLOUT) flush_out(who[k]);
    if (pf[k].revents & (POLLIN | POLLHUP | POLLERR)) {
      Link& l = links_[who[k]];
      if (l.held) park_frame(l);  // the peer hung up: read what it left
      drain_in(who[k]);
    }
  }
  return true;
}

// ---- completion --------------------------------------------------------------------------------

hxcclResult_t Fabric::poll_ticket(int ticket, bool* done, std::string* why) {
  Lock g(mu_);
  if (!tickets_[ticket].finished) pump(0);
  Ticket& t = tickets_[ticket];
  *done = t.finished;
  if (!t.finished) return hxcclSuccess;
  const hxcclResult_t rc = t.rc;
  if (why && rc != hxcclSuccess) *why = t.why;
  t.live = false;
  spare_.push_back(ticket);
  return rc;
}

hxcclResult_t Fabric::wait_ticket(int ticket, std::string* why) {
  const auto t0 = std::chrono::steady_clock::now();
  // An answer that is already on its way arrives within microseconds: look for it without
  // sleeping first, since waking a sleeping thread costs more than the message took. While
  // bytes keep moving the wait keeps polling; it sleeps once nothing came for spin_us_.
  auto quiet_since = t0;
  bool spinning = spin_us_ > 0;
  for (;;) {
    bool moved = false;
    {
      Lock g(mu_);
      if (!tickets_[ticket].finished) moved = pump(spinning ? 0 : 20);
      if (tickets_[ticket].finished) {
        bool done;
        return poll_ticket(ticket, &done, why);
      }
    }
    const auto now = std::chrono::steady_clock::now();
    if (moved) {
      quiet_since = now;
      spinning = spin_us_ > 0;
    } else if (spinning) {
      const auto quiet = now - quiet_since;
      if (quiet > std::chrono::microseconds(spin_us_))
        spinning = false;
      else if (quiet > std::chrono::microseconds(50))
        ::sched_yield();  // with more ranks than cores the peer may be waiting for this core
    }
    if (wait_limit_ms_ > 0 && now - t0 > std::chrono::milliseconds(wait_limit_ms_)) {
      cancel(ticket);
      if (why) *why = "no answer from a peer within HXCCL_NET_TIMEOUT_MS";
      return hxcclTimeout;
    }
  }
}

void Fabric::cancel(int ticket) {
  Lock g(mu_);
  if (ticket < 0 || !tickets_[ticket].live) return;
  self_wanted_.remove_if([&](const Wanted& w) { return w.ticket == ticket; });
  self_sends_.remove_if([&](const SelfSend& s) { return s.ticket == ticket; });
  for (Link& l : links_) {
    for (auto o = l.out.begin(); o != l.out.end(); ++o) {
      if (o->ticket != ticket) continue;
      if (o->sent == 0) {
        l.out.erase(o);
      } else {  // the frame must still go out whole: send the rest from a private copy
        o->keepalive.assign(o->body, o->body + o->head.bytes);
        o->body = o->keepalive.data();
        o->ticket = -1;
      }
      break;
    }
    l.wanted.remove_if([&](const Wanted& w) { return w.ticket == ticket; });
    if (l.in_body && l.in_ticket == ticket) {
      l.in_ticket = -1;
      l.in_orphan = true;
      l.in_buf = nullptr;
      l.in_room = 0;
    }
    for (Parked& p : l.parked)
      if (p.claimer == ticket) {
        p.claimer = -1;
        p.discard = true;
      }
  }
  tickets_[ticket].live = false;
  spare_.push_back(ticket);
}

void Fabric::sever(int peer) {
  Lock g(mu_);
  if (peer == self_ || peer < 0 || peer >= nprocs()) return;
  if (links_[peer].fd >= 0) ::shutdown(links_[peer].fd, SHUT_RDWR);
  link_down(peer, peer_gone(peer));
}

// ---- Channel ---------------------------------------------------------------------------------

hxcclResult_t Channel::allgather(const void* mine, void* all, size_t bytes) {
  const int n = size();
  char* out = static_cast<char*>(all);
  std::memcpy(out + size_t(rank_) * bytes, mine, bytes);
  std::vector<int> ts;
  for (int p = 0; p < n; ++p)
    if (p != rank_) ts.push_back(post_recv(p, kTagCtl, out + size_t(p) * bytes, bytes));
  for (int p = 0; p < n; ++p)
    if (p != rank_) ts.push_back(post_send(p, kTagCtl, mine, bytes));
  hxcclResult_t first = hxcclSuccess;
  std::string first_why;
  for (int t : ts) {
    const hxcclResult_t r = wait_ticket(t);
    if (r != hxcclSuccess && first == hxcclSuccess) {
      first = r;
      first_why = error;
    }
  }
  if (first != hxcclSuccess) error = first_why;
  return first;
}

hxcclResult_t Channel::max_int(int* v) {
  std::vector<int> all(size());
  if (hxcclResult_t r = allgather(v, all.data(), sizeof(int))) return r;
  *v = *std::max_element(all.begin(), all.end());
  return hxcclSuccess;
}

hxcclResult_t Channel::max_u64(uint64_t* v) {
  std::vector<uint64_t> all(size());
  if (hxcclResult_t r = allgather(v, all.data(), sizeof(uint64_t))) return r;
  *v = *std::max_element(all.begin(), all.end());
  return hxcclSuccess;
}

std::shared_ptr<Channel> Channel::child(const std::vector<int>& subset, int new_rank,
                                        uint64_t id) const {
  std::vector<int> procs;
  procs.reserve(subset.size());
  for (int r : subset) procs.push_back(members_[r]);
  return std::make_shared<Channel>(fabric_, id, std::move(procs), new_rank);
}

uint64_t mix_id(uint64_t parent, uint64_t seq, uint64_t salt) {
  uint64_t z = parent ^ (seq * 0x9e3779b97f4a7c15ull) ^ (salt * 0xd1342543de82ef95ull);
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

}  // namespace hx
