// hxcclGetUniqueId / hxcclCommInitRank rendezvous over TCP.
//
// The id names a listening socket owned by the process that created it plus a random nonce.
// Every rank dials that socket and introduces itself; the owner (the "hub", whichever of its
// callers gets there first) checks that ranks 0..n-1 are each present exactly once and that all
// agree on n, then answers every caller with a verdict and the table of mesh listeners. Each
// rank then connects to all lower ranks and accepts all higher ones. A bad id is
// hxcclInvalidArgument; duplicate / inconsistent ranks are hxcclInvalidUsage on every caller;
// socket failures are hxcclSystemError. (Behaviour of the reference: src/net_sock.cc:539-665;
// the wire format here is this library's own.) Unlike the reference the hub does not wait
// forever for a rank that never comes: HXCCL_BOOTSTRAP_TIMEOUT_MS (default 120000) bounds it.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <random>
#include <thread>

#include "fabric.h"

namespace hx {
namespace {

constexpr uint32_t kIdMagic = 0x42327868u;  // "hx2B"
struct IdBody {
  uint32_t magic;
  uint32_t version;
  uint32_t addr;  // network order
  uint16_t port;  // network order
  uint16_t pad;
  uint64_t nonce;
};
static_assert(sizeof(IdBody) <= sizeof(hxcclUniqueId), "id too small");

struct Hello {
  uint64_t nonce;
  int32_t rank;
  int32_t nranks;
  uint32_t addr;
  uint16_t port;
  uint16_t pad;
};
struct Seat {
  uint32_t addr;
  uint16_t port;
  uint16_t pad;
};
struct MeshHello {
  uint64_t nonce;
  int32_t rank;
  int32_t pad;
};

std::mutex g_mu;
std::map<uint64_t, int>& hubs() {  // nonce -> listener fd, for ids made in this process
  static std::map<uint64_t, int> m;
  return m;
}

std::string sys_err(const char* what) { return std::string(what) + ": " + std::strerror(errno); }

long env_ms(const char* name, long dflt) {
  const char* e = std::getenv(name);
  if (!e || !*e) return dflt;
  char* end = nullptr;
  const long v = std::strtol(e, &end, 10);
  return (*end || v <= 0) ? dflt : v;
}

uint32_t listen_addr() {
  const char* e = std::getenv("HXCCL_SOCKET_ADDR");
  in_addr a{};
  if (e && *e && inet_pton(AF_INET, e, &a) == 1) return a.s_addr;
  inet_pton(AF_INET, "127.0.0.1", &a);
  return a.s_addr;
}

bool open_listener(int* fd, uint32_t* addr, uint16_t* port, std::string* why) {
  *fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (*fd < 0) return *why = sys_err("socket"), false;
  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = listen_addr();
  sa.sin_port = 0;
  socklen_t len = sizeof sa;
  if (::bind(*fd, reinterpret_cast<sockaddr*>(&sa), sizeof sa) != 0 || ::listen(*fd, 128) != 0 ||
      ::getsockname(*fd, reinterpret_cast<sockaddr*>(&sa), &len) != 0) {
    *why = sys_err("bind/listen");
    ::close(*fd);
    *fd = -1;
    return false;
  }
  *addr = sa.sin_addr.s_addr;
  *port = sa.sin_port;
  return true;
}

// connect with retries: the other side may not be listening yet
int dial(uint32_t addr, uint16_t port, long limit_ms, std::string* why) {
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return *why = sys_err("socket"), -1;
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = addr;
    sa.sin_port = port;
    if (::connect(fd, reinterpret_cast<sockaddr*>(&sa), sizeof sa) == 0) return fd;
    const int e = errno;
    ::close(fd);
    if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(limit_ms)) {
      errno = e;
      *why = sys_err("connect");
      return -1;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(10));
  }
}

bool put(int fd, const void* p, size_t n) {
  const char* c = static_cast<const char*>(p);
  while (n) {
    const ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
    if (w < 0 && errno == EINTR) continue;
    if (w <= 0) return false;
    c += w;
    n -= static_cast<size_t>(w);
  }
  return true;
}
// blocking read of exactly n bytes, giving up at `deadline`
bool get(int fd, void* p, size_t n, std::chrono::steady_clock::time_point deadline) {
  char* c = static_cast<char*>(p);
  while (n) {
    const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(
                          deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0) return false;
    pollfd pf{fd, POLLIN, 0};
    const int rc = ::poll(&pf, 1, static_cast<int>(std::min<long long>(left, 1000)));
    if (rc < 0 && errno == EINTR) continue;
    if (rc == 0) continue;
    const ssize_t r = ::recv(fd, c, n, 0);
    if (r < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    if (r <= 0) return false;
    c += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}
int accept_until(int lfd, std::chrono::steady_clock::time_point deadline) {
  for (;;) {
    const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(
                          deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0) return -1;
    pollfd pf{lfd, POLLIN, 0};
    const int rc = ::poll(&pf, 1, static_cast<int>(std::min<long long>(left, 1000)));
    if (rc < 0 && errno != EINTR) return -1;
    if (rc <= 0) continue;
    const int fd = ::accept(lfd, nullptr, nullptr);
    if (fd >= 0) return fd;
    if (errno != EINTR && errno != EAGAIN) return -1;
  }
}

void make_mesh_socket(int fd) {
  int one = 1;
  ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  ::fcntl(fd, F_SETFL, ::fcntl(fd, F_GETFL, 0) | O_NONBLOCK);
}

}  // namespace

hxcclResult_t make_unique_id(hxcclUniqueId* id, std::string* why) {
  int fd;
  uint32_t addr;
  uint16_t port;
  if (!open_listener(&fd, &addr, &port, why)) return hxcclSystemError;
  std::random_device rd;
  uint64_t nonce = (uint64_t(rd()) << 32) ^ rd();
  nonce ^= uint64_t(::getpid()) << 17;
  IdBody b{kIdMagic, HXCCL_VERSION_CODE, addr, port, 0, nonce};
  std::memset(id, 0, sizeof *id);
  std::memcpy(id->internal, &b, sizeof b);
  std::lock_guard<std::mutex> g(g_mu);
  hubs()[nonce] = fd;
  return hxcclSuccess;
}

hxcclResult_t rendezvous(const hxcclUniqueId& id, int nranks, int rank,
                         std::shared_ptr<Channel>* out, std::string* why) {
  IdBody b;
  std::memcpy(&b, id.internal, sizeof b);
  if (b.magic != kIdMagic) {
    *why = "the unique id was not made by hxcclGetUniqueId";
    return hxcclInvalidArgument;
  }
  const long limit = env_ms("HXCCL_BOOTSTRAP_TIMEOUT_MS", 120000);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(limit);

  int my_listener;
  uint32_t my_addr;
  uint16_t my_port;
  if (!open_listener(&my_listener, &my_addr, &my_port, why)) return hxcclSystemError;

  int hub_fd = -1;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = hubs().find(b.nonce);
    if (it != hubs().end()) {
      hub_fd = it->second;
      hubs().erase(it);
    }
  }

  std::vector<Seat> table(nranks);
  int32_t verdict = 0;  // 0 ok, 1 the ranks disagree, 2 system trouble
  if (hub_fd >= 0) {
    std::vector<int> callers;
    std::vector<Hello> said;
    std::vector<int> seen(nranks, 0);
    seen[rank] = 1;
    table[rank] = Seat{my_addr, my_port, 0};
    while (static_cast<int>(callers.size()) < nranks - 1) {
      const int fd = accept_until(hub_fd, deadline);
      if (fd < 0) {
        verdict = 2;
        *why = "bootstrap: not every rank arrived within HXCCL_BOOTSTRAP_TIMEOUT_MS";
        break;
      }
      Hello h;
      if (!get(fd, &h, sizeof h, deadline) || h.nonce != b.nonce) {
        ::close(fd);  // a stranger, or a caller that died: keep waiting for the real ones
        continue;
      }
      callers.push_back(fd);
      said.push_back(h);
    }
    if (verdict == 0) {
      for (const Hello& h : said) {
        if (h.nranks != nranks || h.rank < 0 || h.rank >= nranks || seen[h.rank]) {
          verdict = 1;
          *why = "bootstrap: ranks are duplicated, missing or disagree on nranks";
          break;
        }
        seen[h.rank] = 1;
        table[h.rank] = Seat{h.addr, h.port, 0};
      }
    }
    for (int fd : callers) {
      put(fd, &verdict, sizeof verdict);
      if (verdict == 0) put(fd, table.data(), table.size() * sizeof(Seat));
      ::close(fd);
    }
    ::close(hub_fd);
  } else {
    std::string dial_why;
    const int fd = dial(b.addr, b.port, std::min<long>(limit, 30000), &dial_why);
    if (fd < 0) {
      ::close(my_listener);
      *why = "bootstrap: " + dial_why;
      return hxcclSystemError;
    }
    Hello h{b.nonce, rank, nranks, my_addr, my_port, 0};
    bool ok = put(fd, &h, sizeof h) && get(fd, &verdict, sizeof verdict, deadline);
    if (ok && verdict == 0) ok = get(fd, table.data(), table.size() * sizeof(Seat), deadline);
    ::close(fd);
    if (!ok) {
      verdict = 2;
      *why = "bootstrap: lost the connection to the rank that made the unique id";
    } else if (verdict == 1) {
      *why = "bootstrap: ranks are duplicated, missing or disagree on nranks";
    } else if (verdict == 2) {
      *why = "bootstrap: not every rank arrived in time";
    }
  }
  if (verdict != 0) {
    ::close(my_listener);
    return verdict == 1 ? hxcclInvalidUsage : hxcclSystemError;
  }

  // full mesh: dial down, accept up
  std::vector<int> socks(nranks, -1);
  bool ok = true;
  for (int j = 0; j < rank && ok; ++j) {
    std::string dw;
    const int fd = dial(table[j].addr, table[j].port, 30000, &dw);
    MeshHello mh{b.nonce, rank, 0};
    if (fd < 0 || !put(fd, &mh, sizeof mh)) {
      ok = false;
      *why = "mesh: cannot reach rank " + std::to_string(j) + " (" + dw + ")";
      if (fd >= 0) ::close(fd);
      break;
    }
    socks[j] = fd;
  }
  for (int need = nranks - 1 - rank; ok && need > 0;) {
    const int fd = accept_until(my_listener, deadline);
    if (fd < 0) {
      ok = false;
      *why = "mesh: a higher rank never connected";
      break;
    }
    MeshHello mh;
    if (!get(fd, &mh, sizeof mh, deadline) || mh.nonce != b.nonce || mh.rank <= rank ||
        mh.rank >= nranks || socks[mh.rank] >= 0) {
      ::close(fd);
      continue;
    }
    socks[mh.rank] = fd;
    --need;
  }
  ::close(my_listener);
  if (!ok) {
    for (int fd : socks)
      if (fd >= 0) ::close(fd);
    return hxcclSystemError;
  }
  for (int fd : socks)
    if (fd >= 0) make_mesh_socket(fd);
  auto fabric = std::make_shared<Fabric>(rank, std::move(socks));
  std::vector<int> everyone(nranks);
  for (int i = 0; i < nranks; ++i) everyone[i] = i;
  *out = std::make_shared<Channel>(std::move(fabric), b.nonce, std::move(everyone), rank);
  return hxcclSuccess;
}

}  // namespace hx
