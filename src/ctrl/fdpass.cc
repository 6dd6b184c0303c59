#include "fdpass.h"

#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>

namespace hx {
namespace {
socklen_t port_addr(uint64_t chan, int rank, sockaddr_un* sa) {
  std::memset(sa, 0, sizeof *sa);
  sa->sun_family = AF_UNIX;
  // leading NUL byte = abstract namespace
  const int n = std::snprintf(sa->sun_path + 1, sizeof(sa->sun_path) - 1, "hxccl-%016llx-%d",
                              static_cast<unsigned long long>(chan), rank);
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}
struct Note {
  uint32_t kind, from;
};
}  // namespace

FdPort::~FdPort() {
  if (sock_ >= 0) ::close(sock_);
}

bool FdPort::open(uint64_t chan, int rank, std::string* why) {
  sock_ = ::socket(AF_UNIX, SOCK_DGRAM, 0);
  if (sock_ < 0) return *why = std::string("unix socket: ") + std::strerror(errno), false;
  sockaddr_un sa;
  const socklen_t len = port_addr(chan, rank, &sa);
  if (::bind(sock_, reinterpret_cast<sockaddr*>(&sa), len) != 0) {
    *why = std::string("unix bind: ") + std::strerror(errno);
    ::close(sock_);
    sock_ = -1;
    return false;
  }
  return true;
}

bool FdPort::send_fd(uint64_t chan, int to_rank, int fd, uint32_t kind, uint32_t from,
                     std::string* why) {
  sockaddr_un sa;
  const socklen_t len = port_addr(chan, to_rank, &sa);
  Note note{kind, from};
  iovec iov{&note, sizeof note};
  alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))];
  std::memset(ctl, 0, sizeof ctl);
  msghdr m{};
  m.msg_name = &sa;
  m.msg_namelen = len;
  m.msg_iov = &iov;
  m.msg_iovlen = 1;
  m.msg_control = ctl;
  m.msg_controllen = sizeof ctl;
  cmsghdr* c = CMSG_FIRSTHDR(&m);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  for (int tries = 0; tries < 200; ++tries) {
    if (::sendmsg(sock_, &m, 0) >= 0) return true;
    if (errno == EINTR) continue;
    if (errno == ECONNREFUSED || errno == ENOENT || errno == EAGAIN) {  // peer not bound yet
      ::usleep(10000);
      continue;
    }
    break;
  }
  *why = std::string("sending a memory handle: ") + std::strerror(errno);
  return false;
}

bool FdPort::recv_fd(int* fd, uint32_t* kind, uint32_t* from, long timeout_ms, std::string* why) {
  pollfd pf{sock_, POLLIN, 0};
  for (;;) {
    const int rc = ::poll(&pf, 1, static_cast<int>(timeout_ms));
    if (rc < 0 && errno == EINTR) continue;
    if (rc <= 0) return *why = "no memory handle arrived in time", false;
    break;
  }
  Note note{};
  iovec iov{&note, sizeof note};
  alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))];
  msghdr m{};
  m.msg_iov = &iov;
  m.msg_iovlen = 1;
  m.msg_control = ctl;
  m.msg_controllen = sizeof ctl;
  const ssize_t r = ::recvmsg(sock_, &m, 0);
  if (r < static_cast<ssize_t>(sizeof note))
    return *why = std::string("receiving a memory handle: ") + std::strerror(errno), false;
  *fd = -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&m); c; c = CMSG_NXTHDR(&m, c))
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS)
      std::memcpy(fd, CMSG_DATA(c), sizeof(int));
  *kind = note.kind;
  *from = note.from;
  if (*fd < 0) return *why = "a handle message carried no descriptor", false;
  return true;
}

}  // namespace hx
