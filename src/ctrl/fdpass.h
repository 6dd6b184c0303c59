// File-descriptor passing between the processes of one node. The device layer exports each
// rank's window (and the multicast object) as POSIX file descriptors; TCP cannot carry those,
// so they travel as SCM_RIGHTS ancillary data over abstract-namespace Unix datagram sockets,
// one per (communicator channel, rank). The reference has no counterpart: it shares memory
// with cudaIpcGetMemHandle byte blobs over its control network (src/transport_ipc.cc:105-132).
#pragma once
#include <cstdint>
#include <string>

namespace hx {

class FdPort {
 public:
  FdPort() = default;
  ~FdPort();
  FdPort(const FdPort&) = delete;
  FdPort& operator=(const FdPort&) = delete;
  // Binds the port of (chan, rank). Names live in the abstract namespace: nothing to unlink.
  bool open(uint64_t chan, int rank, std::string* why);
  // Sends `fd` to the port of (chan, to_rank); `kind` and `from` ride along as payload.
  bool send_fd(uint64_t chan, int to_rank, int fd, uint32_t kind, uint32_t from, std::string* why);
  // Receives one descriptor; false when none arrives within timeout_ms.
  bool recv_fd(int* fd, uint32_t* kind, uint32_t* from, long timeout_ms, std::string* why);

 private:
  int sock_ = -1;
};

}  // namespace hx
