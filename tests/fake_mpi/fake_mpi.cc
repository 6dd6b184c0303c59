// A one-process stand-in for MPI with working loop-back messages, so that the MPI carrier
// (src/ctrl/mpi_carrier.cc) can be exercised where no MPI is installed: rank 0 of 1, sends to
// self are queued per tag, receives match them in order. It implements the declarations of
// baseline/mpi_stub/mpi.h that the carrier uses; anything else reports failure.
#include <cstring>
#include <deque>
#include <map>
#include <vector>

#include "mpi.h"

namespace {
struct Pending {  // a receive that was posted before its message
  void* buf;
  int room;
  int request;
};
std::map<int, std::deque<std::vector<char>>> g_queue;  // by tag
std::map<int, std::deque<Pending>> g_pending;          // by tag
std::vector<char> g_done(1, 1);                        // request id -> complete (id 0 = MPI_REQUEST_NULL)
int new_request(bool done) {
  g_done.push_back(done ? 1 : 0);
  return int(g_done.size()) - 1;
}
}  // namespace

extern "C" {
int MPI_Comm_size(MPI_Comm, int* n) { *n = 1; return MPI_SUCCESS; }
int MPI_Comm_rank(MPI_Comm, int* r) { *r = 0; return MPI_SUCCESS; }
int MPI_Comm_dup(MPI_Comm, MPI_Comm* o) { *o = 2; return MPI_SUCCESS; }
int MPI_Comm_free(MPI_Comm* c) { *c = MPI_COMM_NULL; return MPI_SUCCESS; }
int MPI_Comm_set_errhandler(MPI_Comm, MPI_Errhandler) { return MPI_SUCCESS; }
int MPI_Isend(const void* b, int n, MPI_Datatype, int peer, int tag, MPI_Comm, MPI_Request* r) {
  if (peer != 0) return MPI_ERR_OTHER;
  auto& waiting = g_pending[tag];
  if (!waiting.empty()) {  // a posted receive takes it at once
    Pending p = waiting.front();
    waiting.pop_front();
    if (n > p.room) return MPI_ERR_OTHER;  // MPI_ERR_TRUNCATE: the carrier never lets this happen
    std::memcpy(p.buf, b, size_t(n));
    g_done[size_t(p.request)] = 1;
  } else {
    g_queue[tag].emplace_back(static_cast<const char*>(b), static_cast<const char*>(b) + n);
  }
  *r = new_request(true);  // buffered: complete at once
  return MPI_SUCCESS;
}
int MPI_Iprobe(int, int tag, MPI_Comm, int* flag, MPI_Status* s) {
  *flag = !g_queue[tag].empty();
  if (*flag && s) s->MPI_SOURCE = 0, s->MPI_TAG = tag, s->MPI_ERROR = MPI_SUCCESS;
  return MPI_SUCCESS;
}
int MPI_Recv(void* b, int n, MPI_Datatype, int, int tag, MPI_Comm, MPI_Status*) {
  auto& q = g_queue[tag];
  if (q.empty() || int(q.front().size()) > n) return MPI_ERR_OTHER;
  std::memcpy(b, q.front().data(), q.front().size());
  q.pop_front();
  return MPI_SUCCESS;
}
int MPI_Irecv(void* b, int n, MPI_Datatype, int, int tag, MPI_Comm, MPI_Request* r) {
  auto& q = g_queue[tag];
  if (!q.empty()) {
    if (int(q.front().size()) > n) return MPI_ERR_OTHER;
    std::memcpy(b, q.front().data(), q.front().size());
    q.pop_front();
    *r = new_request(true);
  } else {
    *r = new_request(false);
    g_pending[tag].push_back(Pending{b, n, *r});
  }
  return MPI_SUCCESS;
}
int MPI_Test(MPI_Request* r, int* flag, MPI_Status*) {
  *flag = g_done[size_t(*r)];
  if (*flag) *r = MPI_REQUEST_NULL;
  return MPI_SUCCESS;
}
int MPI_Testall(int n, MPI_Request* r, int* flag, MPI_Status*) {
  *flag = 1;
  for (int i = 0; i < n; ++i) *flag = *flag && g_done[size_t(r[i])];
  if (*flag)
    for (int i = 0; i < n; ++i) r[i] = MPI_REQUEST_NULL;
  return MPI_SUCCESS;
}
int MPI_Wait(MPI_Request* r, MPI_Status*) { return g_done[size_t(*r)] ? MPI_SUCCESS : MPI_ERR_OTHER; }
int MPI_Waitall(int n, MPI_Request* r, MPI_Status*) {
  for (int i = 0; i < n; ++i)
    if (!g_done[size_t(r[i])]) return MPI_ERR_OTHER;  // would block for ever in one process
  return MPI_SUCCESS;
}
int MPI_Bcast(void*, int, MPI_Datatype, int, MPI_Comm) { return MPI_SUCCESS; }  // one rank: nothing to do
int MPI_Error_string(int e, char* s, int* n) {
  std::strcpy(s, e == MPI_SUCCESS ? "no error" : "loop-back MPI: failed");
  *n = int(std::strlen(s));
  return MPI_SUCCESS;
}
}
