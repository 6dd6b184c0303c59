// Drives the MPI carrier through the loop-back MPI of fake_mpi.cc (one process, messages to
// self): matching by (channel, tag) in posting order, early messages, truncation, empty
// messages, withdrawn receives, and a whole communicator created with hxcclCommInitMPI whose
// host collectives then run over it. Prints "ok" and exits 0 when everything holds.
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "ctrl/mpi_carrier.h"
#include "hxccl.h"

#define EXPECT(cond)                                                  \
  do {                                                                \
    if (!(cond)) {                                                    \
      std::printf("FAILED line %d: %s\n", __LINE__, #cond);           \
      return 1;                                                       \
    }                                                                 \
  } while (0)

int main() {
  using namespace hx;
  auto carrier = std::make_shared<MpiCarrier>(MPI_COMM_WORLD);
  EXPECT(carrier->ok() && carrier->self() == 0 && carrier->nprocs() == 1);
  std::string why;
  // receive first, then the message
  char in[64] = {}, msg[] = "hello over mpi";
  int r = carrier->post_recv(0, 11, 0, in, sizeof in);
  int s = carrier->post_send(0, 11, 0, msg, sizeof msg);
  EXPECT(carrier->wait_ticket(s, &why) == hxcclSuccess && carrier->wait_ticket(r, &why) == hxcclSuccess);
  EXPECT(std::strcmp(in, msg) == 0);
  // messages first (parked), on two channels with the same tag, then receives in the other order
  char a[] = "for channel A", b[] = "for channel B", got_a[32] = {}, got_b[32] = {};
  int sa = carrier->post_send(0, 100, 5, a, sizeof a), sb = carrier->post_send(0, 200, 5, b, sizeof b);
  EXPECT(carrier->wait_ticket(sa, &why) == hxcclSuccess && carrier->wait_ticket(sb, &why) == hxcclSuccess);
  int rb = carrier->post_recv(0, 200, 5, got_b, sizeof got_b), ra = carrier->post_recv(0, 100, 5, got_a, sizeof got_a);
  EXPECT(carrier->wait_ticket(rb, &why) == hxcclSuccess && carrier->wait_ticket(ra, &why) == hxcclSuccess);
  EXPECT(std::strcmp(got_a, a) == 0 && std::strcmp(got_b, b) == 0);
  // two messages of one (channel, tag) arrive in posting order
  int one = 1, two = 2, first = 0, second = 0;
  int s1 = carrier->post_send(0, 7, 1, &one, sizeof one), s2 = carrier->post_send(0, 7, 1, &two, sizeof two);
  int r1 = carrier->post_recv(0, 7, 1, &first, sizeof first), r2 = carrier->post_recv(0, 7, 1, &second, sizeof second);
  for (int t : {s1, s2, r1, r2}) EXPECT(carrier->wait_ticket(t, &why) == hxcclSuccess);
  EXPECT(first == 1 && second == 2);
  // a message longer than its receive: the leading bytes arrive, the receive fails, the sender does not
  char big[100], small[40];
  std::memset(big, 'x', sizeof big);
  std::memset(small, 0, sizeof small);
  int rt = carrier->post_recv(0, 9, 0, small, sizeof small), st = carrier->post_send(0, 9, 0, big, sizeof big);
  EXPECT(carrier->wait_ticket(st, &why) == hxcclSuccess);
  EXPECT(carrier->wait_ticket(rt, &why) == hxcclSystemError && why.find("truncated") != std::string::npos);
  EXPECT(small[0] == 'x' && small[39] == 'x');
  // ... also when the message was there first
  std::memset(small, 0, sizeof small);
  st = carrier->post_send(0, 9, 0, big, sizeof big);
  EXPECT(carrier->wait_ticket(st, &why) == hxcclSuccess);
  rt = carrier->post_recv(0, 9, 0, small, sizeof small);
  EXPECT(carrier->wait_ticket(rt, &why) == hxcclSystemError && small[39] == 'x');
  // an empty message still matches
  int re = carrier->post_recv(0, 9, 3, nullptr, 0), se = carrier->post_send(0, 9, 3, nullptr, 0);
  EXPECT(carrier->wait_ticket(se, &why) == hxcclSuccess && carrier->wait_ticket(re, &why) == hxcclSuccess);
  // a withdrawn receive does not swallow the next message
  int lost = carrier->post_recv(0, 42, 0, in, sizeof in);
  carrier->cancel(lost);
  int value = 77, seen = 0;
  int sv = carrier->post_send(0, 42, 0, &value, sizeof value);
  int rv = carrier->post_recv(0, 42, 0, &seen, sizeof seen);
  EXPECT(carrier->wait_ticket(sv, &why) == hxcclSuccess && carrier->wait_ticket(rv, &why) == hxcclSuccess && seen == 77);
  // a lost peer fails what involves it
  carrier->sever(0);
  int dead = carrier->post_send(0, 1, 0, &value, sizeof value);
  EXPECT(carrier->wait_ticket(dead, &why) == hxcclSystemError);

  // a communicator over MPI: the API's host path end to end (one rank)
  hxcclComm_t comm = nullptr;
  EXPECT(hxcclCommInitMPI(&comm, MPI_COMM_WORLD) == hxcclSuccess && comm);
  int n = 0, me = -1;
  EXPECT(hxcclCommCount(comm, &n) == hxcclSuccess && n == 1 && hxcclCommUserRank(comm, &me) == hxcclSuccess && me == 0);
  float x[5] = {1, 2, 3, 4, 5}, y[5] = {};
  EXPECT(hxcclAllReduce(x, y, 5, hxcclFloat32, hxcclSum, comm, nullptr) == hxcclSuccess && y[4] == 5.0f);
  EXPECT(hxcclGroupStart() == hxcclSuccess);
  EXPECT(hxcclSend(x, 5, hxcclFloat32, 0, comm, nullptr) == hxcclSuccess);
  float z[5] = {};
  EXPECT(hxcclRecv(z, 5, hxcclFloat32, 0, comm, nullptr) == hxcclSuccess);
  EXPECT(hxcclGroupEnd() == hxcclSuccess && z[2] == 3.0f);
  EXPECT(hxcclCommDestroy(comm) == hxcclSuccess);
  std::printf("ok\n");
  return 0;
}
