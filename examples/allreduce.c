/* A complete program against the C API in plain C: N ranks (processes forked here, so that no
 * launcher is needed), the unique id handed around through pipes, an Avg AllReduce and a ring
 * shift with Send/Recv inside a group, on host buffers. With device buffers the calls are the
 * same; only the pointers come from cudaMalloc and the last argument is a stream.
 *
 *   gcc -std=c99 -D_POSIX_C_SOURCE=200809L -Iinclude examples/allreduce.c -Lhxccl_b200/lib -lhxccl -Wl,-rpath,$PWD/hxccl_b200/lib -o allreduce
 *   ./allreduce 4
 */
#include <stdio.h>
#include <stdlib.h>
#include <sys/wait.h>
#include <unistd.h>

#include "hxccl.h"

#define CHECK(call)                                                                     \
  do {                                                                                  \
    hxcclResult_t r_ = (call);                                                          \
    if (r_ != hxcclSuccess) {                                                           \
      fprintf(stderr, "rank %d: %s: %s\n", rank, #call, hxcclGetErrorString(r_));       \
      return 2;                                                                         \
    }                                                                                   \
  } while (0)

static int run(int rank, int n, hxcclUniqueId id) {
  enum { COUNT = 1000 };
  hxcclComm_t comm;
  float x[COUNT], shifted[COUNT];
  int i;
  CHECK(hxcclCommInitRank(&comm, n, id, rank));
  for (i = 0; i < COUNT; ++i) x[i] = (float)(rank + 1);
  CHECK(hxcclAllReduce(x, x, COUNT, hxcclFloat32, hxcclAvg, comm, NULL));
  if (x[0] != (float)(n + 1) / 2.0f || x[COUNT - 1] != x[0]) {
    fprintf(stderr, "rank %d: average is %g\n", rank, x[0]);
    return 3;
  }
  CHECK(hxcclGroupStart());
  CHECK(hxcclSend(x, COUNT, hxcclFloat32, (rank + 1) % n, comm, NULL));
  CHECK(hxcclRecv(shifted, COUNT, hxcclFloat32, (rank + n - 1) % n, comm, NULL));
  CHECK(hxcclGroupEnd());
  if (shifted[COUNT / 2] != x[0]) return 4;
  CHECK(hxcclCommDestroy(comm));
  if (rank == 0) printf("%d ranks: average %g, ring shift ok\n", n, x[0]);
  return 0;
}

int main(int argc, char** argv) {
  const int n = argc > 1 ? atoi(argv[1]) : 2;
  int rank, rc, status;
  int(*pipes)[2];
  hxcclUniqueId id;
  if (n < 1 || n > 64) return 1;
  pipes = malloc(sizeof(int[2]) * (size_t)n);
  for (rank = 1; rank < n; ++rank) { /* children first: none inherits the id's listening socket */
    pid_t pid;
    if (pipe(pipes[rank]) != 0) return 1;
    pid = fork();
    if (pid == 0) {
      close(pipes[rank][1]);
      if (read(pipes[rank][0], &id, sizeof id) != (ssize_t)sizeof id) _exit(5);
      _exit(run(rank, n, id));
    }
    close(pipes[rank][0]);
  }
  rank = 0;
  CHECK(hxcclGetUniqueId(&id));
  for (rank = 1; rank < n; ++rank) {
    if (write(pipes[rank][1], &id, sizeof id) != (ssize_t)sizeof id) return 1;
    close(pipes[rank][1]);
  }
  rc = run(0, n, id);
  while (wait(&status) > 0)
    if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) rc = rc ? rc : 6;
  free(pipes);
  return rc;
}
