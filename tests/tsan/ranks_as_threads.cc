// The ranks of one communicator as threads of one process, on host buffers: under
// ThreadSanitizer (python -m hxccl_b200.build --tsan) this shows data races in what the ranks
// share inside a process (the unique-id listeners, the operator tags, the lazily built tables
// of the reduce loops) and in the transport's hand-overs, which separate processes never show.
// Also runs two threads against ONE communicator handle's fabric through a parent and its Split
// child, which share their connections.
//
//   build/ranks_as_threads [ranks]        exit code 0 = every result right
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "hxccl.h"

namespace {
std::atomic<int> failures{0};
#define EXPECT(cond)                                                        \
  do {                                                                      \
    if (!(cond)) {                                                          \
      std::fprintf(stderr, "rank %d: %s failed (line %d)\n", rank, #cond, __LINE__); \
      ++failures;                                                           \
    }                                                                       \
  } while (0)

void rank_main(int rank, int n, hxcclUniqueId id) {
  hxcclComm_t comm = nullptr;
  EXPECT(hxcclCommInitRank(&comm, n, id, rank) == hxcclSuccess);
  if (!comm) return;
  // sums of floats and of 8-bit floats (the pair tables are built on first use, by whoever comes first)
  const size_t count = 300000;
  std::vector<float> x(count, float(rank + 1)), y(count);
  EXPECT(hxcclAllReduce(x.data(), y.data(), count, hxcclFloat32, hxcclSum, comm, nullptr) == hxcclSuccess);
  EXPECT(y[0] == float(n * (n + 1) / 2) && y[count - 1] == y[0]);
  std::vector<unsigned char> q(8192, 0x38), r8(8192);  // 1.0 in e4m3
  EXPECT(hxcclAllReduce(q.data(), r8.data(), q.size(), hxcclFloat8e4m3, hxcclMax, comm, nullptr) == hxcclSuccess);
  EXPECT(r8[0] == 0x38 && r8[8191] == 0x38);
  // an operator per rank, made and dropped concurrently
  float half = 0.5f;
  hxcclRedOp_t op;
  EXPECT(hxcclRedOpCreatePreMulSum(&op, &half, hxcclFloat32, hxcclScalarHostImmediate, comm) == hxcclSuccess);
  std::vector<float> s(64, 2.0f);
  EXPECT(hxcclAllReduce(s.data(), s.data(), s.size(), hxcclFloat32, op, comm, nullptr) == hxcclSuccess);
  EXPECT(s[0] == float(n));
  EXPECT(hxcclRedOpDestroy(op, comm) == hxcclSuccess);
  // a ring shift inside a group, large enough to arrive ahead of its receive
  std::vector<int> out(1 << 18, rank), in(1 << 18, -1);
  EXPECT(hxcclGroupStart() == hxcclSuccess);
  EXPECT(hxcclSend(out.data(), out.size(), hxcclInt32, (rank + 1) % n, comm, nullptr) == hxcclSuccess);
  EXPECT(hxcclRecv(in.data(), in.size(), hxcclInt32, (rank + n - 1) % n, comm, nullptr) == hxcclSuccess);
  EXPECT(hxcclGroupEnd() == hxcclSuccess);
  EXPECT(in[0] == (rank + n - 1) % n && in.back() == in[0]);
  // parent and child communicators share the connections: use both from two threads at once
  hxcclComm_t child = nullptr;
  EXPECT(hxcclCommSplit(comm, 0, rank, &child, nullptr) == hxcclSuccess);
  if (child) {
    std::vector<double> a(50000, 1.0), b(50000, 2.0);
    std::thread other([&] {
      for (int i = 0; i < 5; ++i)
        if (hxcclAllReduce(b.data(), b.data(), b.size(), hxcclFloat64, hxcclMax, child, nullptr) != hxcclSuccess) ++failures;
    });
    for (int i = 0; i < 5; ++i)
      EXPECT(hxcclAllReduce(a.data(), a.data(), a.size(), hxcclFloat64, hxcclMin, comm, nullptr) == hxcclSuccess);
    other.join();
    EXPECT(a[0] == 1.0 && b[0] == 2.0);
    EXPECT(hxcclCommDestroy(child) == hxcclSuccess);
  }
  EXPECT(hxcclCommDestroy(comm) == hxcclSuccess);
}
}  // namespace

int main(int argc, char** argv) {
  const int n = argc > 1 ? std::atoi(argv[1]) : 4;
  setenv("HXCCL_DEVICE", "0", 1);  // host buffers only
  hxcclUniqueId id;
  if (hxcclGetUniqueId(&id) != hxcclSuccess) return 2;
  std::vector<std::thread> ranks;
  for (int r = 0; r < n; ++r) ranks.emplace_back(rank_main, r, n, id);
  for (auto& t : ranks) t.join();
  std::printf("%d ranks as threads: %d failures\n", n, failures.load());
  return failures.load() ? 1 : 0;
}
