// hx_perf: collective sweep in the style of nccl-tests, one process per GPU, no MPI and no
// Python on the timed path (so small-message figures show launch + device latency, not
// interpreter overhead). The program forks its own ranks, hands the unique id around through
// pipes, and times with CUDA events between barriers; every figure is the maximum over ranks.
//
//   hx_perf -g 8 [-o allreduce|allgather|reducescatter|alltoall|broadcast|reduce|gather|scatter|sendrecv]
//           [-b 8] [-e 1073741824] [-f 2] [-n 20] [-w 5] [-t float|bf16|half|int32|...] [-r sum|max|avg|...]
//           [-H]   host buffers instead of device buffers
//           [-I nccl]  time NCCL instead (libnccl.so.2 found by the loader, or the file named by
//                      HX_PERF_NCCL_LIB), same processes, buffers, barriers and timing, so that
//                      both libraries are measured without an interpreter; allreduce, allgather,
//                      reducescatter, broadcast, reduce, alltoall and sendrecv
//
// Plays the role of the reference's bench/hxccl_perf.cc:53-205 (which compares with MPI and
// times on the host, valid there because its calls block).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <sys/wait.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "hxccl.h"
#include "hxccl_ext.h"

namespace {
#define CK(x)                                                                              \
  do {                                                                                     \
    hxcclResult_t r_ = (x);                                                                \
    if (r_ != hxcclSuccess) {                                                              \
      std::fprintf(stderr, "[rank %d] %s failed: %s (%s)\n", g_rank, #x, hxcclGetErrorString(r_), \
                   g_comm ? hxcclGetLastError(g_comm) : "");                               \
      std::exit(2);                                                                        \
    }                                                                                      \
  } while (0)
int g_rank = 0;
hxcclComm_t g_comm = nullptr;

// The few NCCL entry points the comparison arm needs, resolved at run time so that the tool
// builds and runs where NCCL is absent. Types and values follow nccl.h (ncclDataType_t and
// ncclRedOp_t share hxccl's numbering, which is NCCL's).
struct Nccl {
  void* so = nullptr;
  int (*GetUniqueId)(void*) = nullptr;
  int (*CommInitRank)(void**, int, hxcclUniqueId, int) = nullptr;  // ncclUniqueId is 128 bytes too
  int (*CommDestroy)(void*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*Reduce)(const void*, void*, size_t, int, int, int, void*, cudaStream_t) = nullptr;
  int (*Send)(const void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  void* comm = nullptr;
  bool load() {
    const char* path = std::getenv("HX_PERF_NCCL_LIB");
    so = dlopen(path && *path ? path : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!so) {
      std::fprintf(stderr, "cannot load NCCL: %s\n", dlerror());
      return false;
    }
    auto sym = [&](const char* name) { return dlsym(so, name); };
#define HX_NCCL_SYM(field, name) field = reinterpret_cast<decltype(field)>(sym(name))
    HX_NCCL_SYM(GetUniqueId, "ncclGetUniqueId");
    HX_NCCL_SYM(CommInitRank, "ncclCommInitRank");
    HX_NCCL_SYM(CommDestroy, "ncclCommDestroy");
    HX_NCCL_SYM(AllReduce, "ncclAllReduce");
    HX_NCCL_SYM(AllGather, "ncclAllGather");
    HX_NCCL_SYM(ReduceScatter, "ncclReduceScatter");
    HX_NCCL_SYM(Broadcast, "ncclBroadcast");
    HX_NCCL_SYM(Reduce, "ncclReduce");
    HX_NCCL_SYM(Send, "ncclSend");
    HX_NCCL_SYM(Recv, "ncclRecv");
    HX_NCCL_SYM(GroupStart, "ncclGroupStart");
    HX_NCCL_SYM(GroupEnd, "ncclGroupEnd");
#undef HX_NCCL_SYM
    return GetUniqueId && CommInitRank && CommDestroy && AllReduce && AllGather && ReduceScatter && Broadcast &&
           Reduce && Send && Recv && GroupStart && GroupEnd;
  }
};
Nccl g_nccl;
#define NK(x)                                                                   \
  do {                                                                          \
    const int r_ = (x);                                                         \
    if (r_ != 0) {                                                              \
      std::fprintf(stderr, "[rank %d] %s failed: NCCL result %d\n", g_rank, #x, r_); \
      std::exit(2);                                                             \
    }                                                                           \
  } while (0)

struct Options {
  bool nccl = false;
  int gpus = 1;
  std::string op = "allreduce", type = "float", red = "sum";
  size_t min_bytes = 8, max_bytes = size_t(1) << 30;
  int factor = 2, iters = 20, warmup = 5;
  bool host = false;
};

hxcclDataType_t parse_type(const std::string& t, size_t* es) {
  struct { const char* n; hxcclDataType_t d; size_t s; } tab[] = {
      {"int8", hxcclInt8, 1}, {"uint8", hxcclUint8, 1}, {"int32", hxcclInt32, 4}, {"uint32", hxcclUint32, 4},
      {"int64", hxcclInt64, 8}, {"uint64", hxcclUint64, 8}, {"half", hxcclFloat16, 2}, {"float", hxcclFloat32, 4},
      {"double", hxcclFloat64, 8}, {"bf16", hxcclBfloat16, 2}, {"fp8e4m3", hxcclFloat8e4m3, 1}, {"fp8e5m2", hxcclFloat8e5m2, 1}};
  for (auto& e : tab)
    if (t == e.n) {
      *es = e.s;
      return e.d;
    }
  std::fprintf(stderr, "unknown type %s\n", t.c_str());
  std::exit(1);
}
hxcclRedOp_t parse_red(const std::string& r) {
  if (r == "sum") return hxcclSum;
  if (r == "prod") return hxcclProd;
  if (r == "max") return hxcclMax;
  if (r == "min") return hxcclMin;
  if (r == "avg") return hxcclAvg;
  std::fprintf(stderr, "unknown op %s\n", r.c_str());
  std::exit(1);
}

int run_rank(const Options& o, int rank, const hxcclUniqueId& id, const hxcclUniqueId& nccl_id) {
  g_rank = rank;
  const int n = o.gpus;
  // the NCCL arm keeps an hxccl communicator for the host-side barriers only: no device path
  if (o.nccl) setenv("HXCCL_DEVICE", "0", 1);
  if (!o.host) {
    int ndev = 0;
    cudaGetDeviceCount(&ndev);
    if (ndev < 1) {
      std::fprintf(stderr, "no CUDA device\n");
      return 2;
    }
    cudaSetDevice(rank % ndev);
    cudaFree(nullptr);
  }
  CK(hxcclCommInitRank(&g_comm, n, id, rank));
  if (o.nccl) NK(g_nccl.CommInitRank(&g_nccl.comm, n, nccl_id, rank));
  size_t es = 4;
  const hxcclDataType_t dt = parse_type(o.type, &es);
  const hxcclRedOp_t red = parse_red(o.red);
  const bool gathers = o.op == "allgather" || o.op == "gather";
  const bool scatters = o.op == "reducescatter" || o.op == "alltoall" || o.op == "scatter";
  const size_t cap = o.max_bytes + 256;  // `bytes` is the larger side of every collective here
  char *send = nullptr, *recv = nullptr;
  if (o.host) {
    send = static_cast<char*>(std::malloc(cap));
    recv = static_cast<char*>(std::malloc(cap));
    std::memset(send, 1, cap);
  } else {
    cudaMalloc(&send, cap);
    cudaMalloc(&recv, cap);
    cudaMemset(send, 1, cap);
  }
  cudaStream_t st = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (!o.host) {
    cudaStreamCreate(&st);
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
  }
  char kind[32] = "host";
  if (!o.host) hxcclCommDeviceInfo(g_comm, kind, sizeof kind, nullptr, nullptr);
  if (o.nccl) std::snprintf(kind, sizeof kind, "nccl");
  if (rank == 0)
    std::printf("# hx_perf  op=%s type=%s red=%s ranks=%d buffers=%s path=%s iters=%d warmup=%d\n"
                "# %12s %12s %12s %12s %12s\n",
                o.op.c_str(), o.type.c_str(), o.red.c_str(), n, o.host ? "host" : "device", kind, o.iters, o.warmup,
                "bytes", "count", "time(us)", "algbw(GB/s)", "busbw(GB/s)");
  for (size_t bytes = o.min_bytes; bytes <= o.max_bytes; bytes *= o.factor) {
    // `bytes` is the nccl-tests size: the full vector for allreduce/broadcast/sendrecv, the
    // gathered / scattered total for the others
    const size_t count = std::max<size_t>(1, bytes / es / (gathers || scatters ? n : 1));
    auto call = [&]() {
      if (o.nccl) {
        void* c = g_nccl.comm;
        if (o.op == "allreduce") NK(g_nccl.AllReduce(send, recv, count, dt, red, c, st));
        else if (o.op == "allgather") NK(g_nccl.AllGather(send, recv, count, dt, c, st));
        else if (o.op == "reducescatter") NK(g_nccl.ReduceScatter(send, recv, count, dt, red, c, st));
        else if (o.op == "broadcast") NK(g_nccl.Broadcast(send, recv, count, dt, 0, c, st));
        else if (o.op == "reduce") NK(g_nccl.Reduce(send, recv, count, dt, red, 0, c, st));
        else if (o.op == "alltoall") {
          NK(g_nccl.GroupStart());
          for (int p = 0; p < n; ++p) {
            NK(g_nccl.Send(send + size_t(p) * count * es, count, dt, p, c, st));
            NK(g_nccl.Recv(recv + size_t(p) * count * es, count, dt, p, c, st));
          }
          NK(g_nccl.GroupEnd());
        } else if (o.op == "sendrecv") {
          NK(g_nccl.GroupStart());
          NK(g_nccl.Send(send, count, dt, (rank + 1) % n, c, st));
          NK(g_nccl.Recv(recv, count, dt, (rank + n - 1) % n, c, st));
          NK(g_nccl.GroupEnd());
        } else {
          std::fprintf(stderr, "the NCCL arm has no %s\n", o.op.c_str());
          std::exit(1);
        }
        return;
      }
      if (o.op == "allreduce") CK(hxcclAllReduce(send, recv, count, dt, red, g_comm, st));
      else if (o.op == "allgather") CK(hxcclAllGather(send, recv, count, dt, g_comm, st));
      else if (o.op == "reducescatter") CK(hxcclReduceScatter(send, recv, count, dt, red, g_comm, st));
      else if (o.op == "alltoall") CK(hxcclAlltoAll(send, recv, count, dt, g_comm, st));
      else if (o.op == "broadcast") CK(hxcclBroadcast(send, recv, count, dt, 0, g_comm, st));
      else if (o.op == "reduce") CK(hxcclReduce(send, recv, count, dt, red, 0, g_comm, st));
      else if (o.op == "gather") CK(hxcclGather(send, recv, count, dt, 0, g_comm, st));
      else if (o.op == "scatter") CK(hxcclScatter(send, recv, count, dt, 0, g_comm, st));
      else if (o.op == "sendrecv") {
        CK(hxcclGroupStart());
        CK(hxcclSend(send, count, dt, (rank + 1) % n, g_comm, st));
        CK(hxcclRecv(recv, count, dt, (rank + n - 1) % n, g_comm, st));
        CK(hxcclGroupEnd());
      } else {
        std::fprintf(stderr, "unknown collective %s\n", o.op.c_str());
        std::exit(1);
      }
    };
    auto barrier = [&]() {
      if (!o.host) cudaStreamSynchronize(st);
      int one = 1, out = 0;
      CK(hxcclAllReduce(&one, &out, 1, hxcclInt32, hxcclSum, g_comm, nullptr));  // host path
    };
    for (int i = 0; i < o.warmup; ++i) call();
    barrier();
    const int iters = bytes <= (1u << 20) ? o.iters * 5 : o.iters;
    float ms = 0;
    timespec t0{}, t1{};
    if (o.host) clock_gettime(CLOCK_MONOTONIC, &t0); else cudaEventRecord(e0, st);
    for (int i = 0; i < iters; ++i) call();
    if (o.host) {
      clock_gettime(CLOCK_MONOTONIC, &t1);
      ms = float((t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6);
    } else {
      cudaEventRecord(e1, st);
      cudaEventSynchronize(e1);
      cudaEventElapsedTime(&ms, e0, e1);
    }
    float us = ms * 1e3f / iters, worst = 0;
    CK(hxcclAllReduce(&us, &worst, 1, hxcclFloat32, hxcclMax, g_comm, nullptr));
    const double moved = double(count) * es * (gathers || scatters ? n : 1);
    const double algbw = moved / (worst * 1e-6) / 1e9;
    const double f = o.op == "allreduce" ? 2.0 * (n - 1) / n
                     : (o.op == "broadcast" || o.op == "sendrecv" || o.op == "reduce") ? 1.0 : double(n - 1) / n;
    if (rank == 0)
      std::printf("  %12zu %12zu %12.2f %12.2f %12.2f\n", size_t(moved), count, worst, algbw, algbw * f);
    barrier();
  }
  hxcclResult_t async = hxcclSuccess;
  hxcclCommGetAsyncError(g_comm, &async);
  if (async != hxcclSuccess) std::fprintf(stderr, "[rank %d] asynchronous error: %s\n", rank, hxcclGetLastError(g_comm));
  if (o.nccl) {
    cudaStreamSynchronize(st);
    NK(g_nccl.CommDestroy(g_nccl.comm));
  }
  CK(hxcclCommDestroy(g_comm));
  return async == hxcclSuccess ? 0 : 3;
}
}  // namespace

int main(int argc, char** argv) {
  Options o;
  for (int c; (c = getopt(argc, argv, "g:o:b:e:f:n:w:t:r:HI:")) != -1;) {
    switch (c) {
      case 'g': o.gpus = std::atoi(optarg); break;
      case 'o': o.op = optarg; break;
      case 'b': o.min_bytes = std::strtoull(optarg, nullptr, 10); break;
      case 'e': o.max_bytes = std::strtoull(optarg, nullptr, 10); break;
      case 'f': o.factor = std::max(2, std::atoi(optarg)); break;
      case 'n': o.iters = std::atoi(optarg); break;
      case 'w': o.warmup = std::atoi(optarg); break;
      case 't': o.type = optarg; break;
      case 'r': o.red = optarg; break;
      case 'H': o.host = true; break;
      case 'I': o.nccl = std::string(optarg) == "nccl"; break;
      default: std::fprintf(stderr, "see the header of bench/hx_perf.cc for usage\n"); return 1;
    }
  }
  if (o.gpus < 1 || o.min_bytes < 1 || o.max_bytes < o.min_bytes) return 1;
  if (o.nccl && (o.host || !g_nccl.load())) return 1;
  // rank 0 is this process; the id reaches each child through its own pipe (fork comes first,
  // so that no child inherits a CUDA context or the id's listening socket)
  std::vector<int> wr(o.gpus, -1);
  std::vector<pid_t> kids;
  for (int r = 1; r < o.gpus; ++r) {
    int p[2];
    if (pipe(p) != 0) return 1;
    const pid_t pid = fork();
    if (pid == 0) {
      close(p[1]);
      hxcclUniqueId id, nid;
      if (read(p[0], &id, sizeof id) != ssize_t(sizeof id)) _exit(2);
      if (read(p[0], &nid, sizeof nid) != ssize_t(sizeof nid)) _exit(2);
      _exit(run_rank(o, r, id, nid));
    }
    close(p[0]);
    wr[r] = p[1];
    kids.push_back(pid);
  }
  hxcclUniqueId id, nid;
  std::memset(&nid, 0, sizeof nid);
  if (hxcclGetUniqueId(&id) != hxcclSuccess) return 2;
  if (o.nccl && g_nccl.GetUniqueId(&nid) != 0) return 2;
  for (int r = 1; r < o.gpus; ++r) {
    if (write(wr[r], &id, sizeof id) != ssize_t(sizeof id)) return 2;
    if (write(wr[r], &nid, sizeof nid) != ssize_t(sizeof nid)) return 2;
    close(wr[r]);
  }
  int rc = run_rank(o, 0, id, nid);
  for (pid_t k : kids) {
    int status = 0;
    waitpid(k, &status, 0);
    if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) rc = rc ? rc : 4;
  }
  return rc;
}
