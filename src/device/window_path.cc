#include "device/window_path.h"

#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>

#include "ctrl/fdpass.h"
#include "device/cudrv.h"
#include "math/dtypes.h"

namespace hx {
namespace {

size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

long env_long(const char* name, long dflt) {
  const char* e = std::getenv(name);
  if (!e || !*e) return dflt;
  char* end = nullptr;
  const long v = std::strtol(e, &end, 10);
  return *end ? dflt : v;
}

// identifies the machine (one kernel boot), so that ranks can tell whether they share it
uint64_t host_fingerprint() {
  std::ifstream f("/proc/sys/kernel/random/boot_id");
  std::string s;
  std::getline(f, s);
  char name[256] = {};
  gethostname(name, sizeof name - 1);
  s += name;
  uint64_t h = 1469598103934665603ull;
  for (unsigned char ch : s) h = (h ^ ch) * 1099511628211ull;
  return h;
}

struct RankFacts {
  uint64_t host;
  int device;
  int multicast;  // device attribute
  int fd_handles;  // POSIX fd export supported
  int chunk16;     // HXCCL_IPC_CHUNK in 16-byte units, 0 = not set
};

// HXCCL_IPC_CHUNK of the reference is the size of its staging buffers, so every transfer moves
// in pieces of at most that many bytes (src/memspace_cuda.cc:25-34: 64 B .. 1 GiB, anything
// else means the default; the ranks use the smallest wish, src/transport_ipc.cc:93-98). Here
// it bounds the bytes a CTA moves per pipelined step the same way; unset leaves the tuner's
// own sizes.
int chunk_wish16() {
  const char* e = std::getenv("HXCCL_IPC_CHUNK");
  if (!e || !*e) return 0;
  char* end = nullptr;
  const long long v = std::strtoll(e, &end, 10);
  if (end == e || *end || v < 64 || v > (1LL << 30)) return 0;
  return int(v / 16);
}

}  // namespace

WindowPath::WindowPath(hxcclComm* c) : c_(c), rank_(c->rank), n_(c->nranks) {}

WindowPath::~WindowPath() { release(); }

hxcclResult_t WindowPath::fail(hxcclResult_t r, const std::string& why) {
  error = why;
  return r;
}

bool WindowPath::agree(bool ok) {
  int bad = ok ? 0 : 1;
  if (c_->chan->max_int(&bad) != hxcclSuccess) return false;
  return bad == 0;
}

// Tuning knobs, the status words and (single rank) a plain local window.
hxcclResult_t WindowPath::setup_local() {
  if (cudaGetDevice(&dev_) != cudaSuccess) return fail(hxcclUnhandledCudaError, "no current CUDA device");
  if (cudaFree(nullptr) != cudaSuccess) return fail(hxcclUnhandledCudaError, "cannot create a CUDA context");
  if (cudaHostAlloc(reinterpret_cast<void**>(&status_), 64, cudaHostAllocMapped) != cudaSuccess)
    return fail(hxcclUnhandledCudaError, "cannot allocate the pinned status words");
  std::memset(status_, 0, 64);
  if (cudaEventCreateWithFlags(&order_event_, cudaEventDisableTiming) != cudaSuccess)
    return fail(hxcclUnhandledCudaError, "cannot create an event");
  Tuning& t = eng_.tune;
  load_default_table(&t);
  t.use_table = env_long("HXCCL_TUNE_TABLE", 1) != 0;
  t.max_ctas = int(std::max(1L, std::min<long>(env_long("HXCCL_MAX_CTAS", t.max_ctas), kMaxCtas)));
  t.threads = int(env_long("HXCCL_THREADS", 0));
  if (t.threads != 256 && t.threads != 512) t.threads = 0;
  t.max_ctas = std::min(t.max_ctas, max_resident_ctas(t.threads ? t.threads : 512));
  t.min_steps = int(std::max(2L, env_long("HXCCL_MIN_STEPS", t.min_steps)));
  t.sm_count = max_resident_ctas(512);
  t.roles_min_ranks = int(std::max(2L, env_long("HXCCL_ROLES_MIN_RANKS", t.roles_min_ranks)));
  t.oneshot_max = size_t(env_long("HXCCL_ONESHOT_MAX", long(t.oneshot_max)));
  t.nvls_min = size_t(env_long("HXCCL_NVLS_MIN", long(t.nvls_min)));
  t.single_sub_max = size_t(env_long("HXCCL_SINGLE_SUB_MAX", long(t.single_sub_max)));
  t.sub_max = size_t(std::max(16L, env_long("HXCCL_SUB_MAX", long(t.sub_max)) / 16 * 16));
  t.roles_min = size_t(env_long("HXCCL_ROLES_MIN", long(t.roles_min)));
  t.roles_sub = size_t(std::max(16L, env_long("HXCCL_ROLES_SUB", long(t.roles_sub))));
  t.ring_min = size_t(std::max(0L, env_long("HXCCL_RING_MIN", long(t.ring_min))));
  t.ring_sub = size_t(std::max(16L, env_long("HXCCL_RING_SUB", long(t.ring_sub)) / 16 * 16));
  t.p2p_threads = env_long("HXCCL_P2P_THREADS", t.p2p_threads) == 512 ? 512 : 256;
  t.p2p_bulk = env_long("HXCCL_P2P_BULK", t.p2p_bulk ? 1 : 0) != 0;
  t.ring_max_ranks = int(std::max(2L, env_long("HXCCL_RING_MAX_RANKS", t.ring_max_ranks)));
  t.exact = env_long("HXCCL_EXACT", 1) != 0;
  t.nvls_gather = env_long("HXCCL_NVLS_GATHER", 1) != 0;
  if (const char* path = std::getenv("HXCCL_TUNE_FILE")) {  // applied last, so a file wins
    std::string why;
    if (!load_tune_file(&t, path, &why)) return fail(hxcclInvalidArgument, why);
    t.max_ctas = std::min(t.max_ctas, max_resident_ctas(t.threads ? t.threads : 512));
  }
  if (const char* v = std::getenv("HXCCL_VARIANT")) {
    if (!std::strcmp(v, "oneshot")) eng_.forced_variant = kVarOneShot;
    if (!std::strcmp(v, "twoshot")) eng_.forced_variant = kVarTwoShot;
    if (!std::strcmp(v, "nvls")) eng_.forced_variant = kVarNvls;
    if (!std::strcmp(v, "ring")) eng_.forced_variant = kVarRing;
    if (!std::strcmp(v, "lines")) eng_.forced_variant = kVarLL;
  }
  t.ll_max = size_t(std::max(0L, env_long("HXCCL_LL_MAX", long(t.ll_max))));
  t.ll_mc = env_long("HXCCL_LL_MC", 1) != 0;
  t.mc_copy = env_long("HXCCL_MC_COPY", 1) != 0;
  {
    const long f = env_long("HXCCL_MC_FORCE", -1);
    t.mc_force = f < 0 ? -1 : (f != 0);
  }
  t.rs_ring_min = size_t(std::max(0L, env_long("HXCCL_RS_RING_MIN", long(t.rs_ring_min))));
  return hxcclSuccess;
}

hxcclResult_t WindowPath::init() {
  const bool local_ok = setup_local() == hxcclSuccess;
  if (!agree(local_ok)) return fail(hxcclUnhandledCudaError, local_ok ? "a peer has no usable GPU" : error);
  hxcclResult_t r = setup_windows();
  if (r != hxcclSuccess) return r;
  setup_multicast();

  WinView w{};
  for (int p = 0; p < n_; ++p) w.win[p] = reinterpret_cast<char*>(va_[p]);
  w.mc = nvls_ ? reinterpret_cast<char*>(mc_va_) : nullptr;
  w.status = status_;
  w.soft = status_ + 1;
  const size_t p2p_bytes = round_up(p2p_region_bytes(n_, p2p_slot_), 1u << 20);
  const size_t half = (win_bytes_ - kHeaderBytes - p2p_bytes) / 2 / 4096 * 4096;
  w.p2p_slot = p2p_slot_;
  w.half_off[0] = kHeaderBytes + p2p_bytes;
  w.half_off[1] = w.half_off[0] + half;
  w.half_bytes = half;
  w.wait_ns = uint64_t(std::max(1L, env_long("HXCCL_WAIT_LIMIT_MS", 20000))) * 1000000ull;
  w.rank = rank_;
  w.n = n_;
  if (env_long("HXCCL_TRACE", 0) != 0) {
    const size_t bytes = size_t(kMaxCtas) * kTraceSlots * sizeof(unsigned long long);
    if (cudaMalloc(reinterpret_cast<void**>(&trace_), bytes) == cudaSuccess) cudaMemset(trace_, 0, bytes);
  }
  w.trace = trace_;
  eng_.views.assign(1, w);
  eng_.tune.nvls = nvls_;
  if (std::getenv("HXCCL_DEBUG") && rank_ == 0)
    std::fprintf(stderr, "hxccl: device path %s, %d ranks, window %zu MiB, staging 2 x %zu MiB, max %d CTAs\n",
                 kind(), n_, win_bytes_ >> 20, half >> 20, eng_.tune.max_ctas);
  return hxcclSuccess;
}

hxcclResult_t WindowPath::setup_windows() {
  const CuDriver& d = cu();
  // A communicator made from scratch stages through 512 MiB and moves Send/Recv payload in
  // 1 MiB slots; one made by Split / Shrink gets a quarter of both unless told otherwise, so
  // that many sub-communicators stay affordable (large messages take more pipelined steps,
  // nothing else changes). The values are the same on every rank of a communicator: every
  // rank reads them from the same kind of communicator, and the smallest wish wins below.
  const bool child = c_->device.derived;
  long win_mb = env_long(child ? "HXCCL_CHILD_WINDOW_MB" : "HXCCL_WINDOW_MB", child ? 128 : 512);
  // Send/Recv slots of 1 MiB measured 516 GB/s for a 256 MiB ring shift on two GPUs against 424 with
  // 512 KiB and 301 with 256 KiB: the hand-shake per piece is what a lane pays for
  long slot_kb = env_long(child ? "HXCCL_CHILD_P2P_SLOT_KB" : "HXCCL_P2P_SLOT_KB", child ? 256 : 1024);
  {
    int neg[2] = {int(-std::max(2L, win_mb)), int(-std::max(16L, std::min(slot_kb, 4096L)))};
    if (c_->chan->max_int(&neg[0]) != hxcclSuccess || c_->chan->max_int(&neg[1]) != hxcclSuccess)
      return fail(hxcclSystemError, "window size agreement failed: " + c_->chan->error);
    win_mb = -neg[0];
    slot_kb = -neg[1];
  }
  p2p_slot_ = size_t(slot_kb) * 1024 / 16 * 16;
  const long half_mb = std::max(1L, win_mb / 2);
  const size_t want = kHeaderBytes + round_up(p2p_region_bytes(n_, p2p_slot_), 1u << 20) + 2 * (size_t(half_mb) << 20);
  va_.assign(n_, 0);
  peer_h_.assign(n_, 0);

  if (n_ == 1) {  // nothing to share: a plain allocation serves as the window
    void* p = nullptr;
    win_bytes_ = want;
    if (cudaMalloc(&p, win_bytes_) != cudaSuccess || cudaMemset(p, 0, kHeaderBytes) != cudaSuccess)
      return fail(hxcclUnhandledCudaError, "cannot allocate the window");
    va_[0] = reinterpret_cast<CUdeviceptr>(p);
    return hxcclSuccess;
  }

  // step 1: what each rank has
  RankFacts mine{host_fingerprint(), dev_, 0, 0, chunk_wish16()};
  bool ok = d.ok && n_ <= kMaxRanks && !std::getenv("HXCCL_TEST_FAIL_DEVICE_INIT");
  if (ok) {
    ok = d.CtxGetDevice(&cudev_) == CUDA_SUCCESS;
    int v = 0;
    if (ok && d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev_) == CUDA_SUCCESS) mine.multicast = v;
    if (ok && d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cudev_) == CUDA_SUCCESS)
      mine.fd_handles = v;
    ok = ok && mine.fd_handles;
  }
  std::vector<RankFacts> all(n_);
  if (c_->chan->allgather(&mine, all.data(), sizeof mine) != hxcclSuccess)
    return fail(hxcclSystemError, "exchanging device facts failed: " + c_->chan->error);
  bool all_mc = true;
  int chunk16 = 0;
  for (const RankFacts& f : all) {
    ok = ok && f.host == mine.host && f.fd_handles;
    all_mc = all_mc && f.multicast;
    if (f.chunk16 > 0) chunk16 = chunk16 ? std::min(chunk16, f.chunk16) : f.chunk16;
  }
  if (chunk16 > 0) {
    Tuning& t = eng_.tune;
    const size_t cap = size_t(chunk16) * 16;
    t.sub_max = std::min(t.sub_max, cap);
    t.single_sub_max = std::min(t.single_sub_max, cap);
    t.ring_sub = std::min(t.ring_sub, cap);
    t.roles_sub = std::min(t.roles_sub, cap);
  }
  for (int p = 0; p < n_; ++p)  // two ranks on one GPU cannot run kernels that wait on each other
    for (int q = p + 1; q < n_; ++q) ok = ok && all[p].device != all[q].device;
  if (!agree(ok))
    return fail(hxcclInvalidUsage, "peer windows need one GPU per rank, all on one machine, with "
                                   "file-descriptor memory handles");
  nvls_ = all_mc && env_long("HXCCL_NVLS", 1) != 0;

  // step 2: allocate and map my own window
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = cudev_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 2u << 20;
  ok = d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS;
  if (ok && nvls_) {
    CUmulticastObjectProp mp{};
    mp.numDevices = unsigned(n_);
    mp.size = want;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg)
      gran = std::max(gran, mg);
    else
      nvls_ = false;
  }
  // every rank must arrive at the same size: agree on the coarsest granularity
  uint64_t g64 = gran;
  if (c_->chan->max_u64(&g64) != hxcclSuccess) return fail(hxcclSystemError, "granularity agreement failed");
  win_bytes_ = round_up(want, size_t(g64));
  CUmemAccessDesc acc{};
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  std::string why;
  if (ok) {
    CUresult e = d.MemCreate(&own_h_, win_bytes_, &prop, 0);
    if (e == CUDA_SUCCESS) e = d.MemAddressReserve(&va_[rank_], win_bytes_, size_t(g64), 0, 0);
    if (e == CUDA_SUCCESS) e = d.MemMap(va_[rank_], win_bytes_, 0, own_h_, 0);
    if (e == CUDA_SUCCESS) e = d.MemSetAccess(va_[rank_], win_bytes_, &acc, 1);
    if (e != CUDA_SUCCESS) why = "allocating the window: " + d.err(e), ok = false;
    if (ok && (cudaMemset(reinterpret_cast<void*>(va_[rank_]), 0, kHeaderBytes) != cudaSuccess ||
               cudaDeviceSynchronize() != cudaSuccess))
      why = "clearing the window failed", ok = false;
  }
  vmm_ = true;
  peer_h_[rank_] = own_h_;
  if (!agree(ok)) return fail(hxcclUnhandledCudaError, why.empty() ? "a peer could not allocate its window" : why);

  // step 3: hand my window to every peer and map theirs
  FdPort port;
  int my_fd = -1;
  ok = port.open(c_->chan->id(), rank_, &why);
  if (ok) {
    const CUresult e = d.MemExportToShareableHandle(&my_fd, own_h_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (e != CUDA_SUCCESS) why = "exporting the window: " + d.err(e), ok = false;
  }
  if (!agree(ok)) {
    if (my_fd >= 0) ::close(my_fd);
    return fail(hxcclSystemError, why.empty() ? "a peer could not export its window" : why);
  }
  for (int p = 0; p < n_ && ok; ++p)
    if (p != rank_) ok = port.send_fd(c_->chan->id(), p, my_fd, 1, unsigned(rank_), &why);
  for (int got = 0; ok && got < n_ - 1; ++got) {
    int fd = -1;
    unsigned kind_tag = 0, from = 0;
    ok = port.recv_fd(&fd, &kind_tag, &from, 30000, &why);
    if (!ok) break;
    if (kind_tag != 1 || from >= unsigned(n_) || peer_h_[from]) {
      ::close(fd);
      why = "unexpected memory handle message";
      ok = false;
      break;
    }
    CUresult e = d.MemImportFromShareableHandle(&peer_h_[from], reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    if (e == CUDA_SUCCESS) e = d.MemAddressReserve(&va_[from], win_bytes_, size_t(g64), 0, 0);
    if (e == CUDA_SUCCESS) e = d.MemMap(va_[from], win_bytes_, 0, peer_h_[from], 0);
    if (e == CUDA_SUCCESS) e = d.MemSetAccess(va_[from], win_bytes_, &acc, 1);
    if (e != CUDA_SUCCESS) why = "mapping a peer window: " + d.err(e), ok = false;
  }
  if (my_fd >= 0) ::close(my_fd);
  if (!agree(ok)) return fail(hxcclSystemError, why.empty() ? "a peer could not map the windows" : why);
  return hxcclSuccess;
}

// NVSwitch multicast over the windows. Optional: any failure on any rank turns it off
// everywhere and the unicast kernels carry on.
void WindowPath::setup_multicast() {
  if (n_ < 2) nvls_ = false;
  if (!agree(nvls_)) {
    nvls_ = false;
    return;
  }
  const CuDriver& d = cu();
  std::string why;
  bool ok = true;
  FdPort port;
  // a separate port name keeps these messages apart from the window hand-over
  const uint64_t port_id = mix_id(c_->chan->id(), 0x6d63, 1);
  ok = port.open(port_id, rank_, &why);
  if (!agree(ok)) {
    nvls_ = false;
    return;
  }
  CUmulticastObjectProp mp{};
  mp.numDevices = unsigned(n_);
  mp.size = win_bytes_;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  int mc_fd = -1;
  if (rank_ == 0) {
    CUresult e = d.MulticastCreate(&mc_h_, &mp);
    if (e == CUDA_SUCCESS) e = d.MemExportToShareableHandle(&mc_fd, mc_h_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    ok = e == CUDA_SUCCESS;
    if (!ok) why = "creating the multicast object: " + d.err(e);
  }
  if (!agree(ok)) {  // nothing was handed out yet
    if (mc_fd >= 0) ::close(mc_fd);
    if (mc_h_) d.MemRelease(mc_h_), mc_h_ = 0;
    nvls_ = false;
    if (std::getenv("HXCCL_DEBUG") && rank_ == 0) std::fprintf(stderr, "hxccl: multicast off: %s\n", why.c_str());
    return;
  }
  if (rank_ == 0) {
    for (int p = 1; p < n_; ++p)
      if (!port.send_fd(port_id, p, mc_fd, 2u, 0, &why)) ok = false;
    ::close(mc_fd);
  } else {
    int fd = -1;
    unsigned tag = 0, from = 0;
    ok = port.recv_fd(&fd, &tag, &from, 30000, &why);
    if (ok) {
      const CUresult e = d.MemImportFromShareableHandle(&mc_h_, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (e != CUDA_SUCCESS) why = "importing the multicast object: " + d.err(e), ok = false;
    }
    if (fd >= 0) ::close(fd);
  }
  if (ok) {
    const CUresult e = d.MulticastAddDevice(mc_h_, cudev_);
    if (e != CUDA_SUCCESS) why = "joining the multicast object: " + d.err(e), ok = false;
  }
  if (!agree(ok)) {  // nobody has bound memory yet: dropping the handle is enough
    if (mc_h_) d.MemRelease(mc_h_), mc_h_ = 0;
    nvls_ = false;
    if (std::getenv("HXCCL_DEBUG")) std::fprintf(stderr, "hxccl[%d]: multicast off: %s\n", rank_, why.c_str());
    return;
  }
  CUresult e = d.MulticastBindMem(mc_h_, 0, own_h_, 0, win_bytes_, 0);
  mc_bound_ = e == CUDA_SUCCESS;
  if (e == CUDA_SUCCESS) e = d.MemAddressReserve(&mc_va_, win_bytes_, 0, 0, 0);
  if (e == CUDA_SUCCESS) e = d.MemMap(mc_va_, win_bytes_, 0, mc_h_, 0);
  if (e == CUDA_SUCCESS) {
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = cudev_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    e = d.MemSetAccess(mc_va_, win_bytes_, &acc, 1);
  }
  ok = e == CUDA_SUCCESS;
  if (!ok) why = "binding the multicast object: " + d.err(e);
  if (!agree(ok)) {
    nvls_ = false;  // release() unbinds and unmaps whatever got done
    if (std::getenv("HXCCL_DEBUG")) std::fprintf(stderr, "hxccl[%d]: multicast off: %s\n", rank_, why.c_str());
  }
}

void WindowPath::release() {
  const CuDriver& d = cu();
  cudaSetDevice(dev_);
  if (scratch_) cudaFree(scratch_), scratch_ = nullptr;
  if (trace_) cudaFree(trace_), trace_ = nullptr;
  if (mc_va_) {
    d.MemUnmap(mc_va_, win_bytes_);
    d.MemAddressFree(mc_va_, win_bytes_);
    mc_va_ = 0;
  }
  if (mc_h_) {
    if (mc_bound_) d.MulticastUnbind(mc_h_, cudev_, 0, win_bytes_);
    d.MemRelease(mc_h_);
    mc_h_ = 0;
  }
  if (vmm_) {
    for (int p = 0; p < n_; ++p) {
      if (va_.size() > size_t(p) && va_[p]) {
        d.MemUnmap(va_[p], win_bytes_);
        d.MemAddressFree(va_[p], win_bytes_);
      }
      if (peer_h_.size() > size_t(p) && peer_h_[p]) d.MemRelease(peer_h_[p]);
    }
  } else if (!va_.empty() && va_[0]) {
    cudaFree(reinterpret_cast<void*>(va_[0]));
  }
  va_.clear();
  peer_h_.clear();
  if (order_event_) cudaEventDestroy(order_event_), order_event_ = nullptr;
  if (status_) cudaFreeHost(status_), status_ = nullptr;
}

// ---- launches ----------------------------------------------------------------------------------

hxcclResult_t WindowPath::broken(std::string* why) {
  if (broken_ == hxcclSuccess && status_) {
    const unsigned long long s = *reinterpret_cast<volatile unsigned long long*>(status_);
    if (s) {
      const unsigned code = unsigned(s >> 56), peer = unsigned(s & 0xffffff);
      if (code == kStatTimeout) {
        broken_ = hxcclTimeout;
        broken_why_ = "a device-side wait for rank " + std::to_string(peer) +
                      " ran out of time (HXCCL_WAIT_LIMIT_MS); the device path is unusable";
      } else {
        broken_ = hxcclRemoteError;
        broken_why_ = "rank " + std::to_string(peer) + " (or a rank it waited for) failed during a device transfer";
      }
    }
  }
  if (broken_ == hxcclSuccess && status_) {  // a truncated receive: reported once, not sticky
    volatile unsigned long long* soft = status_ + 1;
    if (*soft) {
      *soft = 0;
      if (why) *why = kTruncatedMsg;
      comm_fail(c_, hxcclSystemError, kTruncatedMsg);
    }
  }
  if (broken_ != hxcclSuccess && why) *why = broken_why_;
  return broken_;
}

// Launches belong on the communicator's device whatever device the caller has current; done()
// puts the caller's device back.
cudaStream_t WindowPath::enter(void* stream) {
  int cur = dev_;
  caller_dev_ = -1;
  if (cudaGetDevice(&cur) == cudaSuccess && cur != dev_) {
    caller_dev_ = cur;
    cudaSetDevice(dev_);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (used_ && st != last_stream_) {  // keep the communicator's launches in one order
    cudaEventRecord(order_event_, last_stream_);
    cudaStreamWaitEvent(st, order_event_, 0);
  }
  last_stream_ = st;
  used_ = true;
  return st;
}

hxcclResult_t WindowPath::done(cudaError_t e, const char* what) {
  if (caller_dev_ >= 0) {
    cudaSetDevice(caller_dev_);
    caller_dev_ = -1;
  }
  if (e == cudaSuccess) return hxcclSuccess;
  if (!eng_.error.empty()) {
    error = eng_.error;
    eng_.error.clear();
    return std::strstr(error.c_str(), "truncated") ? hxcclSystemError : hxcclInvalidUsage;
  }
  error = std::string(what) + ": " + cudaGetErrorString(e);
  return hxcclUnhandledCudaError;
}

hxcclResult_t WindowPath::allreduce(const void* send, void* recv, size_t count, int dt,
                                    const OpPlan& plan, int order, void* stream) {
  if (count == 0) return hxcclSuccess;
  RankBufs b{send, recv};
  const cudaError_t e = eng_.allreduce(&b, count, dt, plan, order, enter(stream));
  // HXCCL_DEBUG=2 (or more): one line per AllReduce on rank 0 with what the tuner chose
  static const int level = [] { const char* v = std::getenv("HXCCL_DEBUG"); return v ? std::atoi(v) : 0; }();
  if (level >= 2 && rank_ == 0) {
    static const char* const names[] = {"auto", "one-shot", "two-shot", "nvls", "two-shot roles", "nvls roles", "ring", "lines"};
    const int v = eng_.last_variant;
    std::fprintf(stderr, "hxccl: AllReduce %zu bytes, dtype %d, order %s -> %s\n", count * dtype_size(dt), dt,
                 order == kOrderRing ? "ring" : "doubling", v >= 0 && v <= 7 ? names[v] : "?");
  }
  return done(e, "AllReduce launch");
}

hxcclResult_t WindowPath::allreduce_cast(const void* send, void* recv, size_t count, int wire_dt,
                                         const OpPlan& plan, void* stream) {
  if (count == 0) return hxcclSuccess;
  if (n_ < 2 || count * dtype_size(wire_dt) < kDoublingMaxBytes) {
    error = "the fused cast AllReduce serves two or more ranks and messages in ring order only";
    return hxcclInvalidUsage;
  }
  RankBufs b{send, recv};
  return done(eng_.allreduce_cast(&b, count, wire_dt, plan, enter(stream)), "AllReduceCast launch");
}
hxcclResult_t WindowPath::allgather(const void* send, void* recv, size_t block, void* stream) {
  if (block == 0) return hxcclSuccess;
  RankBufs b{send, recv};
  return done(eng_.allgather(&b, block, enter(stream)), "AllGather launch");
}
hxcclResult_t WindowPath::reducescatter(const void* send, void* recv, size_t per, int dt,
                                        const OpPlan& plan, void* stream) {
  if (per == 0) return hxcclSuccess;
  RankBufs b{send, recv};
  return done(eng_.reducescatter(&b, per, dt, plan, enter(stream)), "ReduceScatter launch");
}
hxcclResult_t WindowPath::broadcast(const void* send, void* recv, size_t bytes, int root, void* stream) {
  if (bytes == 0) return hxcclSuccess;
  RankBufs b{send, recv};
  return done(eng_.broadcast(&b, bytes, root, enter(stream)), "Broadcast launch");
}
hxcclResult_t WindowPath::reduce(const void* send, void* recv, size_t count, int dt,
                                 const OpPlan& plan, int root, void* stream) {
  if (count == 0) return hxcclSuccess;
  RankBufs b{send, recv};
  return done(eng_.reduce(&b, count, dt, plan, root, enter(stream)), "Reduce launch");
}
hxcclResult_t WindowPath::gather(const void* send, void* recv, size_t block, int root, void* stream) {
  if (block == 0) return hxcclSuccess;
  RankBufs b{send, recv};
  return done(eng_.gather(&b, block, root, enter(stream)), "Gather launch");
}
hxcclResult_t WindowPath::scatter(const void* send, void* recv, size_t block, int root, void* stream) {
  if (block == 0) return hxcclSuccess;
  RankBufs b{send, recv};
  return done(eng_.scatter(&b, block, root, enter(stream)), "Scatter launch");
}

hxcclResult_t WindowPath::alltoallv(const char* send, const size_t* sbytes, const size_t* soff,
                                    char* recv, const size_t* rbytes, const size_t* roff,
                                    size_t max_pair, void* stream) {
  cudaStream_t st = enter(stream);
  if (max_pair == 0) return hxcclSuccess;
  // Identical send and receive layouts in one buffer are safe (each CTA reads a range before
  // it overwrites it); any other overlap goes through a private copy of the send side.
  size_t send_end = 0, recv_end = 0;
  bool same_layout = send == recv;
  for (int j = 0; j < n_; ++j) {
    if (sbytes[j]) send_end = std::max(send_end, soff[j] + sbytes[j]);
    if (rbytes[j]) recv_end = std::max(recv_end, roff[j] + rbytes[j]);
    same_layout = same_layout && soff[j] == roff[j] && sbytes[j] == rbytes[j];
  }
  const bool overlap = send_end && recv_end && send < recv + recv_end && recv < send + send_end;
  if (overlap && !same_layout) {
    if (send_end > scratch_bytes_) {
      cudaStreamSynchronize(st);
      if (scratch_) cudaFree(scratch_);
      scratch_ = nullptr;
      if (cudaMalloc(&scratch_, send_end) != cudaSuccess) return done(cudaErrorMemoryAllocation, "AlltoAll staging");
      scratch_bytes_ = send_end;
    }
    if (cudaError_t e = cudaMemcpyAsync(scratch_, send, send_end, cudaMemcpyDeviceToDevice, st))
      return done(e, "AlltoAll staging");
    send = static_cast<const char*>(scratch_);
  }
  RankV v{send, sbytes, soff, recv, rbytes, roff};
  return done(eng_.alltoallv(&v, max_pair, st), "AlltoAll launch");
}

hxcclResult_t WindowPath::p2p_batch(const std::vector<P2pOp>& ops, void* stream) {
  RankP2p r{ops};
  return done(eng_.p2p(&r, enter(stream)), "Send/Recv launch");
}

int WindowPath::read_trace(unsigned long long* out, int max_ctas) {
  if (!trace_) return 0;
  drain();
  const int rows = std::min(max_ctas, kMaxCtas);
  const size_t bytes = size_t(rows) * kTraceSlots * sizeof(unsigned long long);
  if (cudaMemcpy(out, trace_, bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
  cudaMemset(trace_, 0, size_t(kMaxCtas) * kTraceSlots * sizeof(unsigned long long));
  return rows;
}

hxcclResult_t WindowPath::drain() {
  cudaSetDevice(dev_);
  if (used_) cudaStreamSynchronize(last_stream_);
  return hxcclSuccess;
}

}  // namespace hx
