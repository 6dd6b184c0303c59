// Layout of a rank's communication window and the argument blocks of the kernels. Shared by
// the host launchers and the device code.
//
// Every rank of a communicator owns one window in its GPU's memory, mapped into every peer's
// address space (and, where the node has NVSwitch multicast, bound to one multicast object).
// Kernels move data with plain stores into a peer's window followed by a flag; nothing on the
// data path goes through the host. This replaces the reference's per-pair cudaIpc staging
// buffers with host READY/DONE handshakes (src/transport_ipc.cc:13-32, :358-432).
//
//   [control]  abort word, Send/Recv counters and flags
//   [flags A]  one 64-bit epoch per (CTA, source rank): "my step-e data is in your window"
//   [flags B]  same, for the second phase of two-phase kernels
//   [flags C]  same, for the third role of the three-role pipeline (kernels/roles_body.cuh)
//   [lines]    data-with-epoch lines of the small-message AllReduce (kernels/ll_body.cuh)
//   [p2p]      Send/Recv slots, a ring of kP2pDepth per (sender, worker)
//   [half 0] [half 1]  collective staging, alternating per step
//
// Steps. A collective launch runs K >= 1 steps; the communicator numbers the steps (and the
// opening / closing hand-shakes of multi-step launches) of all its launches with one increasing
// epoch, the same on every rank. A single-step launch stages in half e & 1: in every step each
// rank signals each rank, so a writer that reached epoch e+2 has seen the e+1 signal of the
// window's owner, which that owner sent only after it finished reading epoch e, and the half is
// free again without any extra hand-shake. A multi-step launch owns both halves as a ring of
// four buffers between its two hand-shakes (kernels/coll_body.cuh). Flags only ever grow.
//
// All waits are bounded: a wait that runs out of time records a status in pinned host memory,
// raises the abort word in every peer's window (so they stop too) and the kernel returns.
#pragma once
#include <cstddef>
#include <cstdint>

namespace hx {

constexpr int kMaxRanks = 16;       // ranks of one device communicator
constexpr int kFastRanks = 8;       // the unrolled fold covers this many
constexpr int kMaxCtas = 512;       // flag rows
constexpr int kP2pWorkers = 16;     // independent sub-channels per directed pair
// Two slots of 512 KiB measured faster than four of 256 KiB (256 MiB ring shift on two GPUs:
// 425 against 349 GB/s): the per-piece hand-shake, not the depth, is what limits a lane.
constexpr int kP2pDepth = 2;        // slots a (sender, worker) cycles through
constexpr size_t kP2pSlotBytes = 512 * 1024;  // per (sender, worker, slot): the default, see WinView::p2p_slot

// byte offsets inside a window
constexpr size_t kOffAbort = 0;
constexpr size_t kOffP2pTx = 4096;    // u64 [kMaxRanks][kP2pWorkers]  chunk-slots sent (local)
constexpr size_t kOffP2pRx = 8192;    // u64 [kMaxRanks][kP2pWorkers]  chunk-slots taken (local)
constexpr size_t kOffP2pReady = 12288;  // u64 [sender][worker], written by the sender
constexpr size_t kOffP2pDone = 16384;   // u64 [receiver][worker], written by the receiver
constexpr size_t kOffP2pHdr = 20480;    // u64 [sender][worker][kP2pDepth]: message bytes per slot
static_assert(size_t(kMaxRanks) * kP2pWorkers * 8 <= 4096 && kOffP2pHdr + size_t(kMaxRanks) * kP2pWorkers * 8 * kP2pDepth <= 64 * 1024,
              "Send/Recv words must fit their slots in the header");
constexpr size_t kOffFlagsA = 64 * 1024;
constexpr size_t kOffFlagsB = kOffFlagsA + size_t(kMaxCtas) * kMaxRanks * 8;
constexpr size_t kOffFlagsC = kOffFlagsB + size_t(kMaxCtas) * kMaxRanks * 8;
// Lines of the small-message AllReduce (kernels/ll_body.cuh): two halves by epoch parity, each
// with one slot per source rank. A line is 16 bytes and carries 8 bytes of payload. The region
// is part of the header, which is what gets cleared when a window is created.
constexpr size_t kOffLL = 1u << 20;
constexpr size_t kLLBytes = 8u << 20;
constexpr size_t kHeaderBytes = kOffLL + kLLBytes;
static_assert(kOffFlagsC + size_t(kMaxCtas) * kMaxRanks * 8 <= kOffLL, "flag pages must end before the line region");
inline constexpr size_t ll_slot_bytes(int n) { return kLLBytes / 2 / size_t(n) / 256 * 256; }
inline constexpr size_t ll_max_payload(int n) { return ll_slot_bytes(n) / 2; }
constexpr size_t kOffP2pSlots = kHeaderBytes;

inline constexpr size_t p2p_region_bytes(int n, size_t slot_bytes = kP2pSlotBytes) {
  return size_t(n) * kP2pWorkers * kP2pDepth * slot_bytes;
}

// status word (pinned host memory, one per communicator): 0 fine, else
// (code << 56) | detail. Codes below.
enum : unsigned { kStatTimeout = 1, kStatRemote = 2, kStatTruncated = 3 };

struct WinView {
  char* win[kMaxRanks];   // every rank's window in this rank's address space (win[rank] local)
  char* mc;               // multicast alias of the windows, or null
  unsigned long long* status;  // pinned host status word (sticky failures)
  unsigned long long* soft;    // pinned host word for truncation reports (not sticky)
  size_t half_off[2];     // offsets of the two staging halves
  size_t half_bytes;
  // Bytes of one Send/Recv slot; the same on every rank of the communicator. Communicators made
  // by Split / Shrink use smaller slots (and staging halves) than the one they came from, so
  // that a program with many sub-communicators does not pay the full window for each.
  size_t p2p_slot;
  unsigned long long wait_ns;  // limit of every device-side wait
  // Optional phase timing (HXCCL_TRACE=1): kTraceSlots accumulators of nanoseconds per CTA,
  // filled by thread 0 of each CTA from %globaltimer; null when off.
  unsigned long long* trace;
  int rank, n;
};
constexpr int kTraceSlots = 16;
// what the slots hold (single-role kernels): time spent staging in, raising the first flag,
// waiting for it, combining, raising / waiting for the second flag, staging out; slot 7 = whole kernel
enum : int { kTrIn = 0, kTrSigA = 1, kTrWaitA = 2, kTrMid = 3, kTrSigB = 4, kTrWaitB = 5, kTrOut = 6, kTrAll = 7 };

// How a fold combines the ranks' values for one element (see core/schedule.h):
//   Linear   acc = x[s0]; then x[s0+dir], x[s0+2dir], ... each as the LEFT operand. With
//            ring = 1 the start is the index of the ring block the element belongs to plus
//            `start` (AllReduce ring order start 0; element blocks given by `count`), else
//            `start` itself (ReduceScatter block b: start b+1; Reduce chain: start root+n-1,
//            dir -1).
//   Doubling recursive doubling as rank `rank` sees it.
//   Tree     binomial tree toward `root` (only the root's value is meaningful).
enum : int { kFoldLinear = 0, kFoldDoubling = 1, kFoldTree = 2 };
struct FoldSpec {
  int kind;
  int op;          // kSum..kMin
  int start, dir;  // Linear
  int ring;        // Linear: add the element's ring-block index to start
  int root;        // Tree
  int premul;      // scale own input by the scalar before anything else
  int postdiv;     // integer Avg divisor, 0 = none
  unsigned long long scalar_bits;  // scalar when known at launch
  const void* scalar_ptr;          // else read from here (device memory)
  size_t ring_count;               // Linear+ring: element count that defines the blocks
};

// ---- generic exchange: every rank pushes a block to some peers, then copies or folds what
// ---- landed in its own window. One step moves up to `step_bytes` of every pair's block.
struct XchgArgs {
  WinView w;
  unsigned long long epoch0;
  int steps;
  size_t sub_bytes;      // bytes of a pair's block one CTA moves per step (multiple of 16)
  size_t slot_stride;    // distance between two source ranks' slots in a half
  // push: bytes [0, send_bytes[j]) at send_ptr[j] go to rank j (0 = nothing)
  const char* send_ptr[kMaxRanks];
  size_t send_bytes[kMaxRanks];
  // copy mode: bytes from rank i land at recv_ptr[i]
  char* recv_ptr[kMaxRanks];
  size_t recv_bytes[kMaxRanks];
  // fold mode (fold_bytes > 0): all n sources (own input at own_ptr, not staged) combine into dst
  char* fold_dst;
  const char* own_ptr;
  size_t fold_bytes;
  size_t fold_elem0;     // index of dst[0] in the full vector (ring-block lookup)
  FoldSpec fold;
  int push_scaled;       // pushes carry input * scalar (fold.premul) instead of raw bytes
  // Multicast push (AllGather, Broadcast on a window bound to an NVSwitch multicast object):
  // bytes [0, mc_bytes) at mc_src go to EVERY rank's slot of this rank with one multimem.st per
  // 16 bytes instead of one store per peer, so the sender's link carries the block once.
  // 0 = push peer by peer (send_ptr / send_bytes above, which are filled either way).
  const char* mc_src;
  size_t mc_bytes;
};

// ---- two-shot AllReduce: reduce-scatter into owners, owners fold, all-gather the results
struct TwoShotArgs {
  WinView w;
  unsigned long long epoch0;
  int steps;
  size_t sub_bytes;    // per CTA, per slice, per step (multiple of 16)
  const char* send;
  char* recv;
  size_t bytes;        // whole message
  FoldSpec fold;
  int use_mc;          // all-gather phase through the multicast alias
  // neighbour ring only: 1 = ReduceScatter (the reduce-scatter half alone, every block's chain
  // shifted by one rank so that block r ends on rank r; `send` holds n blocks, `recv` one)
  int ring_rs;
};

// ---- small-message AllReduce with the flag inside the data (kernels/ll_body.cuh)
struct LLArgs {
  WinView w;
  unsigned long long epoch;
  const char* send;
  char* recv;
  size_t bytes;   // at most ll_max_payload(n)
  FoldSpec fold;
  int use_mc;     // lines go out through the multicast alias
};

// ---- NVLS AllReduce: copy in, multimem.ld_reduce own slice, multimem.st, copy out
struct NvlsArgs {
  WinView w;
  unsigned long long epoch0;
  int steps;
  size_t sub_bytes;
  const char* send;
  char* recv;
  size_t bytes;
  int op;        // kSum / kMax / kMin
  int dt;        // hxcclDataType_t
  int premul;    // scale while copying in
  int postdiv;
  unsigned long long scalar_bits;
  const void* scalar_ptr;
};

// ---- Send/Recv lanes
struct P2pLaneOp {
  char* buf;
  size_t bytes;
};
constexpr int kMaxLaneOps = 8;   // operations of one (peer, direction) in one launch
constexpr int kMaxLanes = 2 * kMaxRanks;
struct P2pLane {
  int peer;
  int is_send;
  int nops;
  P2pLaneOp ops[kMaxLaneOps];
};
struct P2pArgs {
  WinView w;
  int nlanes;
  int workers_per_cta;       // a power of two up to kP2pWorkers: workers one CTA serves in turn
  int bulk;                  // senders move their pieces with bulk asynchronous copies (needs the dynamic shared memory)
  P2pLane lanes[kMaxLanes];  // CTA (lane, group) = blockIdx.x / G, % G with G = kP2pWorkers / workers_per_cta
};

}  // namespace hx
