// Turns one rank's collective call into kernel arguments and a launch shape. Pure host code:
// every rank computes the same geometry from the same (agreed) sizes, which the kernels rely
// on (same CTA count and step count everywhere). Used by the production path and by the
// single-GPU world used in tests, so both run exactly the same plans.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

#include "core/devpath.h"
#include "core/schedule.h"
#include "device/proto.h"

namespace hx {

struct Geometry {
  int ctas = 1;
  int threads = 256;
  int steps = 1;
  int epochs = 1;  // epochs the launch consumes: 1, or steps + 2 when pipelined
  size_t sub_bytes = 16;
};

// AllReduce transport variants
enum : int { kVarAuto = 0, kVarOneShot = 1, kVarTwoShot = 2, kVarNvls = 3, kVarTwoShotRoles = 4, kVarNvlsRoles = 5,
       kVarRing = 6, kVarLL = 7 };

struct Tuning {
  int max_ctas = 128;         // upper bound of any collective grid
  size_t oneshot_max = 256 * 1024;  // AllReduce: up to here every rank pushes everything
  bool exact = true;          // floats must match the host path bit for bit
  bool nvls = false;          // multicast alias available
  bool nvls_gather = true;    // two-shot publishes results through the multicast alias
  size_t nvls_min = 512 * 1024;    // AllReduce: from here NVLS, when allowed for (dtype, op)
  size_t single_sub_max = 256 * 1024;  // per-CTA share up to which a launch runs as one step
  size_t sub_max = 256 * 1024;        // largest per-CTA share of one pipelined step
  int min_steps = 4;                  // a pipelined launch aims at this many steps at least
  int threads = 0;                    // CTA width of the large launches, 0 = choose
  int sm_count = 148;                 // SMs of the device (set by the device path)
  int roles_min_ranks = 8;            // exact two-shot: role pipeline only from this many ranks
  size_t roles_min = 96u << 20;       // AllReduce: from here the three-role pipeline
  size_t roles_sub = 64 * 1024;       // its per-lane share of a slice per step
  size_t ring_min = 128u << 20;       // AllReduce: from here the neighbour ring (0 = only when forced)
  int ring_max_ranks = kMaxRanks;     // ... on communicators of at most this many ranks
  size_t ring_sub = 512 * 1024;       // largest per-CTA share of one ring hop
  int p2p_threads = 512;              // CTA width of the Send/Recv lanes
  size_t ll_max = 16 * 1024;          // AllReduce: up to here the flag-in-data kernel (0 = never)
  bool ll_mc = true;                  // ... its lines go out through the multicast alias when there is one
  size_t rs_ring_min = 256u << 20;    // ReduceScatter: neighbour ring from this many input bytes (0 = never)
  bool mc_copy = true;                // AllGather / Broadcast push through the multicast alias
  size_t mc_copy_min = 0;             // ... from this many bytes per block
};

// Sets one tuning knob by name ("max_ctas", "oneshot_max", "nvls_min", "single_sub_max",
// "sub_max", "min_steps", "threads", "roles_min", "roles_sub", "ring_min", "ring_max_ranks", "ring_sub", "p2p_threads",
// "exact", "nvls_gather", "mc_copy", "mc_copy_min", "rs_ring_min", "ll_max", "ll_mc");
// false for an unknown name.
bool set_knob(Tuning* t, const char* name, long value);
// Applies a file of knob settings (HXCCL_TUNE_FILE): one "name value" or "name=value" per line,
// '#' starts a comment. False, with the reason in *why, for an unreadable file or a bad line.
bool load_tune_file(Tuning* t, const char* path, std::string* why);

// generic exchange where the largest block of any pair is `max_pair` bytes
Geometry plan_xchg(size_t max_pair, int n, size_t half_bytes, const Tuning& t, size_t cta_bytes = 16 * 1024);
// two-shot / NVLS AllReduce of `bytes`
Geometry plan_sliced(size_t bytes, int n, size_t half_bytes, const Tuning& t);
// the same as a three-role pipeline: ctas = 3 * lanes, epochs = steps + 1
Geometry plan_roles(size_t bytes, int n, size_t half_bytes, const Tuning& t);

// neighbour ring over blocks of at most `max_block` bytes: steps = rounds,
// epochs = rounds * (2n - 2) + 2; the ReduceScatter form (`rs`) raises n - 1 flags per round:
// epochs = rounds * (n - 1) + 2 (it uses the same 2n - 2 slots, as two alternating sets)
Geometry plan_ring(size_t max_block, int n, size_t half_bytes, const Tuning& t, bool rs = false);

// Checks a launch shape against the window layout the kernels assume: every slot a CTA writes
// lies inside its staging buffer, the steps cover the whole message, the grid fits the flag rows.
// Returns an empty string when all holds, else what does not. `amount` is what the matching
// plan_* function was given. Run before every launch (host arithmetic only).
enum : int { kPlanXchg = 0, kPlanSliced = 1, kPlanRoles = 2, kPlanRing = 3, kPlanRingRs = 4 };
std::string check_geometry(int kind, const Geometry& g, size_t amount, int n, size_t half_bytes);

FoldSpec make_fold(const OpPlan& plan, int kind);

// which variant an AllReduce takes
int choose_variant(size_t bytes, int dt, const OpPlan& plan, int n, const Tuning& t, int forced);

void build_allreduce_oneshot(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                             const void* send, void* recv, size_t count, int dt,
                             const OpPlan& plan, int order);
void build_allreduce_ll(LLArgs* a, const WinView& w, uint64_t epoch, const void* send, void* recv,
                        size_t count, int dt, const OpPlan& plan, int order, bool use_mc);
void build_allreduce_twoshot(TwoShotArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                             const void* send, void* recv, size_t count, int dt,
                             const OpPlan& plan, int order, bool use_mc);
void build_allreduce_nvls(NvlsArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                          const void* send, void* recv, size_t count, int dt, const OpPlan& plan);
void build_reducescatter_ring(TwoShotArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                              const void* send, void* recv, size_t per, int dt, const OpPlan& plan);
void build_reducescatter(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                         const void* send, void* recv, size_t per, int dt, const OpPlan& plan);
void build_reduce(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                  const void* send, void* recv, size_t count, int dt, const OpPlan& plan,
                  int root);
// `multicast`: push through the multicast alias where this rank's buffer allows it
void build_allgather(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                     const void* send, void* recv, size_t block, bool multicast);
void build_broadcast(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                     const void* send, void* recv, size_t bytes, int root, bool multicast);
void build_gather(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                  const void* send, void* recv, size_t block, int root);
void build_scatter(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                   const void* send, void* recv, size_t block, int root);
void build_alltoallv(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                     const char* send, const size_t* sbytes, const size_t* soff, char* recv,
                     const size_t* rbytes, const size_t* roff);

}  // namespace hx
