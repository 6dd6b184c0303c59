// Turns one rank's collective call into kernel arguments and a launch shape. Pure host code:
// every rank computes the same geometry from the same (agreed) sizes, which the kernels rely
// on (same CTA count and step count everywhere). Used by the production path and by the
// single-GPU world used in tests, so both run exactly the same plans.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

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

// One row of the measured tuning table: for collective `coll` on `n` ranks with elements of
// `es` bytes (0 = any) in exact / fast mode (-1 = either), messages of at least `from` bytes
// take `variant`, launched with the given grid limit, CTA width and per-step share (0 = the
// planner's own choice). The row with the largest `from` not above the message wins. Rows come
// from bench/sweep.py --emit-tune (the compiled-in default, src/device/tune_default.inc, was
// produced that way on 8 x B200) or from HXCCL_TUNE_FILE. `bytes` is the message size for
// AllReduce and Broadcast and the per-rank block for AllGather and ReduceScatter.
enum : int { kCollAllReduce = 0, kCollAllGather = 1, kCollReduceScatter = 2, kCollBroadcast = 3 };
struct TuneRow {
  int coll = 0, n = 0, es = 0, exact = -1;
  size_t from = 0;
  int variant = 0;  // AllReduce: kVar*; AllGather / Broadcast: 1 = multicast push; ReduceScatter: 1 = ring
  int ctas = 0, threads = 0;
  size_t sub = 0;
  size_t grain = 0;  // see Tuning::grain
};

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
  bool p2p_bulk = true;               // Send pieces move by bulk asynchronous copies (one driving thread per CTA)
  size_t ll_max = 16 * 1024;          // AllReduce: up to here the flag-in-data kernel (0 = never)
  bool ll_mc = true;                  // ... its lines go out through the multicast alias when there is one
  size_t rs_ring_min = 256u << 20;    // ReduceScatter: neighbour ring from this many input bytes (0 = never)
  // the measured table (shared, so that copying a Tuning per call stays cheap); null or empty =
  // the thresholds above only
  std::shared_ptr<std::vector<TuneRow>> rows;
  bool use_table = true;              // "table 0" (or HXCCL_TUNE_TABLE=0) ignores the rows
  size_t grain = 16 * 1024;           // bytes of a pair's block (a slice) one CTA takes before the grid grows
  int mc_force = -1;                  // AllGather / Broadcast multicast push: 1 always, 0 never, -1 table / default
  bool mc_copy = true;                // AllGather / Broadcast push through the multicast alias
  size_t mc_copy_min = 0;             // ... from this many bytes per block
};

// The row that applies, or null. n matches exactly or falls back to the largest tabled rank
// count below it; an exact element size beats es = 0.
const TuneRow* find_row(const Tuning& t, int coll, int n, int es, bool exact, size_t bytes);
// Appends the rows of the compiled-in default table.
void load_default_table(Tuning* t);
// Parses one "row ..." line (see load_tune_file); false with *why set when malformed.
bool parse_row(const std::string& line, TuneRow* row, std::string* why);

// Sets one tuning knob by name ("max_ctas", "oneshot_max", "nvls_min", "single_sub_max",
// "sub_max", "min_steps", "threads", "roles_min", "roles_sub", "ring_min", "ring_max_ranks", "ring_sub", "p2p_threads",
// "exact", "nvls_gather", "table", "grain", "p2p_bulk", "mc_force", "mc_copy", "mc_copy_min", "rs_ring_min", "ll_max", "ll_mc");
// false for an unknown name.
bool set_knob(Tuning* t, const char* name, long value);
// Applies a tuning file (HXCCL_TUNE_FILE): knob lines "name value" or "name=value", and table
// rows "row <allreduce|allgather|reducescatter|broadcast> n=<ranks> [es=<bytes>] [mode=exact|fast]
// from=<bytes> variant=<name|number> [ctas=<c>] [threads=<256|512>] [sub=<bytes>] [grain=<bytes>]"; the first
// row line of a file replaces the compiled-in table. '#' starts a comment. False, with the
// reason in *why, for an unreadable file or a bad line.
bool load_tune_file(Tuning* t, const char* path, std::string* why);

// generic exchange where the largest block of any pair is `max_pair` bytes
// cta_bytes: bytes of a pair's block per CTA before the grid grows (0 = t.grain)
Geometry plan_xchg(size_t max_pair, int n, size_t half_bytes, const Tuning& t, size_t cta_bytes = 0);
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

// which variant an AllReduce takes; *row (when given) receives the table row behind the choice
int choose_variant(size_t bytes, int dt, const OpPlan& plan, int n, const Tuning& t, int forced,
                   const TuneRow** row = nullptr);
// `t` with a row's grid limit, CTA width and per-step share applied
Tuning with_row(const Tuning& t, const TuneRow* row, int variant);

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
