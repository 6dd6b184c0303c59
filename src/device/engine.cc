#include "device/engine.h"

#include <algorithm>
#include <cstring>

#include "math/dtypes.h"

namespace hx {

Engine::~Engine() {
  if (dev_args_) cudaFree(dev_args_);
}

// Host-side check of every launch shape against the window layout (planner.h); a violation is
// a bug in the planner, reported instead of launched.
#define HX_CHECK_PLAN(KIND, G, AMOUNT)                                                   \
  do {                                                                                   \
    const std::string why_ = check_geometry(KIND, G, AMOUNT, n(), views[0].half_bytes);  \
    if (!why_.empty()) {                                                                 \
      error = "launch plan rejected: " + why_;                                           \
      return cudaErrorInvalidValue;                                                      \
    }                                                                                    \
  } while (0)

LaunchShape Engine::shape(const Geometry& g) const {
  return LaunchShape{g.ctas, g.threads, world() ? int(views.size()) : 0};
}

// Production: the single argument block is passed by value. World: the blocks of all ranks go
// to device memory first (stream-ordered copy from the caller's vector, which outlives it
// because the copy of pageable memory returns only after the source was read).
template <typename Args>
const Args* Engine::stage(const std::vector<Args>& args, cudaStream_t st, cudaError_t* rc) {
  *rc = cudaSuccess;
  if (!world()) return args.data();
  const size_t bytes = args.size() * sizeof(Args);
  if (bytes > dev_args_bytes_) {
    if (dev_args_) cudaFree(dev_args_);
    dev_args_ = nullptr;
    if ((*rc = cudaMalloc(&dev_args_, bytes)) != cudaSuccess) return nullptr;
    dev_args_bytes_ = bytes;
  }
  // earlier launches may still read the buffer
  if ((*rc = cudaStreamSynchronize(st)) != cudaSuccess) return nullptr;
  *rc = cudaMemcpyAsync(dev_args_, args.data(), bytes, cudaMemcpyHostToDevice, st);
  return static_cast<const Args*>(dev_args_);
}

cudaError_t Engine::allreduce(const RankBufs* b, size_t count, int dt, const OpPlan& plan,
                              int order, cudaStream_t st) {
  const size_t bytes = count * dtype_size(dt);
  // One rank, nothing to scale or divide: the result is the input (the reference's path does a
  // plain copy then too, src/algo_ring.cc:17-18). In place that is no work at all.
  if (!world() && n() == 1 && !plan.premul && !(plan.postdiv && plan.divisor != 1)) {
    last_variant = kVarAuto;
    if (b[0].send == b[0].recv) return cudaSuccess;
    ++launches;
    return launch_copy(b[0].recv, b[0].send, bytes, st);
  }
  const TuneRow* row = nullptr;
  int var = choose_variant(bytes, dt, plan, n(), tune, forced_variant, &row);
  const Tuning tune = with_row(this->tune, row, var);  // the row's launch shape, for this call only
  // recursive doubling gives every rank its own operand order; only the variant in which each
  // rank folds for itself can replay that
  if (order == kOrderDoubling && tune.exact && !is_integer(dt) && var != kVarLL) var = kVarOneShot;
  if (world() && var == kVarNvls) var = kVarTwoShot;
  if (var == kVarLL) {
    // A line carries the low 32 bits of the epoch. Zero is what a cleared region holds, and
    // when the upper half of the epoch moves on, lines of 2^32 steps ago could match again:
    // then every rank clears its own region (in stream order) and this call takes the ordinary
    // one-shot kernel, whose all-to-all hand-shake separates the clearing from later lines.
    if ((epoch >> 32) != ll_era_) {
      ll_era_ = epoch >> 32;
      for (const WinView& v : views)
        if (cudaError_t e = cudaMemsetAsync(v.win[v.rank] + kOffLL, 0, kLLBytes, st)) return e;
      var = kVarOneShot;
    } else if (uint32_t(epoch) == 0) {
      var = kVarOneShot;
    }
  }
  last_variant = var;
  cudaError_t rc;
  ++launches;
  if (var == kVarLL) {
    const size_t lines = (bytes + 7) / 8;
    Geometry g;
    g.threads = 256;
    g.ctas = int(std::max<size_t>(1, std::min<size_t>(std::min(128, tune.max_ctas), (lines + 255) / 256)));
    std::vector<LLArgs> args(views.size());
    for (size_t r = 0; r < views.size(); ++r)
      build_allreduce_ll(&args[r], views[r], epoch, b[r].send, b[r].recv, count, dt, plan, order,
                         tune.nvls && tune.ll_mc && !world());
    epoch += 1;
    const LLArgs* a = stage(args, st, &rc);
    return rc != cudaSuccess ? rc : launch_ll(dt, a, shape(g), st);
  }
  if (var == kVarOneShot) {
    // the recursive-doubling order costs n log n combines per element: give a CTA less of it
    const Geometry g = plan_xchg(bytes, n(), views[0].half_bytes, tune,
                                 order == kOrderDoubling ? std::min<size_t>(2 * 1024, tune.grain) : tune.grain);
    HX_CHECK_PLAN(kPlanXchg, g, bytes);
    std::vector<XchgArgs> args(views.size());
    for (size_t r = 0; r < views.size(); ++r)
      build_allreduce_oneshot(&args[r], views[r], epoch, g, b[r].send, b[r].recv, count, dt, plan, order);
    epoch += g.epochs;
    const XchgArgs* a = stage(args, st, &rc);
    return rc != cudaSuccess ? rc : launch_xchg_fold(dt, a, shape(g), st);
  }
  if (var == kVarRing) {
    const size_t es = dtype_size(dt);
    const Geometry g = plan_ring((count + n() - 1) / n() * es, n(), views[0].half_bytes, tune);
    HX_CHECK_PLAN(kPlanRing, g, (count + n() - 1) / n() * es);
    std::vector<TwoShotArgs> args(views.size());
    for (size_t r = 0; r < views.size(); ++r)
      build_allreduce_twoshot(&args[r], views[r], epoch, g, b[r].send, b[r].recv, count, dt, plan, order, false);
    epoch += g.epochs;
    const TwoShotArgs* a = stage(args, st, &rc);
    return rc != cudaSuccess ? rc : launch_ring(dt, a, shape(g), st);
  }
  // The three-role pipeline wins for the multicast reduction from three ranks on; for the
  // exact two-shot it measured faster than the single-role kernel only on eight ranks.
  const bool roles = tune.max_ctas >= 3 &&
                     (row ? (row->variant == kVarTwoShotRoles || row->variant == kVarNvlsRoles)
                          : bytes >= tune.roles_min && (var == kVarNvls ? n() > 2 : n() >= tune.roles_min_ranks));
  const Geometry g = roles ? plan_roles(bytes, n(), views[0].half_bytes, tune)
                           : plan_sliced(bytes, n(), views[0].half_bytes, tune);
  HX_CHECK_PLAN(roles ? kPlanRoles : kPlanSliced, g, bytes);
  if (var == kVarNvls) {
    std::vector<NvlsArgs> args(1);
    build_allreduce_nvls(&args[0], views[0], epoch, g, b[0].send, b[0].recv, count, dt, plan);
    epoch += g.epochs;
    if (roles) last_variant = kVarNvlsRoles;
    return launch_nvls(args.data(), shape(g), st, roles);
  }
  std::vector<TwoShotArgs> args(views.size());
  for (size_t r = 0; r < views.size(); ++r)
    // Publishing results with one multimem.st per vector saves link egress, but measured
    // slower than peer stores wherever the kernel is not egress-bound: it pays off only in
    // the three-role pipeline on more than two ranks.
    build_allreduce_twoshot(&args[r], views[r], epoch, g, b[r].send, b[r].recv, count, dt, plan,
                            order, tune.nvls && tune.nvls_gather && roles && n() > 2 && bytes % 16 == 0);
  epoch += g.epochs;
  const TwoShotArgs* a = stage(args, st, &rc);
  if (rc != cudaSuccess) return rc;
  if (roles) last_variant = kVarTwoShotRoles;
  return roles ? launch_twoshot_roles(dt, a, shape(g), st) : launch_twoshot(dt, a, shape(g), st);
}

cudaError_t Engine::allreduce_cast(const RankBufs* b, size_t count, int wire_dt, const OpPlan& plan,
                                   cudaStream_t st) {
  const size_t bytes = count * dtype_size(wire_dt);
  const Geometry g = plan_sliced(bytes, n(), views[0].half_bytes, tune);
  HX_CHECK_PLAN(kPlanSliced, g, bytes);
  std::vector<TwoShotArgs> args(views.size());
  for (size_t r = 0; r < views.size(); ++r)
    build_allreduce_twoshot(&args[r], views[r], epoch, g, b[r].send, b[r].recv, count, wire_dt, plan, kOrderRing, false);
  epoch += g.epochs;
  ++launches;
  last_variant = kVarTwoShot;
  cudaError_t rc;
  const TwoShotArgs* a = stage(args, st, &rc);
  return rc != cudaSuccess ? rc : launch_twoshot_cast(wire_dt, a, shape(g), st);
}

cudaError_t Engine::reducescatter(const RankBufs* b, size_t per, int dt, const OpPlan& plan,
                                  cudaStream_t st) {
  const size_t block = per * dtype_size(dt);
  // Large inputs go around the neighbour ring (one sender per receiver through the switch, the
  // same schedule and therefore the same bits); smaller ones are pushed to their owners at once.
  const TuneRow* row = forced_variant == kVarAuto ? find_row(this->tune, kCollReduceScatter, n(), int(dtype_size(dt)), true, block) : nullptr;
  const bool ring = row ? row->variant == 1
                        : ((this->tune.rs_ring_min && block * n() >= this->tune.rs_ring_min) || forced_variant == kVarRing);
  const Tuning tune = with_row(this->tune, row, ring ? kVarRing : kVarOneShot);
  if (n() >= 2 && block > 0 && ring) {
    const Geometry g = plan_ring(block, n(), views[0].half_bytes, tune, true);
    HX_CHECK_PLAN(kPlanRingRs, g, block);
    std::vector<TwoShotArgs> args(views.size());
    for (size_t r = 0; r < views.size(); ++r)
      build_reducescatter_ring(&args[r], views[r], epoch, g, b[r].send, b[r].recv, per, dt, plan);
    epoch += g.epochs;
    ++launches;
    cudaError_t rc;
    const TwoShotArgs* a = stage(args, st, &rc);
    return rc != cudaSuccess ? rc : launch_ring(dt, a, shape(g), st);
  }
  const Geometry g = plan_xchg(per * dtype_size(dt), n(), views[0].half_bytes, tune);
  HX_CHECK_PLAN(kPlanXchg, g, per * dtype_size(dt));
  std::vector<XchgArgs> args(views.size());
  for (size_t r = 0; r < views.size(); ++r)
    build_reducescatter(&args[r], views[r], epoch, g, b[r].send, b[r].recv, per, dt, plan);
  epoch += g.epochs;
  ++launches;
  cudaError_t rc;
  const XchgArgs* a = stage(args, st, &rc);
  return rc != cudaSuccess ? rc : launch_xchg_fold(dt, a, shape(g), st);
}

cudaError_t Engine::reduce(const RankBufs* b, size_t count, int dt, const OpPlan& plan, int root,
                           cudaStream_t st) {
  const Geometry g = plan_xchg(count * dtype_size(dt), n(), views[0].half_bytes, tune);
  HX_CHECK_PLAN(kPlanXchg, g, count * dtype_size(dt));
  std::vector<XchgArgs> args(views.size());
  for (size_t r = 0; r < views.size(); ++r)
    build_reduce(&args[r], views[r], epoch, g, b[r].send, b[r].recv, count, dt, plan, root);
  epoch += g.epochs;
  ++launches;
  cudaError_t rc;
  const XchgArgs* a = stage(args, st, &rc);
  return rc != cudaSuccess ? rc : launch_xchg_fold(dt, a, shape(g), st);
}

#define HX_COPY_COLLECTIVE(MAXPAIR, BUILD)                                  \
  const Geometry g = plan_xchg(MAXPAIR, n(), views[0].half_bytes, tune);    \
  HX_CHECK_PLAN(kPlanXchg, g, MAXPAIR);                                     \
  std::vector<XchgArgs> args(views.size());                                 \
  for (size_t r = 0; r < views.size(); ++r) { BUILD; }                      \
  epoch += g.epochs;                                                         \
  ++launches;                                                               \
  cudaError_t rc;                                                           \
  const XchgArgs* a = stage(args, st, &rc);                                 \
  return rc != cudaSuccess ? rc : launch_xchg_copy(a, shape(g), st);

cudaError_t Engine::allgather(const RankBufs* b, size_t block, cudaStream_t st) {
  // AllGather moves the same bytes into every rank whichever way they are pushed, so multicast
  // only spares the sender's link; it pays where the table measured it to.
  const TuneRow* row = find_row(this->tune, kCollAllGather, n(), 0, true, block);
  const Tuning tune = with_row(this->tune, row, kVarOneShot);
  const bool mc = tune.nvls && tune.mc_copy && !world() && block >= tune.mc_copy_min &&
                  (tune.mc_force >= 0 ? tune.mc_force == 1 : (row && row->variant == 1));
  HX_COPY_COLLECTIVE(block, build_allgather(&args[r], views[r], epoch, g, b[r].send, b[r].recv, block, mc))
}
cudaError_t Engine::broadcast(const RankBufs* b, size_t bytes, int root, cudaStream_t st) {
  // A root that stores to every peer sends the message n-1 times over its one link; through
  // the switch's multicast it sends it once. Without a table row: multicast from three ranks on.
  const TuneRow* row = find_row(this->tune, kCollBroadcast, n(), 0, true, bytes);
  const Tuning tune = with_row(this->tune, row, kVarOneShot);
  const bool mc = tune.nvls && tune.mc_copy && !world() && bytes >= tune.mc_copy_min &&
                  (tune.mc_force >= 0 ? tune.mc_force == 1 : (row ? row->variant == 1 : n() > 2));
  HX_COPY_COLLECTIVE(bytes, build_broadcast(&args[r], views[r], epoch, g, b[r].send, b[r].recv, bytes, root, mc))
}
cudaError_t Engine::gather(const RankBufs* b, size_t block, int root, cudaStream_t st) {
  HX_COPY_COLLECTIVE(block, build_gather(&args[r], views[r], epoch, g, b[r].send, b[r].recv, block, root))
}
cudaError_t Engine::scatter(const RankBufs* b, size_t block, int root, cudaStream_t st) {
  HX_COPY_COLLECTIVE(block, build_scatter(&args[r], views[r], epoch, g, b[r].send, b[r].recv, block, root))
}
cudaError_t Engine::alltoallv(const RankV* v, size_t max_pair, cudaStream_t st) {
  HX_COPY_COLLECTIVE(max_pair, build_alltoallv(&args[r], views[r], epoch, g, v[r].send, v[r].sbytes,
                                               v[r].soff, v[r].recv, v[r].rbytes, v[r].roff))
}

// Send/Recv: operations toward one peer in one direction share a lane and keep their order.
// A rank's transfers to itself are paired here and become plain device copies.
cudaError_t Engine::p2p(const RankP2p* ops, cudaStream_t st) {
  const size_t nr = views.size();
  std::vector<std::vector<P2pOp>> left(nr);
  for (size_t r = 0; r < nr; ++r) {
    const int me = views[r].rank;
    std::vector<P2pOp> sends, recvs;
    for (const P2pOp& o : ops[r].ops) {
      if (o.peer != me)
        left[r].push_back(o);
      else
        (o.is_send ? sends : recvs).push_back(o);
    }
    if (sends.size() != recvs.size()) {
      error = "a Send to the calling rank needs a matching Recv in the same group";
      return cudaErrorInvalidValue;
    }
    for (size_t k = 0; k < sends.size(); ++k) {
      const size_t nbytes = std::min(sends[k].bytes, recvs[k].bytes);
      if (nbytes && sends[k].buf != recvs[k].buf) {
        ++launches;
        if (cudaError_t e = launch_copy(recvs[k].buf, sends[k].buf, nbytes, st)) return e;
      }
      if (sends[k].bytes > recvs[k].bytes) {
        error = "message truncated: the receive buffer is smaller than the message";
        return cudaErrorInvalidValue;
      }
    }
  }
  // Every CTA of a lane waits for the matching CTA of its peer, so all CTAs of a launch must be
  // resident at once on every rank. The grid is sized for the most lanes a rank of this
  // communicator can have (a send and a receive lane per peer), from numbers every rank shares:
  // when lanes x kP2pWorkers CTAs do not fit, one CTA serves several workers of its lane one
  // after the other (both ends of a lane walk them in the same order, so the pairing holds).
  const int sharing = world() ? int(nr) : 1;
  const int most_lanes = std::max(1, std::min(kMaxLanes, 2 * (n() - 1)));
  auto workers_per_cta = [&](int width) {
    const int resident = max_resident_ctas(width) / sharing;
    int wpc = 1;
    while (wpc < kP2pWorkers && most_lanes * (kP2pWorkers / wpc) > resident) wpc *= 2;
    return most_lanes * (kP2pWorkers / wpc) <= resident ? wpc : 0;
  };
  int threads = world() ? 256 : tune.p2p_threads;
  int wpc = workers_per_cta(threads);
  if (threads == 512 && wpc != 1) {  // narrower CTAs: twice as many are resident
    const int narrow = workers_per_cta(256);
    if (narrow && (!wpc || narrow < wpc)) threads = 256, wpc = narrow;
  }
  if (!wpc) {
    error = "Send/Recv lanes of " + std::to_string(n()) + " ranks cannot be co-resident on this device";
    return cudaErrorInvalidValue;
  }
  for (;;) {  // a lane takes kMaxLaneOps operations per launch; more go into another round
    bool any = false;
    std::vector<P2pArgs> args(nr);
    int max_lanes = 0;
    for (size_t r = 0; r < nr; ++r) {
      P2pArgs& a = args[r];
      std::memset(&a, 0, sizeof a);
      a.w = views[r];
      a.workers_per_cta = wpc;
      a.bulk = tune.p2p_bulk && !world() ? 1 : 0;
      std::vector<P2pOp> rest;
      for (const P2pOp& o : left[r]) {
        int lane = -1;
        for (int k = 0; k < a.nlanes; ++k)
          if (a.lanes[k].peer == o.peer && a.lanes[k].is_send == int(o.is_send)) lane = k;
        if (lane < 0 && a.nlanes < kMaxLanes) {
          lane = a.nlanes++;
          a.lanes[lane].peer = o.peer;
          a.lanes[lane].is_send = o.is_send;
          a.lanes[lane].nops = 0;
        }
        // an operation that does not fit, or that follows one of its lane that did not fit,
        // waits for the next round so the lane's order holds
        const bool blocked = std::any_of(rest.begin(), rest.end(), [&](const P2pOp& q) {
          return q.peer == o.peer && q.is_send == o.is_send;
        });
        if (lane < 0 || blocked || a.lanes[lane].nops == kMaxLaneOps) {
          rest.push_back(o);
          continue;
        }
        a.lanes[lane].ops[a.lanes[lane].nops++] = P2pLaneOp{static_cast<char*>(o.buf), o.bytes};
      }
      left[r].swap(rest);
      int used = 0;
      for (int k = 0; k < a.nlanes; ++k) used += a.lanes[k].nops > 0;
      any = any || used > 0;
      max_lanes = std::max(max_lanes, a.nlanes);
    }
    if (!any) return cudaSuccess;
    ++launches;
    cudaError_t rc;
    const P2pArgs* a = stage(args, st, &rc);
    if (rc != cudaSuccess) return rc;
    rc = launch_p2p(a, LaunchShape{max_lanes * (kP2pWorkers / wpc), threads, world() ? int(nr) : 0}, st);
    if (rc != cudaSuccess) return rc;
  }
}

}  // namespace hx
