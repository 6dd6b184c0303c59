#include "device/planner.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>

#include "device/nvls_modes.h"
#include "math/dtypes.h"

namespace hx {
namespace {
size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }
size_t round_down(size_t v, size_t m) { return v / m * m; }
size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

int threads_for(size_t bytes_per_cta) { return bytes_per_cta >= 32 * 1024 ? 512 : 256; }

// bytes of one staging buffer: a whole half for a single step, a quarter of the staging area
// (kRing = 4 buffers, device code: prims.cuh) for a pipelined launch
size_t buffer_bytes(size_t half_bytes, int steps) {
  return steps == 1 ? half_bytes : round_down(2 * half_bytes / 4, 256);
}

void clear(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g) {
  std::memset(a, 0, sizeof *a);
  a->w = w;
  a->epoch0 = epoch;
  a->steps = g.steps;
  a->sub_bytes = g.sub_bytes;
  a->slot_stride = round_down(buffer_bytes(w.half_bytes, g.steps) / w.n, 256);
}

// Splits `per_cta_total` bytes (what one CTA moves for one pair / slice over the whole launch)
// into steps. Small amounts go in one step (lowest latency); larger ones in at least eight
// steps of 4..sub_max KiB so that the pipeline has something to overlap.
void split_steps(Geometry* g, size_t per_cta_total, size_t fit_single, size_t fit_ring, const Tuning& t) {
  const size_t want = std::max<size_t>(16, round_up(per_cta_total, 16));
  if (want <= t.single_sub_max && want <= fit_single) {
    g->sub_bytes = want;
    g->steps = 1;
    return;
  }
  size_t sub = std::min(std::max(round_up(want / std::max(2, t.min_steps), 16), size_t(4096)), t.sub_max);
  sub = std::max<size_t>(16, std::min(sub, fit_ring));
  g->steps = int(ceil_div(want, sub));
  if (g->steps == 1 && want > fit_single) g->steps = 2;  // cannot happen with sane windows
  // equal steps: no short last step when the window, not the tuning, set the size
  g->sub_bytes = std::max<size_t>(16, std::min(sub, round_up(ceil_div(want, size_t(g->steps)), 16)));
}
}  // namespace

bool set_knob(Tuning* t, const char* name, long v) {
  const std::string k(name ? name : "");
  if (k == "max_ctas") t->max_ctas = int(std::max(1L, std::min<long>(v, kMaxCtas)));
  else if (k == "oneshot_max") t->oneshot_max = size_t(v);
  else if (k == "nvls_min") t->nvls_min = size_t(v);
  else if (k == "single_sub_max") t->single_sub_max = size_t(v);
  else if (k == "sub_max") t->sub_max = size_t(std::max(16L, v / 16 * 16));
  else if (k == "min_steps") t->min_steps = int(std::max(2L, v));
  else if (k == "threads") t->threads = (v == 256 || v == 512) ? int(v) : 0;
  else if (k == "roles_min") t->roles_min = size_t(v);
  else if (k == "roles_sub") t->roles_sub = size_t(std::max(16L, v / 16 * 16));
  else if (k == "ring_min") t->ring_min = size_t(std::max(0L, v));
  else if (k == "ring_sub") t->ring_sub = size_t(std::max(16L, v / 16 * 16));
  else if (k == "p2p_threads") t->p2p_threads = v == 512 ? 512 : 256;
  else if (k == "ring_max_ranks") t->ring_max_ranks = int(std::max(2L, v));
  else if (k == "roles_min_ranks") t->roles_min_ranks = int(std::max(2L, v));
  else if (k == "exact") t->exact = v != 0;
  else if (k == "nvls_gather") t->nvls_gather = v != 0;
  else if (k == "ll_max") t->ll_max = size_t(std::max(0L, v));
  else if (k == "ll_mc") t->ll_mc = v != 0;
  else if (k == "rs_ring_min") t->rs_ring_min = size_t(std::max(0L, v));
  else if (k == "table") t->use_table = v != 0;
  else if (k == "p2p_bulk") t->p2p_bulk = v != 0;
  else if (k == "grain") t->grain = size_t(std::max(256L, v));
  else if (k == "mc_force") t->mc_force = v < 0 ? -1 : (v != 0);
  else if (k == "mc_copy") t->mc_copy = v != 0;
  else if (k == "mc_copy_min") t->mc_copy_min = size_t(std::max(0L, v));
  else return false;
  return true;
}

namespace {
const char* const kDefaultTable =
#include "device/tune_default.inc"
    ;
const char* const kCollNames[] = {"allreduce", "allgather", "reducescatter", "broadcast"};
const char* const kVariantNames[] = {"auto", "oneshot", "twoshot", "nvls", "twoshot_roles", "nvls_roles", "ring", "lines"};
}  // namespace

bool parse_row(const std::string& line, TuneRow* row, std::string* why) {
  std::istringstream in(line);
  std::string word;
  in >> word;  // "row"
  if (!(in >> word)) {
    *why = "row without a collective";
    return false;
  }
  *row = TuneRow{};
  row->coll = -1;
  for (int c = 0; c < 4; ++c)
    if (word == kCollNames[c]) row->coll = c;
  if (row->coll < 0) {
    *why = "unknown collective '" + word + "' in a table row";
    return false;
  }
  bool have_n = false, have_variant = false;
  while (in >> word) {
    const size_t eq = word.find('=');
    if (eq == std::string::npos) {
      *why = "table row field '" + word + "' is not key=value";
      return false;
    }
    const std::string key = word.substr(0, eq), val = word.substr(eq + 1);
    char* end = nullptr;
    const long long num = std::strtoll(val.c_str(), &end, 10);
    const bool numeric = !val.empty() && *end == 0;
    if (key == "mode") {
      if (val != "exact" && val != "fast" && val != "any") {
        *why = "table row mode '" + val + "'";
        return false;
      }
      row->exact = val == "exact" ? 1 : (val == "fast" ? 0 : -1);
      continue;
    }
    if (key == "variant") {
      have_variant = true;
      if (numeric) {
        row->variant = int(num);
        continue;
      }
      row->variant = -1;
      for (int v = 0; v < 8; ++v)
        if (val == kVariantNames[v]) row->variant = v;
      if (val == "multicast" || val == "ring_rs") row->variant = 1;
      if (val == "unicast" || val == "push") row->variant = 0;
      if (row->variant < 0) {
        *why = "unknown variant '" + val + "' in a table row";
        return false;
      }
      continue;
    }
    if (!numeric || num < 0) {
      *why = "table row field '" + word + "' needs a non-negative number";
      return false;
    }
    if (key == "n") row->n = int(num), have_n = true;
    else if (key == "es") row->es = int(num);
    else if (key == "from") row->from = size_t(num);
    else if (key == "ctas") row->ctas = int(std::min<long long>(num, kMaxCtas));
    else if (key == "threads") row->threads = (num == 256 || num == 512) ? int(num) : 0;
    else if (key == "sub") row->sub = size_t(num) / 16 * 16;
    else if (key == "grain") row->grain = size_t(num);
    else {
      *why = "unknown table row field '" + key + "'";
      return false;
    }
  }
  if (!have_n || !have_variant || row->n < 2 || row->n > kMaxRanks) {
    *why = "a table row needs n=<2..16> and variant=";
    return false;
  }
  return true;
}

void load_default_table(Tuning* t) {
  std::istringstream in(kDefaultTable);
  std::string line, why;
  while (std::getline(in, line)) {
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line.erase(hash);
    if (line.find("row") == std::string::npos) continue;
    TuneRow row;
    if (parse_row(line, &row, &why)) {
      if (!t->rows) t->rows = std::make_shared<std::vector<TuneRow>>();
      t->rows->push_back(row);
    }
  }
}

const TuneRow* find_row(const Tuning& t, int coll, int n, int es, bool exact, size_t bytes) {
  if (!t.use_table || !t.rows) return nullptr;
  int best_n = 0;  // the tabled rank count that serves n
  for (const TuneRow& r : *t.rows)
    if (r.coll == coll && r.n <= n && r.n > best_n) best_n = r.n;
  const TuneRow* best = nullptr;
  for (const TuneRow& r : *t.rows) {
    if (r.coll != coll || r.n != best_n || r.from > bytes) continue;
    if (r.es != 0 && r.es != es) continue;
    if (r.exact >= 0 && r.exact != (exact ? 1 : 0)) continue;
    // later criteria break ties of earlier ones: exact element size, then the largest `from`
    if (!best || (r.es != 0) > (best->es != 0) || ((r.es != 0) == (best->es != 0) && r.from >= best->from)) best = &r;
  }
  return best;
}

Tuning with_row(const Tuning& t, const TuneRow* row, int variant) {
  Tuning out = t;
  if (!row) return out;
  if (row->ctas > 0) out.max_ctas = std::min(row->ctas, kMaxCtas);
  if (row->threads) out.threads = row->threads;
  if (row->grain >= 256) out.grain = row->grain;
  if (row->sub >= 16) {
    if (variant == kVarRing) out.ring_sub = row->sub;
    else if (variant == kVarTwoShotRoles || variant == kVarNvlsRoles) out.roles_sub = row->sub;
    else out.sub_max = row->sub;
  }
  return out;
}

bool load_tune_file(Tuning* t, const char* path, std::string* why) {
  std::ifstream in(path);
  if (!in) {
    *why = std::string("cannot read HXCCL_TUNE_FILE ") + path;
    return false;
  }
  std::string line;
  bool own_rows = false;
  while (std::getline(in, line)) {
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line.erase(hash);
    {
      std::istringstream first(line);
      std::string word;
      if ((first >> word) && word == "row") {
        TuneRow row;
        if (!parse_row(line, &row, why)) {
          *why = "HXCCL_TUNE_FILE: " + *why;
          return false;
        }
        if (!own_rows) t->rows = std::make_shared<std::vector<TuneRow>>();  // replaces the compiled-in table
        own_rows = true;
        t->rows->push_back(row);
        continue;
      }
    }
    for (char& ch : line)
      if (ch == '=' || ch == '\t' || ch == '\r') ch = ' ';
    char name[64];
    long value = 0;
    const int got = std::sscanf(line.c_str(), " %63s %ld", name, &value);
    if (got <= 0) continue;  // blank
    if (got != 2 || !set_knob(t, name, value)) {
      *why = std::string("HXCCL_TUNE_FILE: cannot use the line for '") + name + "'";
      return false;
    }
  }
  return true;
}

namespace {
// Every CTA of a collective launch waits for the same CTA of its peers, so a grid must be
// co-resident: one 512-thread CTA per SM, two of 256 threads. Only a fixed width of 256 can
// count on the second.
int grid_cap(const Tuning& t) {
  const int resident = (t.threads == 256 ? 2 : 1) * std::max(1, t.sm_count);
  return std::max(1, std::min(std::min(t.max_ctas, kMaxCtas), resident));
}
}  // namespace

Geometry plan_xchg(size_t max_pair, int n, size_t half_bytes, const Tuning& t, size_t cta_bytes) {
  Geometry g;
  const int cap = grid_cap(t);
  if (cta_bytes == 0) cta_bytes = t.grain;
  g.ctas = int(std::min<size_t>(cap, std::max<size_t>(1, ceil_div(max_pair, std::max<size_t>(256, cta_bytes)))));
  const size_t fit1 = round_down(round_down(buffer_bytes(half_bytes, 1) / n, 256) / g.ctas, 16);
  const size_t fitr = round_down(round_down(buffer_bytes(half_bytes, 2) / n, 256) / g.ctas, 16);
  split_steps(&g, ceil_div(max_pair, g.ctas), fit1, fitr, t);
  g.epochs = g.steps == 1 ? 1 : g.steps + 2;
  g.threads = t.threads && g.steps > 1 ? t.threads : threads_for(g.sub_bytes * n);
  return g;
}

Geometry plan_sliced(size_t bytes, int n, size_t half_bytes, const Tuning& t) {
  Geometry g;
  const int cap = grid_cap(t);
  g.ctas = int(std::min<size_t>(cap, std::max<size_t>(1, ceil_div(bytes, size_t(n) * std::max<size_t>(256, t.grain)))));
  // a buffer holds the phase A slots in its first half and the phase B slots in its second
  const size_t fit1 = round_down(round_down(buffer_bytes(half_bytes, 1) / 2, 256) / n / g.ctas, 16);
  const size_t fitr = round_down(round_down(buffer_bytes(half_bytes, 2) / 2, 256) / n / g.ctas, 16);
  split_steps(&g, ceil_div(bytes, size_t(n) * g.ctas), fit1, fitr, t);
  g.epochs = g.steps == 1 ? 1 : g.steps + 2;
  g.threads = t.threads && g.steps > 1 ? t.threads : threads_for(g.sub_bytes * n);
  return g;
}

Geometry plan_roles(size_t bytes, int n, size_t half_bytes, const Tuning& t) {
  Geometry g;
  // Unless told otherwise the pipeline runs 256-thread CTAs, two per SM: each role then has
  // twice as many CTAs issuing link traffic, which measured faster than 512-thread CTAs.
  g.threads = t.threads ? t.threads : 256;
  const int per_sm = g.threads <= 256 ? 2 : 1;
  const int cap = std::max(3, std::min(std::min(per_sm * t.max_ctas, per_sm * t.sm_count - 2), kMaxCtas));
  int lanes = std::max(1, cap / 3);
  lanes = int(std::min<size_t>(lanes, std::max<size_t>(1, ceil_div(bytes, size_t(n) * 16 * 1024))));
  // a ring buffer holds the staged inputs in its first half and the results in its second
  const size_t fit = round_down(round_down(buffer_bytes(half_bytes, 2) / 2, 256) / n / lanes, 16);
  g.sub_bytes = std::max<size_t>(16, std::min(std::min(round_up(t.roles_sub, 16), fit),
                                              round_up(ceil_div(bytes, size_t(n) * lanes), 16)));
  g.ctas = 3 * lanes;
  g.steps = int(std::max<size_t>(1, ceil_div(bytes, g.sub_bytes * lanes * n)));
  g.epochs = g.steps + 1;
  return g;
}

Geometry plan_ring(size_t max_block, int n, size_t half_bytes, const Tuning& t, bool rs) {
  Geometry g;
  const int cap = grid_cap(t);
  g.ctas = int(std::min<size_t>(cap, std::max<size_t>(1, ceil_div(max_block, 16 * 1024))));
  // the staging area holds one slot per hop (2n - 2) and CTA
  const size_t hops = size_t(2 * n - 2);
  const size_t fit = round_down(2 * half_bytes / std::max<size_t>(1, hops) / g.ctas, 256);
  const size_t want = std::max<size_t>(16, round_up(ceil_div(max_block, g.ctas), 16));
  g.sub_bytes = std::max<size_t>(16, std::min(want, std::min(round_up(t.ring_sub, 16), fit)));
  g.steps = int(std::max<size_t>(1, ceil_div(want, g.sub_bytes)));
  g.epochs = g.steps * int(rs ? n - 1 : hops) + 2;
  g.threads = t.threads ? t.threads : threads_for(g.sub_bytes);
  return g;
}

std::string check_geometry(int kind, const Geometry& g, size_t amount, int n, size_t half_bytes) {
  auto num = [](size_t v) { return std::to_string(v); };
  if (g.ctas < 1 || g.ctas > kMaxCtas) return "grid of " + num(size_t(g.ctas)) + " CTAs does not fit the flag rows";
  if (g.threads != 256 && g.threads != 512) return "CTA width " + num(size_t(g.threads));
  if (g.steps < 1 || g.sub_bytes < 16 || g.sub_bytes % 16) return "step of " + num(g.sub_bytes) + " bytes";
  if (n < 1 || n > kMaxRanks) return "rank count " + num(size_t(n));
  const size_t ctas = size_t(g.ctas), steps = size_t(g.steps), ranks = size_t(n);
  if (kind == kPlanXchg) {
    const size_t buf = buffer_bytes(half_bytes, g.steps), stride = round_down(buf / ranks, 256);
    if (g.epochs != (g.steps == 1 ? 1 : g.steps + 2)) return "epoch count";
    if (ctas * g.sub_bytes > stride || ranks * stride > buf) return "a source's slots overrun its share of the buffer";
    if (steps * ctas * g.sub_bytes < amount) return "steps do not cover the block";
  } else if (kind == kPlanSliced || kind == kPlanRoles) {
    const bool roles = kind == kPlanRoles;
    if (roles && (g.ctas % 3 || g.epochs != g.steps + 1)) return "role pipeline shape";
    if (!roles && g.epochs != (g.steps == 1 ? 1 : g.steps + 2)) return "epoch count";
    const size_t buf = roles ? buffer_bytes(half_bytes, 2) : buffer_bytes(half_bytes, g.steps);
    const size_t second = round_down(buf / 2, 256), slice = (roles ? ctas / 3 : ctas) * g.sub_bytes;
    if (ranks * slice > second || second + ranks * slice > buf) return "slices overrun a half of the buffer";
    if (steps * ranks * slice < amount) return "steps do not cover the message";
  } else if (kind == kPlanRing || kind == kPlanRingRs) {
    const size_t hops = size_t(2 * n - 2);
    if (n < 2 || g.epochs != g.steps * (kind == kPlanRingRs ? n - 1 : int(hops)) + 2) return "ring shape";
    if (hops * ctas * g.sub_bytes > 2 * half_bytes) return "ring slots overrun the staging area";
    if (steps * ctas * g.sub_bytes < amount) return "rounds do not cover a block";
  } else {
    return "unknown plan kind";
  }
  return std::string();
}

FoldSpec make_fold(const OpPlan& plan, int kind) {
  FoldSpec f{};
  f.kind = kind;
  f.op = plan.base;
  f.dir = 1;
  f.premul = plan.premul ? 1 : 0;
  f.postdiv = plan.postdiv ? plan.divisor : 0;
  std::memcpy(&f.scalar_bits, plan.scalar, 8);
  f.scalar_ptr = plan.scalar_dev;
  return f;
}

int choose_variant(size_t bytes, int dt, const OpPlan& plan, int n, const Tuning& t, int forced,
                   const TuneRow** row_out) {
  if (row_out) *row_out = nullptr;
  const bool nvls_ok = t.nvls && bytes % 16 == 0 && bytes > 0 &&
                       nvls_mode(dt, plan.base) != kNvNone && (is_integer(dt) || !t.exact);
  if (forced == kVarNvls && nvls_ok) return kVarNvls;
  if (forced == kVarOneShot || forced == kVarTwoShot) return forced;
  const bool ll_ok = bytes > 0 && bytes <= ll_max_payload(n) && n >= 2;
  if (forced == kVarLL && ll_ok) return kVarLL;
  if (forced == kVarRing && n >= 2 && bytes > 0) return kVarRing;
  if (forced == kVarAuto && bytes > 0) {  // the measured table first, where it has an answer that can run
    if (const TuneRow* r = find_row(t, kCollAllReduce, n, int(dtype_size(dt)), t.exact, bytes)) {
      int v = r->variant;
      if (v == kVarTwoShotRoles) v = kVarTwoShot;  // the role pipeline is the planner's choice by size
      if (v == kVarNvlsRoles) v = kVarNvls;
      const bool can = (v == kVarLL && ll_ok) || v == kVarOneShot || v == kVarTwoShot || (v == kVarRing && n >= 2) ||
                       (v == kVarNvls && nvls_ok);
      if (can) {
        if (row_out) *row_out = r;
        return v;
      }
    }
  }
  // with two ranks the multicast reduction measured slower than two-shot at every size
  if (nvls_ok && bytes >= t.nvls_min && n > 2) return kVarNvls;
  if (t.ring_min && bytes >= t.ring_min && n >= 2 && n <= t.ring_max_ranks) return kVarRing;
  if (ll_ok && bytes <= t.ll_max && forced == kVarAuto) return kVarLL;
  return bytes <= t.oneshot_max ? kVarOneShot : kVarTwoShot;
}

void build_allreduce_oneshot(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                             const void* send, void* recv, size_t count, int dt,
                             const OpPlan& plan, int order) {
  clear(a, w, epoch, g);
  const size_t bytes = count * dtype_size(dt);
  for (int j = 0; j < w.n; ++j) {
    a->send_ptr[j] = static_cast<const char*>(send);
    a->send_bytes[j] = j == w.rank ? 0 : bytes;
  }
  a->fold_dst = static_cast<char*>(recv);
  a->own_ptr = static_cast<const char*>(send);
  a->fold_bytes = bytes;
  a->fold_elem0 = 0;
  a->fold = make_fold(plan, order == kOrderRing ? kFoldLinear : kFoldDoubling);
  a->fold.ring = order == kOrderRing;
  a->fold.ring_count = count;
  a->push_scaled = plan.premul;
}

void build_allreduce_ll(LLArgs* a, const WinView& w, uint64_t epoch, const void* send, void* recv,
                        size_t count, int dt, const OpPlan& plan, int order, bool use_mc) {
  std::memset(a, 0, sizeof *a);
  a->w = w;
  a->epoch = epoch;
  a->send = static_cast<const char*>(send);
  a->recv = static_cast<char*>(recv);
  a->bytes = count * dtype_size(dt);
  a->fold = make_fold(plan, order == kOrderRing ? kFoldLinear : kFoldDoubling);
  a->fold.ring = order == kOrderRing;
  a->fold.ring_count = count;
  a->use_mc = use_mc && w.mc != nullptr;
}

void build_allreduce_twoshot(TwoShotArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                             const void* send, void* recv, size_t count, int dt,
                             const OpPlan& plan, int order, bool use_mc) {
  std::memset(a, 0, sizeof *a);
  a->w = w;
  a->epoch0 = epoch;
  a->steps = g.steps;
  a->sub_bytes = g.sub_bytes;
  a->send = static_cast<const char*>(send);
  a->recv = static_cast<char*>(recv);
  a->bytes = count * dtype_size(dt);
  a->fold = make_fold(plan, order == kOrderRing ? kFoldLinear : kFoldDoubling);
  a->fold.ring = order == kOrderRing;
  a->fold.ring_count = count;
  a->use_mc = use_mc && w.mc != nullptr;
}

void build_allreduce_nvls(NvlsArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                          const void* send, void* recv, size_t count, int dt, const OpPlan& plan) {
  std::memset(a, 0, sizeof *a);
  a->w = w;
  a->epoch0 = epoch;
  a->steps = g.steps;
  a->sub_bytes = g.sub_bytes;
  a->send = static_cast<const char*>(send);
  a->recv = static_cast<char*>(recv);
  a->bytes = count * dtype_size(dt);
  a->op = plan.base;
  a->dt = dt;
  a->premul = plan.premul;
  a->postdiv = plan.postdiv ? plan.divisor : 0;
  std::memcpy(&a->scalar_bits, plan.scalar, 8);
  a->scalar_ptr = plan.scalar_dev;
}

void build_reducescatter_ring(TwoShotArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                              const void* send, void* recv, size_t per, int dt, const OpPlan& plan) {
  std::memset(a, 0, sizeof *a);
  a->w = w;
  a->epoch0 = epoch;
  a->steps = g.steps;
  a->sub_bytes = g.sub_bytes;
  a->send = static_cast<const char*>(send);
  a->recv = static_cast<char*>(recv);
  a->bytes = per * dtype_size(dt) * size_t(w.n);
  a->fold = make_fold(plan, kFoldLinear);
  a->fold.ring = 1;
  a->fold.ring_count = per * size_t(w.n);  // n equal blocks
  a->ring_rs = 1;
}

void build_reducescatter(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                         const void* send, void* recv, size_t per, int dt, const OpPlan& plan) {
  clear(a, w, epoch, g);
  const size_t block = per * dtype_size(dt);
  for (int j = 0; j < w.n; ++j) {
    a->send_ptr[j] = static_cast<const char*>(send) + size_t(j) * block;
    a->send_bytes[j] = j == w.rank ? 0 : block;
  }
  a->fold_dst = static_cast<char*>(recv);
  a->own_ptr = static_cast<const char*>(send) + size_t(w.rank) * block;
  a->fold_bytes = block;
  a->fold = make_fold(plan, kFoldLinear);  // block b: start with rank b+1, end with rank b
  a->fold.start = (w.rank + 1) % w.n;
  a->push_scaled = plan.premul;
}

void build_reduce(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                  const void* send, void* recv, size_t count, int dt, const OpPlan& plan,
                  int root) {
  clear(a, w, epoch, g);
  const size_t bytes = count * dtype_size(dt);
  for (int j = 0; j < w.n; ++j) {
    a->send_ptr[j] = static_cast<const char*>(send);
    a->send_bytes[j] = (w.rank != root && j == root) ? bytes : 0;
  }
  a->push_scaled = plan.premul;
  // the other ranks need the operator too: their pushes carry the scaled input
  if (bytes < kTreeMaxBytes) {
    a->fold = make_fold(plan, kFoldTree);
    a->fold.root = root;
  } else {  // chain toward the root: farthest position first
    a->fold = make_fold(plan, kFoldLinear);
    a->fold.start = (root + w.n - 1) % w.n;
    a->fold.dir = -1;
  }
  if (w.rank != root) return;  // only the root folds
  a->fold_dst = static_cast<char*>(recv);
  a->own_ptr = static_cast<const char*>(send);
  a->fold_bytes = bytes;
}

namespace {
// One multimem.st reaches every rank's window. It needs the multicast alias, whole 16-byte
// vectors and a 16-byte aligned source; a rank may decide this for itself, because the bytes
// land in the same slots either way.
void offer_multicast(XchgArgs* a, const WinView& w, const void* src, size_t bytes, bool wanted) {
  if (wanted && w.mc && w.n > 1 && bytes >= 16 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
    a->mc_src = static_cast<const char*>(src);
    a->mc_bytes = bytes;
  }
}
}  // namespace

void build_allgather(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                     const void* send, void* recv, size_t block, bool multicast) {
  clear(a, w, epoch, g);
  for (int j = 0; j < w.n; ++j) {
    a->send_ptr[j] = static_cast<const char*>(send);
    a->send_bytes[j] = j == w.rank ? 0 : block;
    a->recv_ptr[j] = static_cast<char*>(recv) + size_t(j) * block;
    a->recv_bytes[j] = block;
  }
  offer_multicast(a, w, send, block, multicast);
}

void build_broadcast(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                     const void* send, void* recv, size_t bytes, int root, bool multicast) {
  clear(a, w, epoch, g);
  for (int j = 0; j < w.n; ++j) {
    a->send_ptr[j] = static_cast<const char*>(send);
    a->send_bytes[j] = (w.rank == root && j != root) ? bytes : 0;
    a->recv_ptr[j] = static_cast<char*>(recv);
    a->recv_bytes[j] = j == root ? bytes : 0;  // on the root this is the send -> recv copy
  }
  if (w.rank == root) offer_multicast(a, w, send, bytes, multicast);
}

void build_gather(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                  const void* send, void* recv, size_t block, int root) {
  clear(a, w, epoch, g);
  for (int j = 0; j < w.n; ++j) {
    a->send_ptr[j] = static_cast<const char*>(send);
    a->send_bytes[j] = (w.rank != root && j == root) ? block : 0;
    if (w.rank == root) {
      a->recv_ptr[j] = static_cast<char*>(recv) + size_t(j) * block;
      a->recv_bytes[j] = block;
    }
  }
}

void build_scatter(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                   const void* send, void* recv, size_t block, int root) {
  clear(a, w, epoch, g);
  for (int j = 0; j < w.n; ++j) {
    a->send_ptr[j] = static_cast<const char*>(send) + size_t(j) * block;
    a->send_bytes[j] = (w.rank == root && j != root) ? block : 0;
    a->recv_ptr[j] = static_cast<char*>(recv);
    a->recv_bytes[j] = j == root ? block : 0;
  }
}

void build_alltoallv(XchgArgs* a, const WinView& w, uint64_t epoch, const Geometry& g,
                     const char* send, const size_t* sbytes, const size_t* soff, char* recv,
                     const size_t* rbytes, const size_t* roff) {
  clear(a, w, epoch, g);
  for (int j = 0; j < w.n; ++j) {
    a->send_ptr[j] = send + soff[j];
    a->send_bytes[j] = j == w.rank ? 0 : sbytes[j];
    a->recv_ptr[j] = recv + roff[j];
    a->recv_bytes[j] = rbytes[j];
  }
}

}  // namespace hx
