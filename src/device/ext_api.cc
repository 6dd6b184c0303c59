// Extension entry points (include/hxccl_ext.h) other than the single-GPU world.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "core/comm.h"
#include "device/planner.h"
#include "device/window_path.h"
#include "hxccl_ext.h"
#include "kernels/launch.h"
#include "math/reduce_host.h"

using namespace hx;

extern "C" {

hxcclResult_t hxcclCommDeviceInfo(hxcclComm_t c, char* kind, size_t kind_len, int* variant,
                                  unsigned long long* launches) {
  if (!c) return hxcclInvalidArgument;
  const char* k = c->device.path ? c->device.path->kind() : "none";
  if (kind && kind_len) {
    std::strncpy(kind, k, kind_len - 1);
    kind[kind_len - 1] = 0;
  }
  auto* w = dynamic_cast<WindowPath*>(c->device.path.get());
  if (variant) *variant = w ? w->engine().last_variant : 0;
  if (launches) *launches = w ? w->engine().launches : 0;
  return hxcclSuccess;
}

hxcclResult_t hxcclCommTune(hxcclComm_t c, int variant, int exact, int max_ctas) {
  if (!c) return hxcclInvalidArgument;
  auto* w = dynamic_cast<WindowPath*>(c->device.path.get());
  if (!w) return hxcclInvalidUsage;
  w->engine().forced_variant = variant;
  w->engine().tune.exact = exact != 0;
  if (max_ctas > 0) w->engine().tune.max_ctas = std::min(std::min(max_ctas, kMaxCtas), max_resident_ctas(512));
  return hxcclSuccess;
}

hxcclResult_t hxcclCommTuneKnob(hxcclComm_t c, const char* name, long value) {
  if (!c) return hxcclInvalidArgument;
  auto* w = dynamic_cast<WindowPath*>(c->device.path.get());
  if (!w) return hxcclInvalidUsage;
  return set_knob(&w->engine().tune, name, value) ? hxcclSuccess : hxcclInvalidArgument;
}

int hxcclCommReadTrace(hxcclComm_t c, unsigned long long* out, int max_ctas) {
  auto* w = c ? dynamic_cast<WindowPath*>(c->device.path.get()) : nullptr;
  return w && out && max_ctas > 0 ? w->read_trace(out, max_ctas) : 0;
}

static hxcclResult_t cuda_rc(cudaError_t e) { return e == cudaSuccess ? hxcclSuccess : hxcclUnhandledCudaError; }

hxcclResult_t hxcclDevReduce(void* dst, const void* src, size_t count, hxcclDataType_t dt,
                             hxcclRedOp_t op, hxcclStream_t stream) {
  if (dtype_size(dt) == 0 || !is_builtin_op(op) || (count && (!dst || !src))) return hxcclInvalidArgument;
  if (count == 0) return hxcclSuccess;
  return cuda_rc(launch_reduce(dst, src, count, dt, op, static_cast<cudaStream_t>(stream)));
}
hxcclResult_t hxcclDevScale(void* dst, const void* src, size_t count, hxcclDataType_t dt,
                            const void* scalar_host, hxcclStream_t stream) {
  if (dtype_size(dt) == 0 || !scalar_host || (count && (!dst || !src))) return hxcclInvalidArgument;
  if (count == 0) return hxcclSuccess;
  return cuda_rc(launch_scale(dst, src, count, dt, scalar_host, static_cast<cudaStream_t>(stream)));
}
hxcclResult_t hxcclDevDivide(void* buf, size_t count, hxcclDataType_t dt, int divisor,
                             hxcclStream_t stream) {
  if (!is_integer(dt) || divisor == 0 || (count && !buf)) return hxcclInvalidArgument;
  if (count == 0) return hxcclSuccess;
  return cuda_rc(launch_divide(buf, count, dt, divisor, static_cast<cudaStream_t>(stream)));
}

hxcclResult_t hxcclHostReduce(void* dst, const void* src, size_t count, hxcclDataType_t dt,
                              hxcclRedOp_t op) {
  if (dtype_size(dt) == 0 || !is_builtin_op(op)) return hxcclInvalidArgument;
  reduce_into(dst, src, count, dt, op);
  return hxcclSuccess;
}
hxcclResult_t hxcclHostScale(void* dst, const void* src, size_t count, hxcclDataType_t dt,
                             const void* scalar) {
  if (dtype_size(dt) == 0 || !scalar) return hxcclInvalidArgument;
  scale_into(dst, src, count, dt, scalar);
  return hxcclSuccess;
}
hxcclResult_t hxcclHostDivide(void* buf, size_t count, hxcclDataType_t dt, int divisor) {
  if (!is_integer(dt) || divisor == 0) return hxcclInvalidArgument;
  divide_trunc(buf, count, dt, divisor);
  return hxcclSuccess;
}
unsigned hxcclHostEncode(hxcclDataType_t dt, float v) {
  switch (dt) {
    case hxcclFloat16: { f16 h; from_f32(v, &h); return h.b; }
    case hxcclBfloat16: { bf16 h; from_f32(v, &h); return h.b; }
    case hxcclFloat8e4m3: { e4m3 h; from_f32(v, &h); return h.b; }
    case hxcclFloat8e5m2: { e5m2 h; from_f32(v, &h); return h.b; }
    default: return 0;
  }
}
float hxcclHostDecode(hxcclDataType_t dt, unsigned bits) {
  switch (dt) {
    case hxcclFloat16: return to_f32(f16{uint16_t(bits)});
    case hxcclBfloat16: return to_f32(bf16{uint16_t(bits)});
    case hxcclFloat8e4m3: return to_f32(e4m3{uint8_t(bits)});
    case hxcclFloat8e5m2: return to_f32(e5m2{uint8_t(bits)});
    default: return 0.0f;
  }
}
void hxcclRingBlock(size_t count, int n, int i, size_t* off, size_t* len) {
  const Span s = ring_block(count, n, i);
  *off = s.off;
  *len = s.len;
}

hxcclResult_t hxcclTestFailSends(hxcclComm_t c, long after) {
  if (!c) return hxcclInvalidArgument;
  c->wire->fail_after = after;
  return hxcclSuccess;
}
hxcclResult_t hxcclTestSeverPeer(hxcclComm_t c, int peer) {
  if (!c || peer < 0 || peer >= c->nranks) return hxcclInvalidArgument;
  c->chan->fabric().sever(c->chan->members()[peer]);
  return hxcclSuccess;
}

hxcclResult_t hxcclTestPlan(int kind, size_t amount, int nranks, size_t half_bytes, int max_ctas,
                            const char* knob, long knob_value, size_t shape[5], char* why, size_t why_len) {
  using namespace hx;
  if (nranks < 1 || nranks > kMaxRanks || !shape) return hxcclInvalidArgument;
  Tuning t;
  load_default_table(&t);
  if (const char* path = std::getenv("HXCCL_TUNE_FILE")) {
    std::string bad_line;
    if (!load_tune_file(&t, path, &bad_line)) {
      if (why && why_len) std::snprintf(why, why_len, "%s", bad_line.c_str());
      return hxcclInvalidArgument;
    }
  }
  if (max_ctas > 0) t.max_ctas = max_ctas;
  if (knob && *knob && !set_knob(&t, knob, knob_value)) return hxcclInvalidArgument;
  Geometry g;
  switch (kind) {
    case kPlanXchg: g = plan_xchg(amount, nranks, half_bytes, t); break;
    case kPlanSliced: g = plan_sliced(amount, nranks, half_bytes, t); break;
    case kPlanRoles: g = plan_roles(amount, nranks, half_bytes, t); break;
    case kPlanRing:
    case kPlanRingRs:
      if (nranks < 2) return hxcclInvalidArgument;
      g = plan_ring(amount, nranks, half_bytes, t, kind == kPlanRingRs);
      break;
    default: return hxcclInvalidArgument;
  }
  shape[0] = size_t(g.ctas);
  shape[1] = size_t(g.threads);
  shape[2] = size_t(g.steps);
  shape[3] = size_t(g.epochs);
  shape[4] = g.sub_bytes;
  const std::string bad = check_geometry(kind, g, amount, nranks, half_bytes);
  if (why && why_len) std::snprintf(why, why_len, "%s", bad.c_str());
  return bad.empty() ? hxcclSuccess : hxcclInternalError;
}

int hxcclTestTableRows(void) {
  hx::Tuning t;
  hx::load_default_table(&t);
  return t.rows ? int(t.rows->size()) : 0;
}

hxcclResult_t hxcclTestChooseVariant(size_t bytes, hxcclDataType_t dt, int nranks, int exact, int nvls,
                                     int* variant, int* from_table, size_t shape[3]) {
  using namespace hx;
  if (nranks < 2 || nranks > kMaxRanks || !variant || dtype_size(dt) == 0) return hxcclInvalidArgument;
  Tuning t;
  load_default_table(&t);
  if (const char* path = std::getenv("HXCCL_TUNE_FILE")) {
    std::string bad_line;
    if (!load_tune_file(&t, path, &bad_line)) return hxcclInvalidArgument;
  }
  t.exact = exact != 0;
  t.nvls = nvls != 0;
  OpPlan plan;
  plan.base = hxcclSum;
  const TuneRow* row = nullptr;
  *variant = choose_variant(bytes, dt, plan, nranks, t, kVarAuto, &row);
  if (from_table) *from_table = row ? 1 : 0;
  if (row && (row->variant == kVarTwoShotRoles || row->variant == kVarNvlsRoles)) *variant = row->variant;
  if (shape) {
    const Tuning used = with_row(t, row, *variant);
    shape[0] = size_t(used.max_ctas);
    shape[1] = size_t(used.threads);
    shape[2] = *variant == kVarRing ? used.ring_sub : used.sub_max;
  }
  return hxcclSuccess;
}

}  // extern "C"
