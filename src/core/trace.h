// Profiler ranges around every collective ("hxccl:<op>"), as in the reference
// (src/trace.h:3-9). NVTX is header-only; without its header the ranges compile away.
#pragma once
#if defined(HXCCL_NVTX) && __has_include(<nvtx3/nvToolsExt.h>)
#include <nvtx3/nvToolsExt.h>
namespace hx {
struct TraceRange {
  explicit TraceRange(const char* name) { nvtxRangePushA(name); }
  ~TraceRange() { nvtxRangePop(); }
};
}  // namespace hx
#else
namespace hx {
struct TraceRange {
  explicit TraceRange(const char*) {}
};
}  // namespace hx
#endif
