// Profiler ranges around every collective ("hxccl:<op>"), as in the reference
// (src/trace.h:3-9). NVTX 3 is header-only and does nothing until a profiler injects itself,
// so the ranges are always compiled in where the header exists (-DHXCCL_NO_NVTX removes them).
#pragma once
#if !defined(HXCCL_NO_NVTX) && __has_include(<nvtx3/nvToolsExt.h>)
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
