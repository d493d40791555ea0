// Trace zones of the provider adapter, gated at compile time like the reference's HYLE_TRACE_* hooks
// (include/hyle/obs/trace.h:1-22: the OFF form evaluates nothing and includes no backend; zones
// "hyle.compute.prepare" / "hyle.compute.submit", src/compute/operation.cc:1211,1882).  The reference
// fills its macros with Tracy; on a CUDA machine the profilers read NVTX, so a build with
// -DHYLE_B200_NVTX turns every zone into an NVTX range (NVTX 3 is header-only: nothing is linked,
// the ranges cost one indirect call while no tool is attached).  Zones: "hyle_b200.propose",
// "hyle_b200.prepare", and around the enqueue of each operator "hyle_b200.enqueue.<entry>", which
// encloses the gathers, the workspace clear and the kernel launch that one submit records.
#pragma once

#if defined(HYLE_B200_NVTX)
#include <nvtx3/nvToolsExt.h>

namespace hyle::compute::b200 {
struct TraceZone final {
  explicit TraceZone(const char *name) noexcept { nvtxRangePushA(name); }
  TraceZone(const TraceZone &) = delete;
  TraceZone &operator=(const TraceZone &) = delete;
  ~TraceZone() { nvtxRangePop(); }
};
}  // namespace hyle::compute::b200
#define HYLE_B200_TRACE_JOIN2(a, b) a##b
#define HYLE_B200_TRACE_JOIN(a, b) HYLE_B200_TRACE_JOIN2(a, b)
#define HYLE_B200_TRACE_ZONE(name) \
  const ::hyle::compute::b200::TraceZone HYLE_B200_TRACE_JOIN(hyle_b200_trace_zone_, __LINE__) { name }
#else
#define HYLE_B200_TRACE_ZONE(name) static_cast<void>(0)
#endif
