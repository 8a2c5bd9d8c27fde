// NVTX ranges around the C-ABI launches, off unless the environment variable LEANFFN_NVTX is set (to anything but
// "0") when the library is first used.  With a profiler attached the ranges name each launch on the timeline; with
// the variable unset the cost is one predictable branch per call.
#pragma once
#include <nvtx3/nvToolsExt.h>

#include <cstdlib>

namespace leanffn {

inline bool nvtx_enabled() {
  static const bool on = []() {
    const char* v = getenv("LEANFFN_NVTX");
    return v != nullptr && v[0] != '\0' && !(v[0] == '0' && v[1] == '\0');
  }();
  return on;
}

struct NvtxRange {
  bool active;
  explicit NvtxRange(const char* name) : active(nvtx_enabled()) {
    if (active) nvtxRangePushA(name);
  }
  ~NvtxRange() {
    if (active) nvtxRangePop();
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace leanffn
