// Optional NVTX ranges around the library's entry points (upstream: PPU_LIB_PERF_INSTRUMENT=1 pushes HGTX
// ranges, csrc/msa_profiling_interface.hpp:289-313).  Off unless MSA_NVTX=1 is set in the environment when the
// library is first called; then every entry point pushes a range named after itself for the duration of the call
// (the launches are asynchronous: the range brackets the enqueue, the kernels carry their own names).
#pragma once

#include <cstdlib>

#include <nvtx3/nvToolsExt.h>

namespace msa {

inline bool nvtx_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("MSA_NVTX");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }();
  return on;
}

struct NvtxRange {
  explicit NvtxRange(const char* name) : active_(nvtx_enabled()) {
    if (active_) nvtxRangePushA(name);
  }
  ~NvtxRange() {
    if (active_) nvtxRangePop();
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;

 private:
  bool active_;
};

}  // namespace msa
