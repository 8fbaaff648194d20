// NVTX ranges around every entry point of the extension (reference: NVTE_API_CALL,
// common/common.h:1196 and common/nvtx.h).  Off unless TEB200_NVTX=1: the check is one cached bool.
#pragma once
#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <utility>

namespace teb200 {

inline bool nvtx_enabled() {
  static const bool on = []() {
    const char* e = std::getenv("TEB200_NVTX");
    return e != nullptr && std::atoi(e) == 1;
  }();
  return on;
}

// RAII range: pushed in the constructor, popped in the destructor (exceptions included).
struct NvtxRange {
  bool on;
  explicit NvtxRange(const char* name) : on(nvtx_enabled()) {
    if (on) nvtxRangePushA(name);
  }
  ~NvtxRange() {
    if (on) nvtxRangePop();
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

// Wraps a free function so that each call runs inside a range of the given name.
template <typename R, typename... A>
auto traced(const char* name, R (*fn)(A...)) {
  return [name, fn](A... args) -> R {
    NvtxRange range(name);
    return fn(std::forward<A>(args)...);
  };
}

}  // namespace teb200
