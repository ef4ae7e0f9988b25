// Scoped NVTX range around one operator call, emitted only while profiling is enabled on the communicator.
// NVTX v3 is header-only: without an attached tool (nsys, ncu, or a library named by NVTX_INJECTION64_PATH) the
// push / pop calls return at once.  The reference reports its operators to msprof through the profiling plugins
// (src/legacy/service/collective/profiling in its tree); on NVIDIA tools the counterpart is a named range per operator.
#pragma once
#include <nvtx3/nvToolsExt.h>

namespace hc {

class NvtxRange {
public:
    NvtxRange(bool enable, const char *name) : on_(enable) { if (on_) nvtxRangePushA(name); }
    ~NvtxRange() { if (on_) nvtxRangePop(); }
    NvtxRange(const NvtxRange &) = delete;
    NvtxRange &operator=(const NvtxRange &) = delete;
private:
    bool on_;
};

}  // namespace hc
