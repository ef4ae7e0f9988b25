// Scoped NVTX range around one operator call, emitted only while profiling is enabled on the communicator.
// NVTX v3 is header-only: without an attached tool (nsys, ncu, or a library named by NVTX_INJECTION64_PATH) the
// push / pop calls return at once.  The reference reports its operators to msprof through the profiling plugins
// (src/legacy/service/collective/profiling in its tree); on NVIDIA tools the counterpart is a named range per operator.
//
// The header sets its entry points up on the first call of any of them, with plain stores that another thread may
// read at the same moment.  The set-up is therefore forced under a once-flag before the first range: after it the
// entry points no longer change.
#pragma once
#include <nvtx3/nvToolsExt.h>

#include <mutex>

namespace hc {

class NvtxRange {
public:
    NvtxRange(bool enable, const char *name) : on_(enable)
    {
        if (!on_) return;
        static std::once_flag first;
        std::call_once(first, [] { nvtxInitialize(nullptr); });
        nvtxRangePushA(name);
    }
    ~NvtxRange() { if (on_) nvtxRangePop(); }
    NvtxRange(const NvtxRange &) = delete;
    NvtxRange &operator=(const NvtxRange &) = delete;
private:
    bool on_;
};

}  // namespace hc
