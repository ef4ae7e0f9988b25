#include "platform.h"

#include "../core/env.h"
#include "../core/log.h"

namespace hc {

Platform *DefaultPlatform()
{
    int sim = EnvConfig::Get().simulate.value;
    if (sim == 1) return SimInstance();
    Platform *cuda = CudaInstance();
    if (cuda) return cuda;
    if (sim == 0) {
        HCCL_ERROR("HCCL_SIM=0 but no CUDA device is usable");
        return nullptr;
    }
    return SimInstance();
}

}  // namespace hc
