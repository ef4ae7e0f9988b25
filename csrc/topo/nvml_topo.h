// nvml_topo.h - what NVML says about the GPUs of this host: PCI identity, active NVLink links,
// whether they end at an NVSwitch, and the fabric (NVLink domain) identity.
//
// libnvidia-ml.so.1 is opened at run time.  Tests install a fake function table with
// SetNvmlApiForTest so that discovery logic is exercised without a GPU.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "hccl/hccl_types.h"

namespace hc {

struct NvmlPci { char busId[32]; };

// The subset of NVML that discovery needs, as plain function pointers (0 = NVML_SUCCESS).
struct NvmlApi {
    int (*init)();
    int (*deviceGetCount)(unsigned *count);
    int (*deviceGetHandleByIndex)(unsigned idx, void **dev);
    int (*deviceGetPciBusId)(void *dev, NvmlPci *pci);
    int (*deviceGetName)(void *dev, char *name, unsigned len);
    int (*deviceGetUuid)(void *dev, char *uuid, unsigned len);
    int (*nvLinkState)(void *dev, unsigned link, unsigned *active);
    int (*nvLinkRemotePci)(void *dev, unsigned link, NvmlPci *pci);
    // type: 0 GPU, 1 IBM NPU, 2 switch, 255 unknown
    int (*nvLinkRemoteType)(void *dev, unsigned link, unsigned *type);
    // state 3 = completed; clique identifies the NVLink domain partition
    int (*fabricInfo)(void *dev, unsigned *state, unsigned *cliqueId, uint8_t clusterUuid[16]);
};

struct GpuTopoInfo {
    int index = 0;
    std::string busId, name, uuid;
    uint32_t activeLinks = 0;
    uint32_t linksToSwitch = 0;
    std::vector<std::string> peerBusIds;   // remote GPUs reached by direct links
    bool fabricKnown = false;
    uint64_t fabricClique = 0;             // hash(clusterUuid) ^ cliqueId, 0 if unknown
};

constexpr unsigned kMaxNvLinks = 18;       // NVLink 5: 18 links per B200

// Enumerates the GPUs of this host.  HCCL_E_NOT_FOUND when NVML is not installed.
HcclResult ProbeLocalGpus(std::vector<GpuTopoInfo> *out);
void SetNvmlApiForTest(const NvmlApi *api);

}  // namespace hc
