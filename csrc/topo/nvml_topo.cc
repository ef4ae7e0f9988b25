#include "nvml_topo.h"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "../core/log.h"

namespace hc {
namespace {

const NvmlApi *g_testApi = nullptr;
NvmlApi g_real{};
bool g_realOk = false;
std::once_flag g_once;
void *g_lib = nullptr;

// Real NVML entry points, looked up by name; signatures restated here so <nvml.h> is not needed
// at run time on machines without the toolkit.
typedef int (*FnVoid)();
typedef int (*FnCount)(unsigned *);
typedef int (*FnHandle)(unsigned, void **);
struct RealPci { char busIdLegacy[16]; unsigned domain, bus, device, pciDeviceId, pciSubSystemId; char busId[32]; };
typedef int (*FnPci)(void *, RealPci *);
typedef int (*FnStr)(void *, char *, unsigned);
typedef int (*FnLinkState)(void *, unsigned, unsigned *);
typedef int (*FnLinkPci)(void *, unsigned, RealPci *);
typedef int (*FnLinkType)(void *, unsigned, unsigned *);
struct RealFabricInfo { uint8_t clusterUuid[16]; int status; unsigned cliqueId; uint8_t state; };
typedef int (*FnFabric)(void *, RealFabricInfo *);

FnVoid r_init; FnCount r_count; FnHandle r_handle; FnPci r_pci; FnStr r_name, r_uuid;
FnLinkState r_lstate; FnLinkPci r_lpci; FnLinkType r_ltype; FnFabric r_fabric;

void LoadReal()
{
    g_lib = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!g_lib) return;
    r_init = (FnVoid)dlsym(g_lib, "nvmlInit_v2");
    r_count = (FnCount)dlsym(g_lib, "nvmlDeviceGetCount_v2");
    r_handle = (FnHandle)dlsym(g_lib, "nvmlDeviceGetHandleByIndex_v2");
    r_pci = (FnPci)dlsym(g_lib, "nvmlDeviceGetPciInfo_v3");
    r_name = (FnStr)dlsym(g_lib, "nvmlDeviceGetName");
    r_uuid = (FnStr)dlsym(g_lib, "nvmlDeviceGetUUID");
    r_lstate = (FnLinkState)dlsym(g_lib, "nvmlDeviceGetNvLinkState");
    r_lpci = (FnLinkPci)dlsym(g_lib, "nvmlDeviceGetNvLinkRemotePciInfo_v2");
    r_ltype = (FnLinkType)dlsym(g_lib, "nvmlDeviceGetNvLinkRemoteDeviceType");
    r_fabric = (FnFabric)dlsym(g_lib, "nvmlDeviceGetGpuFabricInfo");
    if (!r_init || !r_count || !r_handle || !r_pci) return;
    g_real.init = [] { return r_init(); };
    g_real.deviceGetCount = [](unsigned *c) { return r_count(c); };
    g_real.deviceGetHandleByIndex = [](unsigned i, void **d) { return r_handle(i, d); };
    g_real.deviceGetPciBusId = [](void *d, NvmlPci *p) {
        RealPci rp; memset(&rp, 0, sizeof(rp));
        int r = r_pci(d, &rp);
        snprintf(p->busId, sizeof(p->busId), "%s", rp.busId);
        return r;
    };
    g_real.deviceGetName = [](void *d, char *n, unsigned l) { return r_name ? r_name(d, n, l) : 1; };
    g_real.deviceGetUuid = [](void *d, char *n, unsigned l) { return r_uuid ? r_uuid(d, n, l) : 1; };
    g_real.nvLinkState = [](void *d, unsigned l, unsigned *a) { return r_lstate ? r_lstate(d, l, a) : 1; };
    g_real.nvLinkRemotePci = [](void *d, unsigned l, NvmlPci *p) {
        if (!r_lpci) return 1;
        RealPci rp; memset(&rp, 0, sizeof(rp));
        int r = r_lpci(d, l, &rp);
        snprintf(p->busId, sizeof(p->busId), "%s", rp.busId);
        return r;
    };
    g_real.nvLinkRemoteType = [](void *d, unsigned l, unsigned *t) { return r_ltype ? r_ltype(d, l, t) : 1; };
    g_real.fabricInfo = [](void *d, unsigned *state, unsigned *clique, uint8_t uuid[16]) {
        if (!r_fabric) return 1;
        RealFabricInfo fi; memset(&fi, 0, sizeof(fi));
        int r = r_fabric(d, &fi);
        *state = fi.state; *clique = fi.cliqueId; memcpy(uuid, fi.clusterUuid, 16);
        return r;
    };
    g_realOk = true;
}

}  // namespace

void SetNvmlApiForTest(const NvmlApi *api) { g_testApi = api; }

HcclResult ProbeLocalGpus(std::vector<GpuTopoInfo> *out)
{
    out->clear();
    const NvmlApi *api = g_testApi;
    if (!api) {
        std::call_once(g_once, LoadReal);
        if (!g_realOk) return HCCL_E_NOT_FOUND;
        api = &g_real;
    }
    if (api->init() != 0) return HCCL_E_DRV;
    unsigned n = 0;
    if (api->deviceGetCount(&n) != 0) return HCCL_E_DRV;
    for (unsigned i = 0; i < n; ++i) {
        void *dev = nullptr;
        if (api->deviceGetHandleByIndex(i, &dev) != 0) continue;
        GpuTopoInfo g;
        g.index = (int)i;
        NvmlPci pci; memset(&pci, 0, sizeof(pci));
        if (api->deviceGetPciBusId(dev, &pci) == 0) g.busId = pci.busId;
        char buf[96];
        if (api->deviceGetName && api->deviceGetName(dev, buf, sizeof(buf)) == 0) g.name = buf;
        if (api->deviceGetUuid && api->deviceGetUuid(dev, buf, sizeof(buf)) == 0) g.uuid = buf;
        for (unsigned l = 0; l < kMaxNvLinks; ++l) {
            unsigned active = 0;
            if (!api->nvLinkState || api->nvLinkState(dev, l, &active) != 0 || !active) continue;
            ++g.activeLinks;
            unsigned type = 255;
            if (api->nvLinkRemoteType && api->nvLinkRemoteType(dev, l, &type) == 0 && type == 2) { ++g.linksToSwitch; continue; }
            NvmlPci rp; memset(&rp, 0, sizeof(rp));
            if (type == 0 && api->nvLinkRemotePci && api->nvLinkRemotePci(dev, l, &rp) == 0) g.peerBusIds.push_back(rp.busId);
        }
        unsigned state = 0, clique = 0;
        uint8_t uuid[16] = {0};
        if (api->fabricInfo && api->fabricInfo(dev, &state, &clique, uuid) == 0 && state == 3) {
            uint64_t h = 1469598103934665603ull;
            for (int k = 0; k < 16; ++k) h = (h ^ uuid[k]) * 1099511628211ull;
            g.fabricKnown = true;
            g.fabricClique = h ^ clique;
        }
        out->push_back(g);
    }
    return HCCL_SUCCESS;
}

}  // namespace hc
