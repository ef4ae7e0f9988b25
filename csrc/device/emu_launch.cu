#include "emu_launch.h"

#include <cuda_runtime.h>

#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "../core/log.h"

namespace hc {
namespace {

constexpr size_t kMaxParamBytes = 4096;

struct EmuGroup {
    std::mutex mu;
    std::condition_variable cv;
    uint32_t n = 0, arrived = 0;
    uint64_t generation = 0;
    std::vector<uint8_t> table;
    std::vector<cudaEvent_t> ready;
    std::vector<int> ids;
    void *devTable = nullptr;
    cudaStream_t launchStream = nullptr;
    cudaEvent_t done = nullptr;
    HcclResult result = HCCL_SUCCESS;
};

std::mutex g_mu;
std::map<std::string, std::shared_ptr<EmuGroup>> g_groups;

std::shared_ptr<EmuGroup> GroupFor(const std::string &key, uint32_t n)
{
    std::lock_guard<std::mutex> lk(g_mu);
    auto &g = g_groups[key];
    if (!g) {
        g = std::make_shared<EmuGroup>();
        g->n = n;
        g->table.resize(kMaxParamBytes * n);
        g->ready.resize(n);
        g->ids.resize(n);
        for (auto &e : g->ready) cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
        cudaEventCreateWithFlags(&g->done, cudaEventDisableTiming);
        cudaStreamCreateWithFlags(&g->launchStream, cudaStreamNonBlocking);
        cudaMalloc(&g->devTable, kMaxParamBytes * n);
    }
    return g;
}

}  // namespace

void EmuForget(const std::string &key)
{
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_groups.find(key);
    if (it == g_groups.end()) return;
    auto g = it->second;
    cudaStreamSynchronize(g->launchStream);
    for (auto &e : g->ready) cudaEventDestroy(e);
    cudaEventDestroy(g->done);
    cudaStreamDestroy(g->launchStream);
    cudaFree(g->devTable);
    g_groups.erase(it);
}

HcclResult EmuLaunchGeneric(const std::string &key, uint32_t nRanks, uint32_t rank, int id, const void *params, size_t paramBytes, void *stream,
                            const std::function<HcclResult(const void *, uint32_t, void *)> &launch)
{
    if (paramBytes > kMaxParamBytes) return HCCL_E_INTERNAL;
    auto g = GroupFor(key, nRanks);
    std::unique_lock<std::mutex> lk(g->mu);
    uint64_t gen = g->generation;
    memcpy(g->table.data() + (size_t)rank * paramBytes, params, paramBytes);
    g->ids[rank] = id;
    cudaEventRecord(g->ready[rank], (cudaStream_t)stream);   // what this rank queued before must finish first
    if (++g->arrived == g->n) {
        HcclResult r = HCCL_SUCCESS;
        for (uint32_t i = 0; i < g->n; ++i) {
            if (g->ids[i] != id) {
                HCCL_ERROR("ranks sharing a GPU issued different operators (%d vs %d)", g->ids[i], id);
                r = HCCL_E_PARA;
            }
            cudaStreamWaitEvent(g->launchStream, g->ready[i], 0);
        }
        if (r == HCCL_SUCCESS) {
            cudaMemcpyAsync(g->devTable, g->table.data(), paramBytes * g->n, cudaMemcpyHostToDevice, g->launchStream);
            r = launch(g->devTable, g->n, g->launchStream);
            // the host table is reused by the next rendezvous and the launch is test-only: finish it here
            cudaError_t e = cudaStreamSynchronize(g->launchStream);
            if (e != cudaSuccess) { HCCL_ERROR("shared-GPU launch failed: %s", cudaGetErrorString(e)); r = HCCL_E_RUNTIME; }
            cudaEventRecord(g->done, g->launchStream);
        }
        g->result = r;
        g->arrived = 0;
        ++g->generation;
        g->cv.notify_all();
    } else {
        g->cv.wait(lk, [&] { return g->generation != gen; });
    }
    HcclResult r = g->result;
    if (r == HCCL_SUCCESS) cudaStreamWaitEvent((cudaStream_t)stream, g->done, 0);
    return r;
}

HcclResult EmuLaunch(const std::string &key, uint32_t nRanks, uint32_t rank, const FastLaunch &l)
{
    FastLaunch copy = l;
    return EmuLaunchGeneric(key, nRanks, rank, l.kind, &l.args, sizeof(CollArgs), l.stream, [copy](const void *devTable, uint32_t n, void *stream) {
        FastLaunch one = copy;
        int limit = FastMaxCoResidentCtas(one.kind, one.threads, (int)n);
        if (limit <= 0) return HCCL_E_INTERNAL;
        if (one.ctas > limit) one.ctas = limit;
        one.stream = stream;
        one.emuTable = (const CollArgs *)devTable;
        one.emuRanks = (int)n;
        return LaunchFastKernel(one);
    });
}

}  // namespace hc
