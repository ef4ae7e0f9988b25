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

struct EmuGroup {
    std::mutex mu;
    std::condition_variable cv;
    uint32_t n = 0, arrived = 0;
    uint64_t generation = 0;
    std::vector<CollArgs> table;
    std::vector<cudaEvent_t> ready;
    std::vector<int32_t> kinds;
    CollArgs *devTable = nullptr;
    cudaStream_t launchStream = nullptr;
    cudaEvent_t done = nullptr;
    HcclResult result = HCCL_SUCCESS;
    int ctas = 0, threads = 0;
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
        g->table.resize(n);
        g->ready.resize(n);
        g->kinds.resize(n);
        for (auto &e : g->ready) cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
        cudaEventCreateWithFlags(&g->done, cudaEventDisableTiming);
        cudaStreamCreateWithFlags(&g->launchStream, cudaStreamNonBlocking);
        cudaMalloc(&g->devTable, sizeof(CollArgs) * n);
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

HcclResult EmuLaunch(const std::string &key, uint32_t nRanks, uint32_t rank, const FastLaunch &l)
{
    auto g = GroupFor(key, nRanks);
    std::unique_lock<std::mutex> lk(g->mu);
    uint64_t gen = g->generation;
    g->table[rank] = l.args;
    g->kinds[rank] = l.kind;
    g->ctas = l.ctas;
    g->threads = l.threads;
    // what this rank queued before the collective must finish first
    cudaEventRecord(g->ready[rank], (cudaStream_t)l.stream);
    if (++g->arrived == g->n) {
        HcclResult r = HCCL_SUCCESS;
        for (uint32_t i = 0; i < g->n; ++i) {
            if (g->kinds[i] != l.kind) {
                HCCL_ERROR("ranks sharing a GPU issued different kernels (%s vs %s)", FastKindName(g->kinds[i]), FastKindName(l.kind));
                r = HCCL_E_PARA;
            }
            cudaStreamWaitEvent(g->launchStream, g->ready[i], 0);
        }
        if (r == HCCL_SUCCESS) {
            int limit = FastMaxCoResidentCtas(l.kind, g->threads, (int)g->n);
            if (limit <= 0) r = HCCL_E_INTERNAL;
            else if (g->ctas > limit) g->ctas = limit;
        }
        if (r == HCCL_SUCCESS) {
            cudaMemcpyAsync(g->devTable, g->table.data(), sizeof(CollArgs) * g->n, cudaMemcpyHostToDevice, g->launchStream);
            FastLaunch one = l;
            one.ctas = g->ctas;
            one.stream = g->launchStream;
            one.emuTable = g->devTable;
            one.emuRanks = (int)g->n;
            r = LaunchFastKernel(one);
            // the table is read at kernel start only, but the host vector is reused by the next call
            cudaStreamSynchronize(g->launchStream);
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
    if (r == HCCL_SUCCESS) cudaStreamWaitEvent((cudaStream_t)l.stream, g->done, 0);
    return r;
}

}  // namespace hc
