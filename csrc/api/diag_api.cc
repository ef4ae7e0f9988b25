// diag_api.cc - diagnostics (include/hccl/hccl_diag.h): operator record ring, exec counters, the
// device wait-status block, heartbeat view, snapshots of a communicator and process-snapshot hooks.
#include <cstddef>
#include <cstring>
#include <algorithm>
#include <sstream>

#include "../alg/selector.h"
#include "../comm/comm.h"
#include "../core/dtype.h"
#include "../core/log.h"
#include "hccl/hccl_comm.h"
#include "hccl/hccl_diag.h"

using namespace hc;

extern "C" {

HcclResult HcclDiagGetOpRecords(HcclComm comm, HcclOpRecord *records, uint32_t capacity, uint32_t *written)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(records); CHK_PTR_NULL(written);
    std::lock_guard<std::mutex> lk(c->diagMu);
    uint64_t have = std::min<uint64_t>(c->opRingNext, c->opRing.size());
    uint32_t n = (uint32_t)std::min<uint64_t>(have, capacity);
    for (uint32_t i = 0; i < n; ++i) records[i] = c->opRing[(c->opRingNext - n + i) % c->opRing.size()];   // oldest first
    *written = n;
    return HCCL_SUCCESS;
}

HcclResult HcclDiagGetOpCounters(HcclComm comm, uint64_t *launched, uint64_t *headCount, uint64_t *tailCount)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    if (launched) *launched = c->opSeq;
    uint64_t ht[2] = {0, 0};
    if (c->opCounters) CHK_RET(c->plat->PeekSync(ht, c->opCounters, sizeof(ht)));
    if (headCount) *headCount = ht[0];
    if (tailCount) *tailCount = ht[1];
    return HCCL_SUCCESS;
}

HcclResult HcclDiagGetKernelTimes(HcclComm comm, uint64_t *startNs, uint64_t *endNs, uint32_t capacity, uint32_t *written)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(written);
    *written = 0;
    if (!c->devStruct || c->plat->kind() != PlatKind::CUDA) return HCCL_SUCCESS;     // the simulator runs no kernels
    uint64_t ht[2] = {0, 0}, ring[2 * HC_DEV_TIME_SLOTS];
    CHK_RET(c->plat->PeekSync(ht, c->opCounters, sizeof(ht)));
    CHK_RET(c->plat->PeekSync(ring, (char *)c->devStruct + HC_DEV_TIMES_OFFSET, sizeof(ring)));
    // slots are written only while profiling is on: entries without a start time are skipped
    const uint64_t have = std::min<uint64_t>(ht[0], HC_DEV_TIME_SLOTS);
    for (uint64_t k = ht[0] - have; k < ht[0] && *written < capacity; ++k) {
        if (ring[2 * (k % HC_DEV_TIME_SLOTS)] == 0) continue;
        if (startNs) startNs[*written] = ring[2 * (k % HC_DEV_TIME_SLOTS)];
        if (endNs) endNs[*written] = ring[2 * (k % HC_DEV_TIME_SLOTS) + 1];
        ++*written;
    }
    return HCCL_SUCCESS;
}

HcclResult HcclDiagGetWaitStatus(HcclComm comm, HcclDeviceWaitStatus *status)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(status);
    memcpy(status, c->waitStatus, sizeof(*status));
    return HCCL_SUCCESS;
}

HcclResult HcclDiagClearWaitStatus(HcclComm comm)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    memset(c->waitStatus, 0, sizeof(HcclDeviceWaitStatus));
    return HCCL_SUCCESS;
}

HcclResult HcclDiagGetHeartbeat(HcclComm comm, uint64_t *ageMs, uint32_t capacity, uint64_t *lostMask)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    std::vector<uint64_t> ages;
    c->boot->HeartbeatAges(&ages);
    uint64_t worldMask = c->boot->LostMask(), mask = 0;
    for (uint32_t i = 0; i < c->nRanks; ++i) {
        uint32_t w = c->worldRanks[i];
        if (ageMs && i < capacity) ageMs[i] = w < ages.size() ? ages[w] : UINT64_MAX;
        if (worldMask & (1ull << (w & 63))) mask |= 1ull << i;
    }
    if (lostMask) *lostMask = mask;
    return HCCL_SUCCESS;
}

HcclResult HcclDiagPauseHeartbeat(HcclComm comm)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    c->boot->StopHeartbeat();
    return HCCL_SUCCESS;
}

HcclResult HcclDiagSetProfiling(HcclComm comm, int enable)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    c->profiling = enable != 0;
    if (c->devStruct && c->plat->kind() == PlatKind::CUDA) {      // kernels start to time-stamp themselves
        c->hostDev.profile = enable != 0 ? 1u : 0u;
        CHK_RET(c->plat->MemcpySync((char *)c->devStruct + offsetof(CommDev, profile), &c->hostDev.profile, sizeof(uint32_t)));
    }
    return HCCL_SUCCESS;
}

HcclResult HcclDiagDump(HcclComm comm, char *buf, uint32_t bufLen)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(buf);
    std::ostringstream os;
    os << "communicator " << c->cfg.name << " rank " << c->rank << "/" << c->nRanks << " platform " << c->plat->name() << " state " << c->state.load()
       << " asyncError " << c->asyncError.load() << "\n" << c->graph.Describe() << "\n";
    uint64_t ht[2] = {0, 0};
    if (c->opCounters) c->plat->PeekSync(ht, c->opCounters, sizeof(ht));
    os << "operators launched " << c->opSeq << " kernel head " << ht[0] << " tail " << ht[1] << "\n";
    const HcclDeviceWaitStatus &s = *c->waitStatus;
    if (s.valid) os << "expired wait: rank " << s.rank << " on rank " << s.peer << " kind " << s.kind << " slot " << s.slot << " block " << s.block << " expected " << s.expected << " saw " << s.seen << " op #" << s.seq << "\n";
    {
        std::lock_guard<std::mutex> lk(c->diagMu);
        uint64_t have = std::min<uint64_t>(c->opRingNext, 16);
        for (uint64_t i = 0; i < have; ++i) {
            const HcclOpRecord &r = c->opRing[(c->opRingNext - have + i) % c->opRing.size()];
            os << "  #" << r.seq << " " << CmdName((HcclCMDType)r.cmdType) << " " << r.count << " x " << DtypeName((HcclDataType)r.dataType) << " " << r.algName
               << " host " << (r.hostEndNs - r.hostStartNs) / 1000 << " us\n";
        }
    }
    std::string out = os.str();
    snprintf(buf, bufLen, "%s", out.c_str());
    return HCCL_SUCCESS;
}

// ------------------------------------------------------------------------------- snapshots
// Layout: "HCSN" u32 version | u32 rank | u32 nRanks | u64 opCount | u32 nameLen name | u32 algoLen algo |
//         u32 bufferMB | u32 deterministic | u32 expansionMode | i32 execTimeout | u32 tableLen table-stream

static std::vector<uint8_t> BuildSnapshot(Comm *c)
{
    std::vector<uint8_t> b;
    auto p32 = [&](uint32_t v) { b.insert(b.end(), (uint8_t *)&v, (uint8_t *)&v + 4); };
    auto p64 = [&](uint64_t v) { b.insert(b.end(), (uint8_t *)&v, (uint8_t *)&v + 8); };
    auto ps = [&](const std::string &s) { p32((uint32_t)s.size()); b.insert(b.end(), s.begin(), s.end()); };
    p32(0x4e534348); p32(1); p32(c->rank); p32(c->nRanks); p64(c->opSeq); ps(c->cfg.name); ps(c->cfg.algo);
    p32(c->cfg.bufferMB); p32(c->cfg.deterministic); p32(c->cfg.opExpansionMode); p32((uint32_t)c->cfg.execTimeoutSec);
    auto t = c->table.Serialize();
    p32((uint32_t)t.size());
    b.insert(b.end(), t.begin(), t.end());
    return b;
}

HcclResult HcclCommSnapshotSize(HcclComm comm, uint64_t *size)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(size);
    *size = BuildSnapshot(c).size();
    return HCCL_SUCCESS;
}

HcclResult HcclCommSnapshotSave(HcclComm comm, void *buf, uint64_t bufLen, uint64_t *written)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(buf);
    auto b = BuildSnapshot(c);
    if (bufLen < b.size()) return HCCL_E_MEMORY;
    memcpy(buf, b.data(), b.size());
    if (written) *written = b.size();
    return HCCL_SUCCESS;
}

HcclResult HcclCommSnapshotInfo(const void *buf, uint64_t len, uint32_t *rankSize, uint32_t *rank, char *commName, uint64_t *opCount)
{
    CHK_PTR_NULL(buf);
    const uint8_t *p = (const uint8_t *)buf, *e = p + len;
    auto g32 = [&](uint32_t *v) { if (e - p < 4) return false; memcpy(v, p, 4); p += 4; return true; };
    uint32_t magic, ver, r, n, nl;
    uint64_t ops;
    if (!g32(&magic) || magic != 0x4e534348 || !g32(&ver) || ver != 1 || !g32(&r) || !g32(&n)) return HCCL_E_PARA;
    if (e - p < 8) return HCCL_E_PARA;
    memcpy(&ops, p, 8); p += 8;
    if (!g32(&nl) || (uint64_t)(e - p) < nl) return HCCL_E_PARA;
    if (rank) *rank = r;
    if (rankSize) *rankSize = n;
    if (opCount) *opCount = ops;
    if (commName) { size_t k = std::min<size_t>(nl, COMM_NAME_MAX_LENGTH - 1); memcpy(commName, p, k); commName[k] = 0; }
    return HCCL_SUCCESS;
}

// Process-snapshot hooks (reference: framework/cluster_maintenance/snapshot/snapshot_control.h:24-72):
// PRE suspends every communicator, POST resumes them in the same process, RESTORE marks them invalid
// in a restored process image, where device state no longer exists.
HcclResult HcclSnapshotPre(void)
{
    HcclResult first = HCCL_SUCCESS;
    RegistryForEach([&](Comm *c) { HcclResult r = HcclCommSuspend((HcclComm)c); if (r != HCCL_SUCCESS && first == HCCL_SUCCESS) first = r; });
    return first;
}
HcclResult HcclSnapshotPost(void)
{
    // Resume is collective per communicator; every process must call this hook.
    HcclResult first = HCCL_SUCCESS;
    RegistryForEach([&](Comm *c) {
        if (c->state.load() != (int)CommState::SUSPENDED) return;
        HcclResult r = HcclCommResume((HcclComm)c);
        if (r != HCCL_SUCCESS && first == HCCL_SUCCESS) first = r;
    });
    return first;
}
HcclResult HcclSnapshotRestore(void)
{
    RegistryForEach([&](Comm *c) { c->state.store((int)CommState::DESTROYED); });
    return HCCL_SUCCESS;
}

}  // extern "C"
