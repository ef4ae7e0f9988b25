// team_api.cc - SHMEM-style teams (include/hccl/hccl_team.h; reference: src/coll_communicator_mgr/team).
//
// A team reserves, on every member, a block of 64-bit words inside the symmetric flag page:
//   for each member m of the team:  signal[signalCount] | counter[counterCount] | barrier[barrierCount]
// Member i signals member j by adding to j's words in row i, so every word has one writer.  The
// handle given to the caller is the address of a record {magic, rankNum, myIndex, counts, words per
// row, heap offset of the block, then for each member the address of ITS block as mapped here} that
// device code of the SM engine can read directly.
#include <cstring>
#include <map>

#include "../comm/comm.h"
#include "../core/log.h"
#include "hccl/hccl_comm.h"
#include "hccl/hccl_sym_win.h"
#include "hccl/hccl_team.h"

using namespace hc;

namespace {

constexpr uint64_t kTeamMagic = 0x4d414554434c4348ull;   // "HCLCTEAM"
enum { T_MAGIC = 0, T_RANKS, T_MYIDX, T_SIGNALS, T_COUNTERS, T_BARRIERS, T_ROWWORDS, T_OFFSET, T_HEADER };

struct Team {
    Comm *comm = nullptr;
    Team *world = nullptr;
    std::vector<uint32_t> members;        // ranks of the communicator
    uint32_t myIndex = 0;
    HcommTeamSyncMemRequirement req{};
    uint32_t rowWords = 0;
    uint64_t heapOffset = 0;
    uint64_t *record = nullptr;           // host-visible record handed out as the handle
    void *devRecord = nullptr;
    std::vector<uint64_t> barrierWaited;  // per barrier index: rounds completed
    std::vector<uint64_t> signalSent;
    Bootstrap::Group group;
    std::vector<HcclCommSymWindow> windows;
};

std::mutex g_mu;
std::map<uint64_t *, std::unique_ptr<Team>> g_teams;

Team *AsTeam(HcommTeamHandle h)
{
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_teams.find(h);
    return it == g_teams.end() ? nullptr : it->second.get();
}

uint64_t *Word(Team *t, uint32_t owner, uint32_t row, uint32_t idx)
{
    Comm *c = t->comm;
    return (uint64_t *)(c->PeerHeap(t->members[owner]) + HC_OFF_TEAM_SYNC + t->heapOffset) + (uint64_t)row * t->rowWords + idx;
}

HcclResult Build(Comm *c, Team *world, const HcclTeamCreateDesc *desc, HcommTeamHandle *out)
{
    if (desc->header.magicWord != HCCL_TEAM_CREATE_DESC_MAGIC_WORD) { RPT_ERR("EI0003", "HcclTeamCreateDesc was not initialised with HcclTeamCreateDescInit"); return HCCL_E_PARA; }
    std::unique_ptr<Team> t(new Team());
    t->comm = c;
    t->world = world;
    if (desc->rankIds && desc->rankNum) t->members.assign(desc->rankIds, desc->rankIds + desc->rankNum);
    else for (uint32_t i = 0; i < c->nRanks; ++i) t->members.push_back(i);
    t->myIndex = ~0u;
    for (uint32_t i = 0; i < t->members.size(); ++i) {
        if (t->members[i] >= c->nRanks) return HCCL_E_PARA;
        if (t->members[i] == c->rank) t->myIndex = i;
    }
    if (t->myIndex == ~0u) { RPT_ERR("EI0003", "rank %u is not a member of the team it creates", c->rank); return HCCL_E_PARA; }
    t->req = desc->requirement;
    t->rowWords = desc->requirement.signalCount + desc->requirement.counterCount + desc->requirement.barrierCount;
    if (t->rowWords == 0) t->rowWords = 1;
    uint64_t bytes = ((uint64_t)t->rowWords * t->members.size() * 8 + 255) & ~255ull;
    // Members agree on the offset: the largest "used" mark among them (sub teams are created by members only).
    std::vector<uint32_t> world32;
    for (uint32_t m : t->members) world32.push_back(c->worldRanks[m]);
    uint32_t gid = Crc32(world32.data(), world32.size() * 4, 0x7ea30000u ^ c->group.id);
    t->group = c->boot->MakeGroup(gid ? gid : 1, world32);
    Blob mine((uint8_t *)&c->teamSyncUsed, (uint8_t *)&c->teamSyncUsed + 8);
    std::vector<Blob> all;
    CHK_RET(c->boot->AllGather(t->group, mine, &all));
    uint64_t off = 0;
    for (auto &b : all) { uint64_t v = 0; if (b.size() == 8) memcpy(&v, b.data(), 8); off = std::max(off, v); }
    if (off + bytes > (1ull << 20)) { RPT_ERR("EI0003", "team synchronisation memory exhausted (1 MB per rank)"); return HCCL_E_UNAVAIL; }
    t->heapOffset = off;
    c->teamSyncUsed = off + bytes;
    CHK_RET(c->plat->MemsetSync(c->LocalHeap() + HC_OFF_TEAM_SYNC + off, 0, bytes));
    t->barrierWaited.assign(std::max<uint32_t>(1, t->req.barrierCount), 0);
    size_t words = T_HEADER + t->members.size() * 2;
    void *rec = nullptr;
    CHK_RET(c->plat->HostAlloc(words * 8, &rec));
    t->record = (uint64_t *)rec;
    t->record[T_MAGIC] = kTeamMagic; t->record[T_RANKS] = t->members.size(); t->record[T_MYIDX] = t->myIndex;
    t->record[T_SIGNALS] = t->req.signalCount; t->record[T_COUNTERS] = t->req.counterCount; t->record[T_BARRIERS] = t->req.barrierCount;
    t->record[T_ROWWORDS] = t->rowWords; t->record[T_OFFSET] = HC_OFF_TEAM_SYNC + off;
    for (size_t i = 0; i < t->members.size(); ++i) {
        t->record[T_HEADER + i] = (uint64_t)(uintptr_t)(c->PeerHeap(t->members[i]) + HC_OFF_TEAM_SYNC + off);
        t->record[T_HEADER + t->members.size() + i] = t->members[i];
    }
    CHK_RET(c->boot->Barrier(t->group));   // all blocks cleared before anyone signals
    *out = t->record;
    std::lock_guard<std::mutex> lk(g_mu);
    g_teams[t->record] = std::move(t);
    return HCCL_SUCCESS;
}

}  // namespace

extern "C" {

HcclResult HcclWorldTeamCreate(HcclComm comm, const HcclTeamCreateDesc *desc, HcommTeamHandle *worldTeam)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(desc); CHK_PTR_NULL(worldTeam);
    return Build(c, nullptr, desc, worldTeam);
}

HcclResult HcclSubTeamCreate(HcommTeamHandle worldTeam, const HcclTeamCreateDesc *desc, HcommTeamHandle *team)
{
    Team *w = AsTeam(worldTeam);
    CHK_PTR_NULL(w); CHK_PTR_NULL(desc); CHK_PTR_NULL(team);
    if (!desc->rankIds || !desc->rankNum) return HCCL_E_PARA;
    for (uint32_t i = 0; i < desc->rankNum; ++i)
        if (std::find(w->members.begin(), w->members.end(), desc->rankIds[i]) == w->members.end()) { RPT_ERR("EI0003", "rank %u is not in the world team", desc->rankIds[i]); return HCCL_E_PARA; }
    return Build(w->comm, w, desc, team);
}

HcclResult HcclTeamDestroy(HcommTeamHandle team)
{
    Team *t = AsTeam(team);
    CHK_PTR_NULL(t);
    t->comm->plat->HostFree(t->record);
    std::lock_guard<std::mutex> lk(g_mu);
    g_teams.erase(team);
    return HCCL_SUCCESS;
}

HcclResult HcclTeamWindowRegister(HcclComm comm, HcommTeamHandle worldTeam, const CommMem *localMem, HcommWindowHandle *window, uint32_t flag)
{
    Team *t = AsTeam(worldTeam);
    CHK_PTR_NULL(t); CHK_PTR_NULL(localMem); CHK_PTR_NULL(window);
    if (t->members.size() != t->comm->nRanks) { RPT_ERR("EI0003", "windows are registered on a team that spans the communicator"); return HCCL_E_NOT_SUPPORT; }
    HcclCommSymWindow w;
    CHK_RET(HcclCommSymWinRegister(comm, localMem->addr, localMem->size, &w, flag));
    t->windows.push_back(w);
    *window = (HcommWindowHandle)w;
    return HCCL_SUCCESS;
}

HcclResult HcclTeamWindowDeregister(HcommTeamHandle worldTeam, HcommWindowHandle window)
{
    Team *t = AsTeam(worldTeam);
    CHK_PTR_NULL(t); CHK_PTR_NULL(window);
    auto it = std::find(t->windows.begin(), t->windows.end(), (HcclCommSymWindow)window);
    if (it == t->windows.end()) return HCCL_E_NOT_FOUND;
    t->windows.erase(it);
    return HcclCommSymWinDeregister((HcclCommSymWindow)window);
}

// Every pair of members already shares the symmetric heap; creating channels means acquiring the
// communicator channels so that the primitives API can be used between team members.
HcclResult HcclTeamChannelsCreate(HcclComm comm, HcommTeamHandle team, const HcclTeamCreateChannelsDesc *desc)
{
    Team *t = AsTeam(team);
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(t); CHK_PTR_NULL(c); CHK_PTR_NULL(desc);
    if (desc->header.magicWord != HCCL_TEAM_CREATE_CHANNELS_DESC_MAGIC_WORD) return HCCL_E_PARA;
    // Pair handshakes are ordered by (lower rank, higher rank) on both sides so that they cannot cross.
    for (uint32_t m : t->members) {
        if (m == c->rank) continue;
        HcclChannelDesc d;
        HcclChannelDescInit(&d, 1);
        d.remoteRank = m;
        d.notifyNum = desc->notifyNum;
        ChannelHandle h;
        CHK_RET(HcclChannelAcquire(comm, desc->engine == COMM_ENGINE_RESERVED ? COMM_ENGINE_CPU_TS : desc->engine, &d, 1, &h));
    }
    return HCCL_SUCCESS;
}

HcclResult HcclTeamGetInfo(HcommTeamHandle team, uint32_t *rankNum, uint32_t *myIndex)
{
    Team *t = AsTeam(team);
    CHK_PTR_NULL(t);
    if (rankNum) *rankNum = (uint32_t)t->members.size();
    if (myIndex) *myIndex = t->myIndex;
    return HCCL_SUCCESS;
}

HcclResult HcclTeamWindowGetPeerPointer(HcommTeamHandle team, HcommWindowHandle window, uint32_t memberIdx, void **ptr, uint64_t *size)
{
    Team *t = AsTeam(team);
    CHK_PTR_NULL(t); CHK_PTR_NULL(window); CHK_PTR_NULL(ptr);
    if (memberIdx >= t->members.size()) return HCCL_E_PARA;
    Window *w = (Window *)window;
    if (size) *size = w->size;
    return HcclSymWinGetPeerPointer((HcclCommSymWindow)window, 0, t->members[memberIdx], ptr);
}

// Adds `value` to signal word `signalIdx` that member `memberIdx` keeps for the caller.
HcclResult HcclTeamSignal(HcommTeamHandle team, uint32_t memberIdx, uint32_t signalIdx, uint64_t value, aclrtStream stream)
{
    Team *t = AsTeam(team);
    CHK_PTR_NULL(t);
    if (memberIdx >= t->members.size() || signalIdx >= t->req.signalCount) return HCCL_E_PARA;
    Stream s = t->comm->plat->kind() == PlatKind::SIM ? nullptr : stream;
    return t->comm->plat->FlagAddAsync(Word(t, memberIdx, t->myIndex, signalIdx), value, s);
}

// Waits until the signal word that member `memberIdx` writes here has reached `value`.
HcclResult HcclTeamSignalWait(HcommTeamHandle team, uint32_t memberIdx, uint32_t signalIdx, uint64_t value, aclrtStream stream)
{
    Team *t = AsTeam(team);
    CHK_PTR_NULL(t);
    if (memberIdx >= t->members.size() || signalIdx >= t->req.signalCount) return HCCL_E_PARA;
    Comm *c = t->comm;
    Stream s = c->plat->kind() == PlatKind::SIM ? nullptr : stream;
    WaitReport rep;
    rep.status = c->waitStatus; rep.abortWord = c->abortWord; rep.rank = c->rank; rep.peer = t->members[memberIdx]; rep.kind = HC_WAIT_CHAN_NOTIFY; rep.slot = signalIdx;
    CHK_RET(c->plat->FlagWaitGeAsync(Word(t, t->myIndex, memberIdx, signalIdx), value, c->TimeoutMs(), rep, s));
    return c->plat->kind() == PlatKind::SIM ? CommPollDeviceStatus(c) : HCCL_SUCCESS;
}

HcclResult HcclTeamBarrier(HcommTeamHandle team, uint32_t barrierIdx, aclrtStream stream)
{
    Team *t = AsTeam(team);
    CHK_PTR_NULL(t);
    if (barrierIdx >= std::max<uint32_t>(1, t->req.barrierCount) || t->req.barrierCount == 0) return HCCL_E_PARA;
    Comm *c = t->comm;
    Stream s = c->plat->kind() == PlatKind::SIM ? nullptr : stream;
    uint32_t col = t->req.signalCount + t->req.counterCount + barrierIdx;
    uint64_t round = ++t->barrierWaited[barrierIdx];
    for (uint32_t m = 0; m < t->members.size(); ++m)
        if (m != t->myIndex) CHK_RET(c->plat->FlagAddAsync(Word(t, m, t->myIndex, col), 1, s));
    for (uint32_t m = 0; m < t->members.size(); ++m) {
        if (m == t->myIndex) continue;
        WaitReport rep;
        rep.status = c->waitStatus; rep.abortWord = c->abortWord; rep.rank = c->rank; rep.peer = t->members[m]; rep.kind = HC_WAIT_BARRIER; rep.slot = barrierIdx;
        CHK_RET(c->plat->FlagWaitGeAsync(Word(t, t->myIndex, m, col), round, c->TimeoutMs(), rep, s));
    }
    return c->plat->kind() == PlatKind::SIM ? CommPollDeviceStatus(c) : HCCL_SUCCESS;
}

}  // extern "C"
