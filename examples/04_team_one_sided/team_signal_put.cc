// Teams (signals, barrier, windows) and one-sided put / get.
//   * a world team with sync memory; every member registers a window (a piece of its communication buffer),
//     writes into the next member's window through the peer pointer, signals it and waits for its own signal;
//   * the one-sided service: register a region, exchange descriptors with a peer, put a block into it and get it back.
#include <cstring>

#include "../common.h"
#include "hccl/hccl_one_sided.h"
#include "hccl/hccl_res.h"
#include "hccl/hccl_team.h"

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    ExRunRanks(n, [&](uint32_t rank, HcclComm comm) {
        void *buf = nullptr;
        uint64_t size = 0;
        EX_CHECK(HcclGetHcclBuffer(comm, &buf, &size));
        EX_EXPECT(size >= (1u << 16));

        // ---- team with one signal word and one barrier per member
        HcclTeamCreateDesc td;
        EX_CHECK(HcclTeamCreateDescInit(&td));
        td.selfRankId = rank;
        td.requirement.signalCount = 2;
        td.requirement.counterCount = 1;
        td.requirement.barrierCount = 1;
        HcommTeamHandle team = nullptr;
        EX_CHECK(HcclWorldTeamCreate(comm, &td, &team));
        uint32_t members = 0, myIdx = 99;
        EX_CHECK(HcclTeamGetInfo(team, &members, &myIdx));
        EX_EXPECT(members == n && myIdx == rank);

        CommMem mem;
        std::memset(&mem, 0, sizeof(mem));
        mem.type = COMM_MEM_TYPE_DEVICE;
        mem.addr = buf;
        mem.size = 4096;
        HcommWindowHandle win = nullptr;
        EX_CHECK(HcclTeamWindowRegister(comm, team, &mem, &win, 0));
        const uint32_t next = (rank + 1) % n, prev = (rank + n - 1) % n;
        void *nextPtr = nullptr;
        uint64_t nextSize = 0;
        EX_CHECK(HcclTeamWindowGetPeerPointer(team, win, next, &nextPtr, &nextSize));
        EX_EXPECT(nextSize >= 4096);
        for (uint64_t round = 1; round <= 3; ++round) {
            ((volatile uint64_t *)nextPtr)[0] = 1000 * round + rank;          // a store into the neighbour's window
            EX_CHECK(HcclTeamSignal(team, next, 0, 1, nullptr));              // add 1 to the signal word `next` keeps for me
            EX_CHECK(HcclTeamSignalWait(team, prev, 0, round, nullptr));      // the word I keep for `prev` reaches `round`
            EX_EXPECT(((volatile uint64_t *)buf)[0] == 1000 * round + prev);
            EX_CHECK(HcclTeamBarrier(team, 0, nullptr));
        }
        EX_CHECK(HcclTeamWindowDeregister(team, win));
        EX_CHECK(HcclTeamDestroy(team));

        // ---- one-sided put / get with the right neighbour
        char *region = (char *)buf + 8192;
        HcclMemDesc mine, theirs;
        EX_CHECK(HcclRegisterMem(comm, next, 0, region, 4096, &mine));
        HcclMemDescs local{&mine, 1}, remote{&theirs, 1};
        uint32_t got = 0;
        // descriptors travel in both directions of a pair: talk to `next` and `prev` in an order that cannot deadlock
        HcclMemDesc mineForPrev, fromPrev;
        EX_CHECK(HcclRegisterMem(comm, prev, 0, region, 4096, &mineForPrev));
        HcclMemDescs localPrev{&mineForPrev, 1}, remotePrev{&fromPrev, 1};
        if (n == 2) {
            EX_CHECK(HcclExchangeMemDesc(comm, next, &local, 60, &remote, &got));
        } else if (rank % 2 == 0) {
            EX_CHECK(HcclExchangeMemDesc(comm, next, &local, 60, &remote, &got));
            EX_CHECK(HcclExchangeMemDesc(comm, prev, &localPrev, 60, &remotePrev, &got));
        } else {
            EX_CHECK(HcclExchangeMemDesc(comm, prev, &localPrev, 60, &remotePrev, &got));
            EX_CHECK(HcclExchangeMemDesc(comm, next, &local, 60, &remote, &got));
        }
        CommMem remoteMem;
        EX_CHECK(HcclEnableMemAccess(comm, &theirs, &remoteMem));
        std::vector<uint32_t> src(256), back(256, 0);
        for (uint32_t i = 0; i < 256; ++i) src[i] = rank * 1000 + i;
        HcclOneSideOpDesc put{src.data(), remoteMem.addr, 256, HCCL_DATA_TYPE_UINT32};
        EX_CHECK(HcclBatchPut(comm, next, &put, 1, nullptr));
        EX_CHECK(HcclBarrier(comm, nullptr));                                  // all puts have landed
        EX_EXPECT(((uint32_t *)region)[7] == prev * 1000 + 7);                 // what my left neighbour put here
        HcclOneSideOpDesc get{back.data(), remoteMem.addr, 256, HCCL_DATA_TYPE_UINT32};
        EX_CHECK(HcclBatchGet(comm, next, &get, 1, nullptr));
        EX_EXPECT(back[200] == rank * 1000 + 200);
        EX_CHECK(HcclBarrier(comm, nullptr));
        EX_CHECK(HcclDisableMemAccess(comm, &theirs));
        EX_CHECK(HcclDeregisterMem(comm, &mine));
        EX_CHECK(HcclDeregisterMem(comm, &mineForPrev));
    });
    std::printf("team_signal_put: %u ranks ok\n", n);
    return 0;
}
