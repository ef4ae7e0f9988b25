// Going on after ranks were lost.  One process per rank; after the first step the process of rank 0 - the one that hosts
// the rendezvous of the communicator - exits without a word.  The others notice (HcclGetCommAsyncError reports
// HCCL_E_REMOTE), call HcclCommRecover together and continue in a new communicator over themselves, numbered in their
// old order.  Nothing has to be passed around by the application for this: the survivors find each other over the
// ranks' local sockets.                                                   Run: HCCL_SIM=1 ./a.out 4
// A rank leaves between steps only, with none of its operators in flight.
#include <sys/wait.h>
#include <unistd.h>

#include <cstring>
#include <fstream>
#include <string>

#include "../common.h"

static int RankMain(uint32_t rank, uint32_t n, const std::string &ticket)
{
    HcclRootInfo info;
    if (rank == 0) {
        EX_CHECK(HcclGetRootInfo(&info));
        std::ofstream f(ticket + ".tmp", std::ios::binary);
        f.write((const char *)&info, sizeof(info));
        f.close();
        std::rename((ticket + ".tmp").c_str(), ticket.c_str());
    } else {
        for (int tries = 0; tries < 3000 && access(ticket.c_str(), R_OK) != 0; ++tries) usleep(10000);
        std::ifstream f(ticket, std::ios::binary);
        f.read((char *)&info, sizeof(info));
        EX_EXPECT((size_t)f.gcount() == sizeof(info));
    }
    HcclComm comm = nullptr;
    EX_CHECK(HcclCommInitRootInfo(n, &info, rank, &comm));
    std::vector<float> in(1024, (float)(rank + 1)), out(1024, 0.f);
    EX_CHECK(HcclAllReduce(in.data(), out.data(), 1024, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));     // step 1: everybody
    EX_EXPECT(out[0] == (float)(n * (n + 1) / 2));
    if (rank == 0) _exit(0);                               // gone, the communicator's control plane with it

    HcclResult err = HCCL_SUCCESS;
    for (int tries = 0; tries < 2000 && err == HCCL_SUCCESS; ++tries) {
        EX_CHECK(HcclGetCommAsyncError(comm, &err));
        if (err == HCCL_SUCCESS) usleep(10000);
    }
    EX_EXPECT(err == HCCL_E_REMOTE);
    HcclComm fresh = nullptr;
    uint32_t size = 0;
    std::vector<uint32_t> oldRanks(n);
    EX_CHECK(HcclCommRecover(comm, 30, &fresh, &size, oldRanks.data()));
    uint32_t newRank = 99;
    EX_CHECK(HcclGetRankId(fresh, &newRank));
    EX_EXPECT(size == n - 1 && oldRanks[newRank] == rank);
    EX_CHECK(HcclAllReduce(in.data(), out.data(), 1024, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, fresh, nullptr));    // step 2: the survivors
    EX_EXPECT(out[0] == (float)(n * (n + 1) / 2 - 1));
    EX_CHECK(HcclCommDestroy(fresh));
    EX_CHECK(HcclCommDestroy(comm));                       // what is left of the old one
    return 0;
}

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    const std::string ticket = "/tmp/hccl_recovery_ticket_" + std::to_string((long)getpid());
    std::vector<pid_t> kids;
    for (uint32_t r = 0; r < n; ++r) {
        pid_t p = fork();
        if (p == 0) _exit(RankMain(r, n, ticket));
        kids.push_back(p);
    }
    int bad = 0;
    for (pid_t p : kids) {
        int st = 0;
        waitpid(p, &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) ++bad;
    }
    unlink(ticket.c_str());
    if (bad) { std::fprintf(stderr, "%d rank process(es) failed\n", bad); return 1; }
    std::printf("survivors_go_on: %u of %u ranks ok\n", n - 1, n);
    return 0;
}
