// One process per rank, communicator from a root-info ticket: rank 0 creates the ticket (HcclGetRootInfo) and hands it
// to the other processes - an application would broadcast it with MPI, through a key-value store or, as here, a file.
// The parent forks the rank processes and collects their exit codes.     Run: HCCL_SIM=1 ./a.out 4
// (reference sample: examples/01_communicators/01_one_device_per_process/main.cc)
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
    // on GPUs: cudaSetDevice(rank) goes here, before the communicator is created
    HcclComm comm = nullptr;
    EX_CHECK(HcclCommInitRootInfo(n, &info, rank, &comm));
    const uint64_t count = 4096;
    std::vector<float> in(count, (float)(rank + 1)), out(count, 0.f);
    EX_CHECK(HcclAllReduce(in.data(), out.data(), count, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    for (uint64_t i = 0; i < count; ++i) EX_EXPECT(out[i] == (float)(n * (n + 1) / 2));
    EX_CHECK(HcclBarrier(comm, nullptr));
    EX_CHECK(HcclCommDestroy(comm));
    return 0;
}

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    const std::string ticket = "/tmp/hccl_root_info_" + std::to_string((long)getpid());
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
    std::printf("root_info_processes: %u ranks ok\n", n);
    return 0;
}
