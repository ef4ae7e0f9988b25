// One process per rank, communicator from a rank table (cluster description file): every process reads the same JSON
// file and calls HcclCommInitClusterInfo with its own rank; the rendezvous address is derived from the table, nothing
// else has to be exchanged.                                               Run: HCCL_SIM=1 ./a.out 4
// (reference sample: examples/01_communicators/02_one_device_per_process_rank_table/main.cc and its rank_table_v2.json)
#include <sys/wait.h>
#include <unistd.h>

#include <fstream>
#include <sstream>
#include <string>

#include "../common.h"

// A version-2 table for n ranks on one node: one network layer, one fabric instance.
static std::string MakeRankTable(uint32_t n)
{
    std::ostringstream os;
    os << "{\"version\": \"2.0\", \"rank_count\": " << n << ", \"status\": \"completed\", \"rank_list\": [";
    for (uint32_t r = 0; r < n; ++r) {
        os << (r ? ", " : "") << "{\"rank_id\": " << r << ", \"device_id\": " << r << ", \"local_id\": " << r
           << ", \"level_list\": [{\"net_layer\": 0, \"net_instance_id\": \"node0\", \"net_type\": \"TOPO_FILE_DESC\", \"net_attr\": \"\", "
           << "\"rank_addr_list\": [{\"addr_type\": \"IPV4\", \"addr\": \"127.0.0.1\", \"ports\": [\"0/" << r << "\"]}]}]}";
    }
    os << "]}";
    return os.str();
}

static int RankMain(uint32_t rank, uint32_t n, const std::string &table)
{
    HcclComm comm = nullptr;
    EX_CHECK(HcclCommInitClusterInfo(table.c_str(), rank, &comm));
    uint32_t size = 0;
    EX_CHECK(HcclGetRankSize(comm, &size));
    EX_EXPECT(size == n);
    std::vector<int32_t> mine(16, (int32_t)rank), all(16 * n, -1);
    EX_CHECK(HcclAllGather(mine.data(), all.data(), 16, HCCL_DATA_TYPE_INT32, comm, nullptr));
    for (uint32_t q = 0; q < n; ++q) EX_EXPECT(all[q * 16 + 3] == (int32_t)q);
    EX_CHECK(HcclCommDestroy(comm));
    return 0;
}

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    const std::string table = "/tmp/hccl_rank_table_" + std::to_string((long)getpid()) + ".json";
    {
        std::ofstream f(table);
        f << MakeRankTable(n);
    }
    std::vector<pid_t> kids;
    for (uint32_t r = 0; r < n; ++r) {
        pid_t p = fork();
        if (p == 0) _exit(RankMain(r, n, table));
        kids.push_back(p);
    }
    int bad = 0;
    for (pid_t p : kids) {
        int st = 0;
        waitpid(p, &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) ++bad;
    }
    unlink(table.c_str());
    if (bad) { std::fprintf(stderr, "%d rank process(es) failed\n", bad); return 1; }
    std::printf("rank_table_processes: %u ranks ok\n", n);
    return 0;
}
