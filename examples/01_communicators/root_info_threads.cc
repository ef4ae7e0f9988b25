// Communicator from a root-info ticket, then AllReduce / AllGather / Broadcast / ReduceScatter.
// The ticket of rank 0 (HcclGetRootInfo) is what an application would broadcast with MPI or a file; here the
// ranks are threads and share it directly.          Build: see tests/test_examples.py.   Run: HCCL_SIM=1 ./a.out 4
#include <cmath>

#include "../common.h"

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    const uint64_t count = 1 << 16;
    ExRunRanks(n, [&](uint32_t rank, HcclComm comm) {
        uint32_t size = 0, id = 99;
        EX_CHECK(HcclGetRankSize(comm, &size));
        EX_CHECK(HcclGetRankId(comm, &id));
        EX_EXPECT(size == n && id == rank);

        std::vector<float> in(count), out(count);
        for (uint64_t i = 0; i < count; ++i) in[i] = (float)(rank + 1) + (float)(i % 7);
        EX_CHECK(HcclAllReduce(in.data(), out.data(), count, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
        for (uint64_t i = 0; i < count; ++i) EX_EXPECT(out[i] == (float)(n * (n + 1) / 2) + (float)n * (float)(i % 7));

        std::vector<int32_t> mine(100, (int32_t)rank), all(100 * n);
        EX_CHECK(HcclAllGather(mine.data(), all.data(), 100, HCCL_DATA_TYPE_INT32, comm, nullptr));
        for (uint32_t q = 0; q < n; ++q) EX_EXPECT(all[q * 100 + 17] == (int32_t)q);

        std::vector<double> b(33, rank == 1 ? 2.5 : 0.0);
        EX_CHECK(HcclBroadcast(b.data(), 33, HCCL_DATA_TYPE_FP64, 1, comm, nullptr));
        EX_EXPECT(b[32] == 2.5);

        std::vector<float> rsIn(64 * n, (float)rank), rsOut(64);
        EX_CHECK(HcclReduceScatter(rsIn.data(), rsOut.data(), 64, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_MAX, comm, nullptr));
        EX_EXPECT(rsOut[5] == (float)(n - 1));
        EX_CHECK(HcclBarrier(comm, nullptr));
    });
    std::printf("root_info_threads: %u ranks ok\n", n);
    return 0;
}
