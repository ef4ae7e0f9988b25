// One process drives every rank: HcclCommInitAll creates the communicators of all devices in one call, a thread per rank
// issues the operators, and at the end one thread destroys the handles one after the other.
//                                                                         Run: HCCL_SIM=1 ./a.out 4
// (reference sample: examples/01_communicators/03_one_device_per_pthread/main.cc)
// On GPUs every rank thread calls cudaSetDevice(devices[r]) before it uses its communicator.
#include <numeric>

#include "../common.h"

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    std::vector<int32_t> devices(n);
    std::iota(devices.begin(), devices.end(), 0);
    std::vector<HcclComm> comms(n, nullptr);
    EX_CHECK(HcclCommInitAll(n, devices.data(), comms.data()));

    std::vector<std::thread> ranks;
    for (uint32_t r = 0; r < n; ++r)
        ranks.emplace_back([&, r] {
            uint32_t size = 0, id = 99;
            EX_CHECK(HcclGetRankSize(comms[r], &size));
            EX_CHECK(HcclGetRankId(comms[r], &id));
            EX_EXPECT(size == n && id == r);
            // every rank contributes its number; everybody ends up with the sum and with everybody's number
            std::vector<float> mine(1024, (float)(r + 1)), sum(1024, 0.f), all(1024 * n, 0.f);
            EX_CHECK(HcclAllReduce(mine.data(), sum.data(), 1024, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comms[r], nullptr));
            EX_CHECK(HcclAllGather(mine.data(), all.data(), 1024, HCCL_DATA_TYPE_FP32, comms[r], nullptr));
            EX_EXPECT(sum[0] == (float)(n * (n + 1) / 2) && sum[1023] == sum[0]);
            for (uint32_t q = 0; q < n; ++q) EX_EXPECT(all[q * 1024 + 7] == (float)(q + 1));
        });
    for (auto &t : ranks) t.join();

    // No call waits for ranks that only this thread can bring along: a handle whose peers have not arrived yet is
    // released when the last one of this process is destroyed.
    for (HcclComm c : comms) EX_CHECK(HcclCommDestroy(c));
    std::printf("init_all_one_process: %u ranks ok\n", n);
    return 0;
}
