// Host-side messages of sizes the receiver does not know in advance (include/hccl/hccl_msg.h).
// Rank 0 plays a coordinator: every worker reports how much work it has (a message whose length differs per rank), the
// coordinator answers each with a plan.  Receivers probe first, learn source, tag and size from the status, then receive
// into a buffer of that size - MPI's matched probe.  The messages travel over the communicator's control plane, next to
// the collectives; they are meant for control data.                       Run: HCCL_SIM=1 ./a.out 4
#include <unistd.h>

#include <numeric>

#include "../common.h"
#include "hccl/hccl_msg.h"

enum { TAG_REPORT = 1, TAG_PLAN = 2 };

// Waits for a message that matches (source, tag; either may be a wildcard) and receives it.
static std::vector<int32_t> Receive(HcclComm comm, int source, int tag, HcclStatus *status)
{
    int flag = 0;
    HcclMessage msg = nullptr;
    while (!flag) {
        EX_CHECK(HcclImprobe(source, tag, comm, &flag, &msg, status));
        if (!flag) usleep(200);
    }
    int count = 0;
    EX_CHECK(HcclGetCount(status, HCCL_DATA_TYPE_INT32, &count));
    std::vector<int32_t> data((size_t)count);
    HcclRequest req = nullptr;
    EX_CHECK(HcclImrecv(data.data(), count, HCCL_DATA_TYPE_INT32, &msg, &req));
    int done = 0;
    EX_CHECK(HcclTestSome(1, &req, &done, nullptr, nullptr));
    EX_EXPECT(done == 1);
    return data;
}

static void Send(HcclComm comm, int dst, int tag, std::vector<int32_t> &data)
{
    HcclRequest req = nullptr;
    EX_CHECK(HcclIsend(data.data(), (int)data.size(), HCCL_DATA_TYPE_INT32, dst, tag, comm, &req));
    int done = 0;
    EX_CHECK(HcclTestSome(1, &req, &done, nullptr, nullptr));    // a send is complete when it returns
}

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    ExRunRanks(n, [&](uint32_t rank, HcclComm comm) {
        if (rank != 0) {
            std::vector<int32_t> items(rank * 3);              // rank r has 3 r items
            std::iota(items.begin(), items.end(), (int32_t)(rank * 100));
            Send(comm, 0, TAG_REPORT, items);
            HcclStatus st;
            std::vector<int32_t> plan = Receive(comm, 0, TAG_PLAN, &st);
            EX_EXPECT(plan.size() == 2 && plan[0] == (int32_t)rank && plan[1] == (int32_t)(rank * 3));
        } else {
            // reports arrive in any order: take them as they come
            std::vector<int> sizes(n, -1);
            for (uint32_t k = 1; k < n; ++k) {
                HcclStatus st;
                std::vector<int32_t> items = Receive(comm, HCCL_ANY_SOURCE, TAG_REPORT, &st);
                EX_EXPECT(st.srcRank >= 1 && st.srcRank < (int)n && sizes[st.srcRank] == -1);
                EX_EXPECT(items.size() == (size_t)st.srcRank * 3 && (items.empty() || items[0] == st.srcRank * 100));
                sizes[st.srcRank] = (int)items.size();
            }
            for (uint32_t k = 1; k < n; ++k) {
                std::vector<int32_t> plan = {(int32_t)k, (int32_t)sizes[k]};
                Send(comm, (int)k, TAG_PLAN, plan);
            }
        }
        // the collectives run next to the messages
        float one = 1.f, sum = 0.f;
        EX_CHECK(HcclAllReduce(&one, &sum, 1, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
        EX_EXPECT(sum == (float)n);
    });
    std::printf("plan_exchange: %u ranks ok\n", n);
    return 0;
}
