// Writing a communication operator with the resource and primitive API: every rank sends a block to its right
// neighbour through the communication buffer and reads the block of its left neighbour.
//
//   resources : one thread (a stream with notifies) and one channel per peer with three notifies (ACK, DATA, FIN)
//   send side : copy the payload into the local communication buffer, record DATA on the channel to the right
//   recv side : wait for DATA from the left, read the payload out of the left peer's buffer, record ACK back
//   send side : wait for ACK before the buffer may be reused
// The protocol of a channel is taken from the rank graph (NVLink between GPUs, shared memory on the simulator).
#include <cstring>

#include "../common.h"
#include "hccl/hccl_channel.h"
#include "hccl/hccl_rank_graph.h"
#include "hccl/hccl_res.h"
#include "hcomm_primitives.h"

enum { NOTIFY_ACK = 0, NOTIFY_DATA = 1, NOTIFY_FIN = 2 };

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    const uint64_t bytes = 4096;
    ExRunRanks(n, [&](uint32_t rank, HcclComm comm) {
        const uint32_t right = (rank + 1) % n, left = (rank + n - 1) % n;
        ThreadHandle thread = 0;
        EX_CHECK(HcclThreadAcquire(comm, COMM_ENGINE_CPU_TS, 1, 2, &thread));

        HcclChannelDesc descs[2];
        EX_CHECK(HcclChannelDescInit(descs, 2));
        const uint32_t peers[2] = {right, left};
        for (int i = 0; i < 2; ++i) {
            CommLink *links = nullptr;
            uint32_t linkNum = 0;
            EX_CHECK(HcclRankGraphGetLinks(comm, 0, rank, peers[i], &links, &linkNum));
            EX_EXPECT(linkNum >= 1);
            descs[i].remoteRank = peers[i];
            descs[i].notifyNum = 3;
            descs[i].channelProtocol = links[0].linkAttr.linkProtocol;
        }
        ChannelHandle ch[2] = {0, 0};
        const uint32_t chNum = n == 2 ? 1 : 2;             // with two ranks left and right are the same peer
        EX_CHECK(HcclChannelAcquire(comm, COMM_ENGINE_CPU_TS, descs, chNum, ch));
        ChannelHandle toRight = ch[0], toLeft = chNum == 2 ? ch[1] : ch[0];

        void *localBuf = nullptr, *leftBuf = nullptr;
        uint64_t localSize = 0, leftSize = 0;
        EX_CHECK(HcclGetHcclBuffer(comm, &localBuf, &localSize));
        EX_CHECK(HcclChannelGetHcclBuffer(comm, toLeft, &leftBuf, &leftSize));
        EX_EXPECT(localSize >= bytes && leftSize >= bytes);

        std::vector<uint8_t> payload(bytes), received(bytes, 0);
        for (uint64_t i = 0; i < bytes; ++i) payload[i] = (uint8_t)(rank * 31 + i);

        for (int round = 0; round < 3; ++round) {
            // send to the right
            EX_CHECK(HcommLocalCopyOnThread(thread, localBuf, payload.data(), bytes));
            EX_CHECK(HcommChannelNotifyRecordOnThread(thread, toRight, NOTIFY_DATA));
            // receive from the left
            EX_CHECK(HcommChannelNotifyWaitOnThread(thread, toLeft, NOTIFY_DATA, 1800));
            EX_CHECK(HcommReadOnThread(thread, toLeft, received.data(), leftBuf, bytes));
            EX_CHECK(HcommChannelNotifyRecordOnThread(thread, toLeft, NOTIFY_ACK));
            // my buffer is free again once the right neighbour has read it
            EX_CHECK(HcommChannelNotifyWaitOnThread(thread, toRight, NOTIFY_ACK, 1800));
            EX_CHECK(HcommThreadSynchronize(thread));
            for (uint64_t i = 0; i < bytes; ++i) EX_EXPECT(received[i] == (uint8_t)(left * 31 + i));
            std::memset(received.data(), 0, bytes);
        }
        EX_CHECK(HcclBarrier(comm, nullptr));
        EX_CHECK(HcclChannelDestroy(comm, ch, chNum));
    });
    std::printf("mesh_send_recv: %u ranks ok\n", n);
    return 0;
}
