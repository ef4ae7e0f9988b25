// A reduce-scatter written with the data-plane primitives, exercising the rest of the resource API:
//   * registered memory with a tag, visible to the peers through HcclChannelGetRemoteMems;
//   * an engine context (a tagged blob the operator keeps between calls);
//   * write-with-notify, read-reduce and local-reduce primitives, a batch of transfers, a channel fence;
//   * batch mode and the task cache: the operator's task list is recorded once and replayed on new buffers.
// Every rank owns one block of the result: it adds up that block of everybody's input.
#include <algorithm>
#include <cstring>
#include <string>

#include "../common.h"
#include "hccl/hccl_channel.h"
#include "hccl/hccl_res.h"
#include "hcomm_primitives.h"

struct OpCtx { uint32_t calls; uint32_t peers; };

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    const uint64_t block = 1024;                       // floats per block
    ExRunRanks(n, [&](uint32_t rank, HcclComm comm) {
        // ---- resources
        ThreadHandle thread = 0;
        EX_CHECK(HcclThreadAcquire(comm, COMM_ENGINE_CPU_TS, 1, 1, &thread));
        void *ccl = nullptr;
        uint64_t cclSize = 0;
        EX_CHECK(HcclGetHcclBuffer(comm, &ccl, &cclSize));
        EX_EXPECT(cclSize >= n * block * sizeof(float) * 2);
        // a tagged region inside the communication buffer: peers find it by its tag
        CommMem mem;
        std::memset(&mem, 0, sizeof(mem));
        mem.type = COMM_MEM_TYPE_DEVICE;
        mem.addr = (char *)ccl + (1 << 20);
        mem.size = n * block * sizeof(float);
        HcclMemHandle memHandle = nullptr;
        EX_CHECK(HcclCommMemReg(comm, "rs_staging", &mem, &memHandle));
        EX_CHECK(HcclBarrier(comm, nullptr));          // everybody has registered before channels exchange the lists

        std::vector<HcclChannelDesc> descs(n - 1);
        EX_CHECK(HcclChannelDescInit(descs.data(), n - 1));
        std::vector<uint32_t> peers;
        for (uint32_t i = 1; i < n; ++i) peers.push_back((rank + i) % n);
        // both ends of a pair must create their channels in the same order: sort by peer rank
        std::sort(peers.begin(), peers.end());
        for (uint32_t i = 0; i < n - 1; ++i) { descs[i].remoteRank = peers[i]; descs[i].notifyNum = 2; }
        std::vector<ChannelHandle> ch(n - 1);
        EX_CHECK(HcclChannelAcquire(comm, COMM_ENGINE_CPU_TS, descs.data(), n - 1, ch.data()));
        std::vector<float *> peerStaging(n - 1);
        for (uint32_t i = 0; i < n - 1; ++i) {
            uint32_t memNum = 0;
            CommMem *mems = nullptr;
            char **tags = nullptr;
            EX_CHECK(HcclChannelGetRemoteMems(comm, ch[i], &memNum, &mems, &tags));
            peerStaging[i] = nullptr;
            for (uint32_t k = 0; k < memNum; ++k)
                if (std::string(tags[k]) == "rs_staging") peerStaging[i] = (float *)mems[k].addr;
            EX_EXPECT(peerStaging[i] != nullptr);
        }
        // ---- engine context: survives between calls of the operator
        void *ctxPtr = nullptr;
        EX_CHECK(HcclEngineCtxCreate(comm, "rs_prims", COMM_ENGINE_CPU_TS, sizeof(OpCtx), &ctxPtr));
        OpCtx init{0, n - 1};
        EX_CHECK(HcclEngineCtxCopy(comm, COMM_ENGINE_CPU_TS, "rs_prims", &init, sizeof(init), 0));

        float *staging = (float *)mem.addr;
        std::vector<float> in(n * block), out(block);
        for (int call = 0; call < 3; ++call) {
            for (uint64_t i = 0; i < n * block; ++i) in[i] = (float)(rank + 1) * (float)(call + 1) + (float)(i % 5);
            void *ctxAgain = nullptr;
            uint64_t ctxSize = 0;
            EX_CHECK(HcclEngineCtxGet(comm, "rs_prims", COMM_ENGINE_CPU_TS, &ctxAgain, &ctxSize));
            EX_EXPECT(ctxAgain == ctxPtr && ctxSize == sizeof(OpCtx) && ((OpCtx *)ctxAgain)->peers == n - 1);
            ((OpCtx *)ctxAgain)->calls++;

            // my copy of block q goes into slot `rank` of peer q's staging, with a notify
            for (uint32_t i = 0; i < n - 1; ++i) {
                const uint32_t q = peers[i];
                EX_CHECK(HcommWriteWithNotifyOnThread(thread, ch[i], peerStaging[i] + rank * block, in.data() + q * block, block * sizeof(float), 0));
            }
            // start from my own contribution, add what the peers wrote
            EX_CHECK(HcommLocalCopyOnThread(thread, out.data(), in.data() + rank * block, block * sizeof(float)));
            for (uint32_t i = 0; i < n - 1; ++i) {
                EX_CHECK(HcommChannelNotifyWaitOnThread(thread, ch[i], 0, 1800));
                EX_CHECK(HcommLocalReduceOnThread(thread, out.data(), staging + peers[i] * block, block, HCOMM_DATA_TYPE_FP32, HCOMM_REDUCE_SUM));
            }
            // tell the writers that their slot may be reused, and wait for the same from my readers
            for (uint32_t i = 0; i < n - 1; ++i) EX_CHECK(HcommChannelNotifyRecordOnThread(thread, ch[i], 1));
            for (uint32_t i = 0; i < n - 1; ++i) EX_CHECK(HcommChannelNotifyWaitOnThread(thread, ch[i], 1, 1800));
            EX_CHECK(HcommThreadSynchronize(thread));
            for (uint64_t i = 0; i < block; ++i) {
                const float want = (float)(n * (n + 1) / 2) * (float)(call + 1) + (float)n * (float)((rank * block + i) % 5);
                EX_EXPECT(out[i] == want);
            }
        }
        EX_EXPECT(((OpCtx *)ctxPtr)->calls == 3);

        // ---- a batch of transfers (read my block from a peer's input copy in its staging, reduce on the way) and a fence
        if (n >= 2) {
            // everybody parks block `rank` of its input in its own staging slot n-1 ... reuse slot `rank`
            std::memcpy(staging + rank * block, in.data() + rank * block, block * sizeof(float));
            // The staging lives in the communication buffer, which the library's own operators (HcclBarrier among them)
            // use as well: while it holds data, the ranks synchronise through the channels' notifies instead.
            auto syncPeers = [&]() {
                for (uint32_t i = 0; i < n - 1; ++i) EX_CHECK(HcommChannelNotifyRecordOnThread(thread, ch[i], 1));
                for (uint32_t i = 0; i < n - 1; ++i) EX_CHECK(HcommChannelNotifyWaitOnThread(thread, ch[i], 1, 1800));
                EX_CHECK(HcommThreadSynchronize(thread));
            };
            syncPeers();
            std::vector<float> acc(block, 0.0f);
            HcommBatchTransferDesc bt[2];
            std::memset(bt, 0, sizeof(bt));
            bt[0].transType = HCOMM_TRANSFER_TYPE_READ;
            bt[0].transferInfo.read.len = block * sizeof(float);
            bt[0].transferInfo.read.dst = acc.data();
            bt[0].transferInfo.read.src = peerStaging[0] + peers[0] * block;
            bt[1].transType = HCOMM_TRANSFER_TYPE_READ_REDUCE;
            bt[1].transferInfo.reduce.count = block;
            bt[1].transferInfo.reduce.dst = acc.data();
            bt[1].transferInfo.reduce.src = peerStaging[0] + peers[0] * block;
            bt[1].transferInfo.reduce.reduceOp = HCOMM_REDUCE_SUM;
            bt[1].transferInfo.reduce.dataType = HCOMM_DATA_TYPE_FP32;
            EX_CHECK(HcommBatchTransferOnThread(thread, ch[0], bt, 2));
            EX_CHECK(HcommChannelFenceOnThread(thread, ch[0]));
            EX_CHECK(HcommThreadSynchronize(thread));
            const uint32_t q = peers[0];
            for (uint64_t i = 0; i < block; ++i) EX_EXPECT(acc[i] == 2.0f * ((float)(q + 1) * 3.0f + (float)((q * block + i) % 5)));
            syncPeers();
        }

        // ---- batch mode + task cache: record a local copy chain once, replay it on other buffers
        std::vector<float> a1(256, 1.5f), b1(256, 0.0f), a2(256, 7.0f), b2(256, 0.0f);
        const std::string tag = "copy_chain_" + std::to_string(rank);
        bool hit = true;
        EX_CHECK(HcommAicpuTsTaskCacheLookup(tag.c_str(), &hit));
        EX_EXPECT(!hit);
        void *addrs1[2] = {a1.data(), b1.data()};
        uint64_t sizes[2] = {256 * sizeof(float), 256 * sizeof(float)};
        EX_CHECK(HcommAicpuTsTaskCacheStart(tag.c_str(), addrs1, sizes, 2));
        EX_CHECK(HcommBatchModeStart(tag.c_str()));
        EX_CHECK(HcommLocalCopyOnThread(thread, b1.data(), a1.data(), 128 * sizeof(float)));
        EX_CHECK(HcommLocalCopyOnThread(thread, b1.data() + 128, a1.data() + 128, 128 * sizeof(float)));
        EX_CHECK(HcommBatchModeEnd(tag.c_str()));
        EX_CHECK(HcommAicpuTsTaskCacheEnd(tag.c_str()));
        EX_CHECK(HcommThreadSynchronize(thread));
        EX_EXPECT(b1[0] == 1.5f && b1[255] == 1.5f);
        EX_CHECK(HcommAicpuTsTaskCacheLookup(tag.c_str(), &hit));
        EX_EXPECT(hit);
        void *addrs2[2] = {a2.data(), b2.data()};
        EX_CHECK(HcommAicpuTsTaskCacheExecute(tag.c_str(), addrs2, sizes, 2));
        EX_CHECK(HcommThreadSynchronize(thread));
        EX_EXPECT(b2[0] == 7.0f && b2[200] == 7.0f);
        EX_CHECK(HcommAicpuTsTaskCacheClear(tag.c_str()));

        EX_CHECK(HcclBarrier(comm, nullptr));
        EX_CHECK(HcclEngineCtxDestroy(comm, "rs_prims", COMM_ENGINE_CPU_TS));
        EX_CHECK(HcclChannelDestroy(comm, ch.data(), n - 1));
        EX_CHECK(HcclCommMemUnreg(comm, memHandle));
    });
    std::printf("reduce_scatter_primitives: %u ranks ok\n", n);
    return 0;
}
