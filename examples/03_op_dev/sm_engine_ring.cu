// A communication operator written as a CUDA kernel against the device-side channel API (the SM engine): every rank
// sends a block to its right neighbour and receives the block of its left neighbour, all from inside one kernel per
// rank.  One rank per GPU (kernels of different ranks wait for each other, so they must not share a GPU).
//
//   host  : one channel per neighbour on the SM engine, HcclChannelGetDeviceView hands the kernel the peer's heap and
//           the notify words; the payload travels through the communication (CCL) buffer
//   kernel: 1. store the payload straight into the right neighbour's communication buffer (peer stores over NVLink)
//           2. record DATA on the channel to the right            (release: the stores above are visible first)
//           3. wait for DATA from the left                        (bounded: gives up after two seconds)
//           4. copy the block that arrived in the local communication buffer to the output
//           5. record ACK to the left, wait for ACK from the right: the buffers may be written again
// This is the seven-step recipe of the reference's operator guide (buffer - slice - copy-in - pre-sync - transfer -
// post-sync - copy-out, docs/zh/comm_op_dev_guide/aiv_comm_op_dev/task_sched.md:25-60) with the transfer done by the
// kernel itself.  Build: nvcc -gencode arch=compute_100a,code=sm_100a -Iinclude sm_engine_ring.cu -lhcomm.
#include <cuda_runtime.h>

#include <cstring>
#include <thread>
#include <vector>

#include "../common.h"
#include "hccl/hccl_channel.h"
#include "hccl/hccl_rank_graph.h"
#include "hccl/hccl_res.h"
#include "hcomm_device.cuh"

enum { NOTIFY_ACK = 0, NOTIFY_DATA = 1 };

#define CUDA_CHECK(call)                                                                                      \
    do {                                                                                                      \
        cudaError_t e_ = (call);                                                                              \
        if (e_ != cudaSuccess) { std::fprintf(stderr, "%s:%d: %s -> %s\n", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); std::exit(1); } \
    } while (0)

// round: 1, 2, ... - notify words only grow, the host tells the kernel which value this call waits for.
__global__ void RingStep(const hcdev::ChannelView *toRight, const hcdev::ChannelView *fromLeft, char *localBuf, const char *payload, char *received,
                         uint64_t bytes, uint64_t round, uint32_t *status)
{
    const uint64_t budgetNs = 2000000000ull;
    __shared__ int ok;
    hcdev::BlockCopy16(hcdev::ChannelPeerBuffer(toRight), payload, bytes);
    __syncthreads();
    if (threadIdx.x == 0) {
        hcdev::ChannelNotifyRecord(toRight, NOTIFY_DATA);
        ok = hcdev::ChannelNotifyWait(fromLeft, NOTIFY_DATA, round, budgetNs) ? 1 : 0;
    }
    __syncthreads();
    if (!ok) {
        if (threadIdx.x == 0) *status = 1;      // the left neighbour never signalled: report, do not hang
        return;
    }
    hcdev::BlockCopy16(received, localBuf, bytes);
    __syncthreads();
    if (threadIdx.x == 0) {
        hcdev::ChannelNotifyRecord(fromLeft, NOTIFY_ACK);
        if (!hcdev::ChannelNotifyWait(toRight, NOTIFY_ACK, round, budgetNs)) *status = 2;
    }
}

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 2;
    int gpus = 0;
    CUDA_CHECK(cudaGetDeviceCount(&gpus));
    if ((uint32_t)gpus < n || n < 2) {
        std::printf("sm_engine_ring needs %u GPUs (one per rank), found %d: skipped\n", n, gpus);
        return 0;
    }
    const uint64_t bytes = 1 << 20;
    HcclRootInfo info;
    EX_CHECK(HcclGetRootInfo(&info));
    std::vector<std::thread> ts;
    for (uint32_t rank = 0; rank < n; ++rank) {
        ts.emplace_back([&, rank] {
            CUDA_CHECK(cudaSetDevice((int)rank));
            HcclComm comm = nullptr;
            EX_CHECK(HcclCommInitRootInfo(n, &info, rank, &comm));
            const uint32_t right = (rank + 1) % n, left = (rank + n - 1) % n;
            HcclChannelDesc descs[2];
            EX_CHECK(HcclChannelDescInit(descs, 2));
            const uint32_t peers[2] = {right, left};
            for (int i = 0; i < 2; ++i) {
                CommLink *links = nullptr;
                uint32_t linkNum = 0;
                EX_CHECK(HcclRankGraphGetLinks(comm, 0, rank, peers[i], &links, &linkNum));
                EX_EXPECT(linkNum >= 1);
                descs[i].remoteRank = peers[i];
                descs[i].notifyNum = 2;
                descs[i].channelProtocol = links[0].linkAttr.linkProtocol;
            }
            ChannelHandle ch[2] = {0, 0};
            const uint32_t chNum = n == 2 ? 1 : 2;             // with two ranks left and right are the same peer
            EX_CHECK(HcclChannelAcquire(comm, COMM_ENGINE_AIV, descs, chNum, ch));
            void *viewRight = nullptr, *viewLeft = nullptr;
            EX_CHECK(HcclChannelGetDeviceView(comm, ch[0], &viewRight));
            EX_CHECK(HcclChannelGetDeviceView(comm, chNum == 2 ? ch[1] : ch[0], &viewLeft));
            void *localBuf = nullptr;
            uint64_t localSize = 0;
            EX_CHECK(HcclGetHcclBuffer(comm, &localBuf, &localSize));
            EX_EXPECT(localSize >= bytes);

            std::vector<uint8_t> payload(bytes), received(bytes, 0);
            char *dPayload = nullptr, *dReceived = nullptr;
            uint32_t *dStatus = nullptr;
            CUDA_CHECK(cudaMalloc(&dPayload, bytes));
            CUDA_CHECK(cudaMalloc(&dReceived, bytes));
            CUDA_CHECK(cudaMalloc(&dStatus, sizeof(uint32_t)));
            CUDA_CHECK(cudaMemset(dStatus, 0, sizeof(uint32_t)));
            cudaStream_t stream;
            CUDA_CHECK(cudaStreamCreate(&stream));
            for (uint64_t round = 1; round <= 3; ++round) {
                for (uint64_t i = 0; i < bytes; ++i) payload[i] = (uint8_t)(rank * 31 + i + round);
                CUDA_CHECK(cudaMemcpyAsync(dPayload, payload.data(), bytes, cudaMemcpyHostToDevice, stream));
                RingStep<<<1, 512, 0, stream>>>((const hcdev::ChannelView *)viewRight, (const hcdev::ChannelView *)viewLeft, (char *)localBuf, dPayload, dReceived,
                                                bytes, round, dStatus);
                CUDA_CHECK(cudaGetLastError());
                uint32_t status = 0;
                CUDA_CHECK(cudaMemcpyAsync(received.data(), dReceived, bytes, cudaMemcpyDeviceToHost, stream));
                CUDA_CHECK(cudaMemcpyAsync(&status, dStatus, sizeof(status), cudaMemcpyDeviceToHost, stream));
                CUDA_CHECK(cudaStreamSynchronize(stream));
                EX_EXPECT(status == 0);
                for (uint64_t i = 0; i < bytes; i += 4097) EX_EXPECT(received[i] == (uint8_t)(left * 31 + i + round));
            }
            cudaFree(dPayload); cudaFree(dReceived); cudaFree(dStatus);
            cudaStreamDestroy(stream);
            EX_CHECK(HcclChannelDestroy(comm, ch, chNum));
            EX_CHECK(HcclCommDestroy(comm));
        });
    }
    for (auto &t : ts) t.join();
    std::printf("sm_engine_ring: %u ranks ok\n", n);
    return 0;
}
