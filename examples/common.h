// Shared scaffolding of the examples: every rank of the job is a thread of this process.
//
// Run with HCCL_SIM=1 for a CPU-only walk-through (buffers are host memory, operators complete before they
// return when the stream argument is NULL).  On GPUs the same calls take device pointers and a cudaStream_t; bind
// each rank thread to its device with cudaSetDevice before it creates the communicator.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <thread>
#include <vector>

#include "hccl/hccl.h"
#include "hccl/hccl_comm.h"

#define EX_CHECK(call)                                                                                         \
    do {                                                                                                       \
        int rc_ = (int)(call);                                                                                 \
        if (rc_ != 0) {                                                                                        \
            std::fprintf(stderr, "%s:%d: %s -> %d (%s)\n", __FILE__, __LINE__, #call, rc_, HcclGetErrorString((HcclResult)rc_)); \
            std::exit(1);                                                                                      \
        }                                                                                                      \
    } while (0)

#define EX_EXPECT(cond)                                                                      \
    do {                                                                                     \
        if (!(cond)) {                                                                       \
            std::fprintf(stderr, "%s:%d: expectation failed: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(2);                                                                    \
        }                                                                                    \
    } while (0)

// Creates `n` communicators from one root info (rank 0's ticket) and runs fn(rank, comm) in n threads.
inline void ExRunRanks(uint32_t n, const std::function<void(uint32_t, HcclComm)> &fn)
{
    HcclRootInfo info;
    EX_CHECK(HcclGetRootInfo(&info));
    std::vector<std::thread> ts;
    for (uint32_t r = 0; r < n; ++r) {
        ts.emplace_back([&, r] {
            HcclComm comm = nullptr;
            EX_CHECK(HcclCommInitRootInfo(n, &info, r, &comm));
            fn(r, comm);
            EX_CHECK(HcclCommDestroy(comm));
        });
    }
    for (auto &t : ts) t.join();
}
