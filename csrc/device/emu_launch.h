// emu_launch.h - one launch for several ranks that share a GPU.
//
// When all ranks of a communicator are threads of one process bound to the same GPU (how the
// multi-rank kernels are exercised on a single device), their kernels wait for each other and
// therefore must be ONE cooperative launch.  Each rank thread calls in with its own parameter block;
// the call blocks until all ranks of the group have arrived, the last arrival copies the blocks into a
// device table and launches once with gridDim.y = nRanks on a stream owned by the group, and every
// rank's stream is made to wait for the completion.
#pragma once
#include <functional>
#include <string>

#include "coll_kernels.h"

namespace hc {

// launch(devTable, nRanks, stream) is called once, by the last rank to arrive, with the device address of
// the nRanks parameter blocks (each paramBytes long, in rank order).  `id` must be the same on all ranks
// for one rendezvous (it detects ranks issuing different operators).
HcclResult EmuLaunchGeneric(const std::string &groupKey, uint32_t nRanks, uint32_t rank, int id, const void *params, size_t paramBytes, void *stream,
                            const std::function<HcclResult(const void *devTable, uint32_t nRanks, void *stream)> &launch);
HcclResult EmuLaunch(const std::string &groupKey, uint32_t nRanks, uint32_t rank, const FastLaunch &l);
void EmuForget(const std::string &groupKey);

}  // namespace hc
