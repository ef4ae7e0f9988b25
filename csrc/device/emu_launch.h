// emu_launch.h - one launch for several ranks that share a GPU.
//
// When all ranks of a communicator are threads of one process bound to the same GPU (how the
// multi-rank kernels are exercised on a single device), their kernels wait for each other and
// therefore must be ONE cooperative launch.  Each rank thread calls EmuLaunch with its own argument
// block; the call blocks until all ranks of the group have arrived, the last arrival launches the
// kernel with gridDim.y = nRanks on a stream owned by the group, and every rank's stream is made to
// wait for its completion.
#pragma once
#include <string>

#include "coll_kernels.h"

namespace hc {

HcclResult EmuLaunch(const std::string &groupKey, uint32_t nRanks, uint32_t rank, const FastLaunch &l);
void EmuForget(const std::string &groupKey);

}  // namespace hc
