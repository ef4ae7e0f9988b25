// templates.h - algorithm templates: functions that emit a Schedule for one collective and one
// strategy.  They are the B200 counterpart of the reference's alg_template directory
// (src/legacy/ascend910/algorithm/base/alg_template/*, 105 templates) reduced to the strategies
// that are distinct on a switch-connected node plus the classic multi-step ones:
//
//   mesh     every rank talks to every peer at once (one-shot for small data, two-shot otherwise)
//   ring     p-1 neighbour steps (reduce_scatter_ring.cc:87-312 of the reference for the step order)
//   hd       recursive halving / doubling with folding of the ranks beyond the largest power of two
//            (recursive_halvingdoubling_base.cc:21-90)
//   bruck    non-uniform Bruck for all-gather on any rank count ("NB")
//   pairwise step i exchanges with rank+i / rank-i (alltoallv_pairwise.cc:74-290)
//   tree     binomial tree for broadcast / reduce
//
// Conventions every template follows
//   notify 0 READY  receiver -> sender: "my scratch for this operator is free"
//   notify 1 DATA   sender -> receiver: "what I wrote to you is complete"
//   notify 2 FIN    owner -> reader:    "the slice you will read from me is final"
//   notify 3 DONE   reader -> owner:    "I finished reading from you"
//   A remote WRITE to rank q is always ordered after a WAIT(q, READY); a rank whose scratch is READ
//   by peers ends its program by waiting for DONE from each reader.  Reductions add contributions
//   in ascending rank order on every rank, so all ranks obtain bit-identical results.
#pragma once
#include <string>
#include <vector>

#include "ir.h"

namespace hc {

enum Notify : uint16_t { N_READY = 0, N_DATA = 1, N_FIN = 2, N_DONE = 3, N_COUNT = 4 };

enum class Algo : uint8_t { AUTO = 0, MESH, MESH_ONESHOT, RING, HD, BRUCK, PAIRWISE, TREE, NVLS, STAR, NHR };
const char *AlgoName(Algo a);
// Accepts the reference's spellings: ring, fullmesh, H-D_R, pairwise, NHR, NHR_V1, NB, AHC, AHC_BROKE, pipeline, null.
bool ParseAlgoName(const std::string &s, Algo *out);

struct CollShape {
    HcclCMDType cmd = HCCL_CMD_INVALID;
    uint32_t nRanks = 1;
    uint32_t root = 0;
    uint64_t count = 0;             // per-collective meaning: AR total, RS recvCount, AG sendCount, A2A per-peer count ...
    uint32_t elemSize = 4;
    // Variable-count collectives: per-rank rows (nRanks x nRanks for all-to-all, 1 x nRanks otherwise).
    std::vector<std::vector<uint64_t>> sendCounts, sendDispls, recvCounts, recvDispls;
    // Point-to-point: src and dst ranks.
    uint32_t p2pSrc = 0, p2pDst = 0;
    int onlyRank = -1;              // >= 0: emit only this rank's program (what a real rank needs)
};

// Returns false (and explains in *why) when the strategy cannot serve the shape, e.g. halving-doubling
// reduce-scatter on a rank count that is not a power of two.
bool BuildSchedule(const CollShape &shape, Algo algo, Schedule *out, std::string *why);
// Strategies that BuildSchedule accepts for a collective, best-first for a switch-connected node.
std::vector<Algo> AlgosFor(HcclCMDType cmd, uint32_t nRanks);
// Elements per slice used by uniform layouts: ceil(total/nSlices) rounded up to a 16-byte multiple.
uint64_t AlignedSliceCount(uint64_t total, uint32_t nSlices, uint32_t elemSize);

}  // namespace hc
