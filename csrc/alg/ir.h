// ir.h - the schedule IR: what every algorithm template produces and every engine consumes.
//
// A Schedule is, for each rank, a list of primitives grouped into logical threads.  A logical
// thread is an ordered execution context: a CUDA stream on the host-TS engine, one CTA on the SM
// engine (the interpreter kernel), a worker thread on the simulator.  Data is addressed in whole
// *slices*: a buffer is an array of slices described by per-slice displacement and count, and a
// primitive moves `nSlices` consecutive slices.  Because no primitive ever touches part of a slice,
// an engine may split every slice by columns into independent "channels" and run one replica of
// the schedule per channel without creating cross-channel dependencies.
//
// The primitive set is the one the reference's A5 flow lowers its templates to
// (service/collective/alg primitive/primitive.h:31-32, instruction/instruction.h:29-40):
//   COPY / REDUCE                local data movement
//   WRITE / WRITE_REDUCE         local source -> peer destination (peer's SCRATCH or registered OUTPUT)
//   READ / READ_REDUCE           peer source -> local destination
//   POST(peer, notify)           add one to notify slot `notify` that `peer` owns for this rank
//   WAIT(peer, notify)           consume one post from `peer` on slot `notify`
// POST/WAIT with peer == self and `toThread` set synchronise two logical threads of one rank.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "hccl/hccl_types.h"

namespace hc {

enum class PrimOp : uint8_t { COPY = 0, REDUCE, WRITE, WRITE_REDUCE, READ, READ_REDUCE, POST, WAIT, NOP };
const char *PrimOpName(PrimOp op);

// Which array of slices an operand lives in.
enum class BufId : uint8_t {
    INPUT = 0,    // the caller's send buffer (local only unless the op runs zero-copy)
    OUTPUT = 1,   // the caller's receive buffer
    SCRATCH = 2,  // this operator's half of the CCL buffer: peer-visible
    NONE = 3
};

struct Prim {
    PrimOp op = PrimOp::NOP;
    uint8_t thread = 0;        // logical thread that executes it
    int16_t peer = -1;         // remote rank (WRITE/READ/POST/WAIT); -1 for local ops
    BufId srcBuf = BufId::NONE, dstBuf = BufId::NONE;
    uint32_t srcSlice = 0, dstSlice = 0, nSlices = 1;
    uint16_t notify = 0;       // slot index for POST/WAIT
    uint8_t toThread = 0;      // POST/WAIT between threads of the same rank: the partner thread
    uint8_t step = 0;          // algorithm step, for traces and the checker's messages
    // Element count of moved slice i is the count of slice (lenSlice + i) of lenBuf.  Templates set it
    // to the operand that is a caller buffer, so that variable-count collectives move exact sizes.
    BufId lenBuf = BufId::NONE;
    uint32_t lenSlice = 0;
};

// Geometry of one operand kind, identical on every rank unless perRank is set.
struct SliceLayout {
    uint32_t nSlices = 0;
    // displ[i], count[i] in elements; empty = uniform: displ = i*sliceCount, count = sliceCount
    // clipped so that the total never exceeds `total`.
    std::vector<uint64_t> displ, count;
    uint64_t sliceCount = 0;
    uint64_t total = 0;
    uint64_t DisplOf(uint32_t i) const { return displ.empty() ? (uint64_t)i * sliceCount : displ[i]; }
    uint64_t CountOf(uint32_t i) const
    {
        if (!count.empty()) return count[i];
        uint64_t b = (uint64_t)i * sliceCount;
        if (b >= total) return 0;
        return (total - b < sliceCount) ? total - b : sliceCount;
    }
};

struct RankProgram {
    std::vector<Prim> prims;   // in issue order; per-thread order is the order within this list
    uint32_t nThreads = 1;
};

struct Schedule {
    std::string name;                 // "AllReduceRing", ...
    HcclCMDType cmd = HCCL_CMD_INVALID;
    uint32_t nRanks = 0;
    uint32_t root = 0;
    std::vector<RankProgram> ranks;
    // Layouts are per rank for the V-variants (counts differ per rank); index by rank, or size 1 = same everywhere.
    std::vector<SliceLayout> input, output;
    SliceLayout scratch;              // scratch geometry is always uniform
    uint32_t nNotify = 1;             // notify slots used per peer
    const SliceLayout &In(uint32_t r) const { return input.size() == 1 ? input[0] : input[r]; }
    const SliceLayout &Out(uint32_t r) const { return output.size() == 1 ? output[0] : output[r]; }
    std::string Dump(uint32_t rank) const;
    size_t TotalPrims() const;
};

// Compact form handed to the device interpreter (32 bytes per primitive).
struct DevPrim {
    uint8_t op, thread, srcBuf, dstBuf;
    int16_t peer;
    uint16_t notify;
    uint32_t srcSlice, dstSlice, nSlices;
    uint8_t toThread, step, lenBuf, pad;
    uint32_t lenSlice;
    uint32_t reserved;
};
static_assert(sizeof(DevPrim) == 32, "DevPrim is 32 bytes");

}  // namespace hc
