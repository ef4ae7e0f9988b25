// exec.h - running a Schedule on the host engines.
//
// The host executor walks this rank's program and turns every primitive into platform work on one
// stream: COPY/WRITE/READ become (peer-to-peer) memcpys, REDUCE a reduce kernel (or a CPU loop on the
// simulator), POST a release-add on the peer's notify word, WAIT a bounded wait on the local one.
// Slices larger than the scratch capacity are processed in column chunks; the READY handshake at the
// head of every schedule keeps consecutive chunks from overwriting each other.
// This is the engine behind op-expansion modes "host" and "host-TS" and the only engine of the
// simulator; the SM engine (device interpreter and specialised kernels) lives in csrc/device.
#pragma once
#include "../alg/ir.h"
#include "../comm/comm.h"

namespace hc {

struct ExecArgs {
    const void *in = nullptr;
    void *out = nullptr;
    HcclDataType dtype = HCCL_DATA_TYPE_FP32;
    HcclReduceOp op = HCCL_REDUCE_SUM;
    Stream stream = nullptr;
};

// Largest number of elements per slice that one pass can move given the schedule's scratch geometry.
uint64_t ScratchCapacityElems(const Comm *c, const Schedule &s, uint32_t elemSize);
HcclResult ExecuteOnHost(Comm *c, const Schedule &s, const ExecArgs &a);

}  // namespace hc
