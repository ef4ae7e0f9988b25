// platform.h - the one seam between the portable host runtime and a device.
//
// Two implementations exist: CudaPlatform (B200: CUDA VMM memory, CUDA streams, small helper
// kernels) and SimPlatform (host: memfd-backed shared memory, worker threads as streams).  The
// simulator plays the role the reference's stub runtime plays for its unit tests
// (test/ut/stub/llt_hccl_stub.cc): ranks may be threads of one process or separate processes, and
// the complete control plane, symmetric-memory exchange, schedule generation and host-engine
// execution run unchanged on it.
//
// Symmetric memory is built from four verbs that both back ends provide with identical meaning:
//   PhysAlloc    a block of physical memory that can be shared by file descriptor
//   PhysExportFd / PhysImportFd   move the block between processes
//   VaReserve    a range of addresses with nothing behind it
//   Map          put a block behind part of a reserved range
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <vector>

#include "hccl/hccl_diag.h"
#include "hccl/hccl_types.h"

namespace hc {

enum class PlatKind { SIM = 0, CUDA = 1 };

struct PhysMem {
    uint64_t handle = 0;   // CUmemGenericAllocationHandle, or the memfd on the simulator
    size_t bytes = 0;
    bool imported = false;
};

using Stream = void *;

// Shared by every bounded wait: where to report when the wait gives up.
struct WaitReport {
    HcclDeviceWaitStatus *status = nullptr;  // host-visible record (pinned memory on CUDA)
    uint32_t *abortWord = nullptr;           // set to 1 on expiry; later waits return at once
    uint32_t rank = 0, peer = 0, kind = 0, slot = 0;
    uint64_t seq = 0;
};

class Platform {
public:
    virtual ~Platform() {}
    virtual PlatKind kind() const = 0;
    virtual const char *name() const = 0;
    virtual int DeviceCount() = 0;
    virtual HcclResult SetDevice(int dev) = 0;  // binds the calling thread
    virtual int CurrentDevice() = 0;

    // ---- symmetric memory verbs
    virtual size_t Granularity() = 0;
    virtual HcclResult PhysAlloc(size_t bytes, PhysMem *out) = 0;
    virtual HcclResult PhysExportFd(const PhysMem &m, int *fd) = 0;   // caller closes *fd
    virtual HcclResult PhysImportFd(int fd, size_t bytes, PhysMem *out) = 0;
    virtual HcclResult PhysRelease(PhysMem *m) = 0;
    virtual HcclResult VaReserve(size_t bytes, void **base) = 0;
    virtual HcclResult VaFree(void *base, size_t bytes) = 0;
    virtual HcclResult Map(void *va, const PhysMem &m, size_t bytes) = 0;
    virtual HcclResult Unmap(void *va, size_t bytes) = 0;
    // If `ptr` lies in memory created through the VMM verbs, returns its backing block.
    virtual HcclResult RetainPhys(void *ptr, PhysMem *out, void **allocBase, size_t *allocBytes) = 0;
    // Fallback for memory that came from a plain allocator (cudaMalloc): opaque IPC tokens.
    virtual HcclResult IpcExport(void *ptr, std::vector<uint8_t> *token, size_t *offsetInAlloc) = 0;
    virtual HcclResult IpcImport(const std::vector<uint8_t> &token, void **base) = 0;
    virtual HcclResult IpcClose(void *base) = 0;

    // ---- multicast (NVLS); the simulator reports unsupported
    virtual bool MulticastSupported() = 0;
    virtual HcclResult McCreate(size_t bytes, int numDevices, PhysMem *mc) = 0;
    virtual HcclResult McAddDevice(const PhysMem &mc) = 0;
    virtual HcclResult McBind(const PhysMem &mc, size_t mcOffset, const PhysMem &phys, size_t bytes) = 0;
    virtual HcclResult McUnbind(const PhysMem &mc, size_t mcOffset, size_t bytes) = 0;

    // ---- plain memory
    virtual HcclResult DevAlloc(size_t bytes, void **ptr) = 0;
    virtual HcclResult DevFree(void *ptr) = 0;
    virtual HcclResult HostAlloc(size_t bytes, void **ptr) = 0;   // pinned + device-visible on CUDA
    virtual HcclResult HostFree(void *ptr) = 0;
    virtual HcclResult MemsetSync(void *ptr, int v, size_t bytes) = 0;
    virtual HcclResult MemcpySync(void *dst, const void *src, size_t bytes) = 0;

    // ---- ordered execution
    // Copies a few bytes of device memory to the host without touching the streams of the application (works while
    // a kernel of the communicator is still running or stuck).
    virtual HcclResult PeekSync(void *hostDst, const void *devSrc, size_t bytes) = 0;
    virtual HcclResult StreamCreate(Stream *s) = 0;
    virtual HcclResult StreamDestroy(Stream s) = 0;
    virtual HcclResult StreamSync(Stream s) = 0;
    // Everything enqueued on `after` from now on runs after what is on `before` now.
    virtual HcclResult StreamOrder(Stream before, Stream after) = 0;
    virtual bool StreamCapturing(Stream s) = 0;

    // ---- task primitives of the host-TS engine
    virtual HcclResult MemcpyAsync(void *dst, const void *src, size_t bytes, Stream s) = 0;
    virtual HcclResult ReduceAsync(void *dst, const void *src, uint64_t count, HcclDataType t, HcclReduceOp op,
                                   Stream s) = 0;
    // *flag += v with release semantics visible to every GPU and the host.
    // buf[i] = buf[i] * scale for floating-point element types (fp16 / bf16 are scaled in fp32).
    virtual HcclResult ScaleAsync(void *buf, uint64_t count, HcclDataType t, float scale, Stream s) = 0;
    virtual HcclResult FlagAddAsync(uint64_t *flag, uint64_t v, Stream s) = 0;
    // Blocks the stream until *flag >= expected, or timeoutMs elapses (then fills `rep`).
    virtual HcclResult FlagWaitGeAsync(uint64_t *flag, uint64_t expected, uint32_t timeoutMs, const WaitReport &rep,
                                       Stream s) = 0;
    virtual HcclResult HostFuncAsync(std::function<void()> fn, Stream s) = 0;
};

// Process singletons.  CudaInstance() returns nullptr when no usable driver or device is present.
Platform *SimInstance();
Platform *CudaInstance();
// Applies HCCL_SIM: 1 -> simulator, 0 -> CUDA or failure, unset -> CUDA when available else simulator.
Platform *DefaultPlatform();
// Simulator only, for tests of the failure paths: the next n flag writes issued by this process are dropped.
void SimWithholdFlagWrites(int n);
// CUDA only: load the stream-engine helper kernels on the current device (see cuda_platform.cu).
void PreloadPlatformKernels();

}  // namespace hc
