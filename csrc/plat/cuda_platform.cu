// cuda_platform.cu - Platform on a B200: CUDA VMM symmetric memory, NVLS multicast objects,
// CUDA streams, and the small helper kernels of the host-TS engine (reduce, flag add, bounded
// flag wait).
//
// The library links the CUDA runtime statically and never links libcuda: driver entry points are
// resolved at first use through cudaGetDriverEntryPoint, so the shared object also loads on a
// machine without a driver (where CudaInstance() simply returns nullptr).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <mutex>

#include "../core/dtype.h"
#include "../core/log.h"
#include "platform.h"

namespace hc {
namespace {

#define CUDA_CHK(expr)                                                                        \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess) {                                                              \
            HCCL_ERROR("%s -> %s", #expr, cudaGetErrorString(_e));                            \
            return HCCL_E_RUNTIME;                                                            \
        }                                                                                     \
    } while (0)

struct Driver {
    bool ok = false;
#define HC_DRV_FN(name) decltype(&name) p_##name = nullptr;
    HC_DRV_FN(cuMemCreate)
    HC_DRV_FN(cuMemRelease)
    HC_DRV_FN(cuMemExportToShareableHandle)
    HC_DRV_FN(cuMemImportFromShareableHandle)
    HC_DRV_FN(cuMemAddressReserve)
    HC_DRV_FN(cuMemAddressFree)
    HC_DRV_FN(cuMemMap)
    HC_DRV_FN(cuMemUnmap)
    HC_DRV_FN(cuMemSetAccess)
    HC_DRV_FN(cuMemGetAllocationGranularity)
    HC_DRV_FN(cuMemRetainAllocationHandle)
    HC_DRV_FN(cuMemGetAddressRange)
    HC_DRV_FN(cuMulticastCreate)
    HC_DRV_FN(cuMulticastAddDevice)
    HC_DRV_FN(cuMulticastBindMem)
    HC_DRV_FN(cuMulticastUnbind)
    HC_DRV_FN(cuMulticastGetGranularity)
    HC_DRV_FN(cuDeviceGetAttribute)
    HC_DRV_FN(cuGetErrorString)
#undef HC_DRV_FN
    void Load()
    {
        ok = true;
#define HC_DRV_LOAD(name)                                                                             \
    {                                                                                                 \
        void *fn = nullptr;                                                                           \
        cudaDriverEntryPointQueryResult q;                                                            \
        if (cudaGetDriverEntryPoint(#name, &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {       \
            HCCL_WARNING("driver entry point %s unavailable", #name);                                 \
            ok = false;                                                                               \
        }                                                                                             \
        p_##name = (decltype(p_##name))fn;                                                            \
    }
        HC_DRV_LOAD(cuMemCreate) HC_DRV_LOAD(cuMemRelease) HC_DRV_LOAD(cuMemExportToShareableHandle)
        HC_DRV_LOAD(cuMemImportFromShareableHandle) HC_DRV_LOAD(cuMemAddressReserve) HC_DRV_LOAD(cuMemAddressFree)
        HC_DRV_LOAD(cuMemMap) HC_DRV_LOAD(cuMemUnmap) HC_DRV_LOAD(cuMemSetAccess)
        HC_DRV_LOAD(cuMemGetAllocationGranularity) HC_DRV_LOAD(cuMemRetainAllocationHandle)
        HC_DRV_LOAD(cuMemGetAddressRange) HC_DRV_LOAD(cuMulticastCreate) HC_DRV_LOAD(cuMulticastAddDevice)
        HC_DRV_LOAD(cuMulticastBindMem) HC_DRV_LOAD(cuMulticastUnbind) HC_DRV_LOAD(cuMulticastGetGranularity)
        HC_DRV_LOAD(cuDeviceGetAttribute) HC_DRV_LOAD(cuGetErrorString)
#undef HC_DRV_LOAD
        cudaGetLastError();
    }
};
Driver g_drv;

#define DRV_CHK(call)                                                                         \
    do {                                                                                      \
        CUresult _r = (call);                                                                 \
        if (_r != CUDA_SUCCESS) {                                                             \
            const char *_s = nullptr;                                                         \
            if (g_drv.p_cuGetErrorString) g_drv.p_cuGetErrorString(_r, &_s);                  \
            HCCL_ERROR("%s -> %d (%s)", #call, (int)_r, _s ? _s : "?");                       \
            return _r == CUDA_ERROR_OUT_OF_MEMORY ? HCCL_E_OOM : HCCL_E_DRV;                  \
        }                                                                                     \
    } while (0)

// ------------------------------------------------------------------------- helper kernels

template <typename T> struct Acc { using type = T; };
template <> struct Acc<__half> { using type = float; };
template <> struct Acc<__nv_bfloat16> { using type = float; };

template <typename A> __device__ __forceinline__ A OpApply(int op, A a, A b)
{
    switch (op) {
        case HCCL_REDUCE_SUM: return a + b;
        case HCCL_REDUCE_PROD: return a * b;
        case HCCL_REDUCE_MAX: return a > b ? a : b;
        default: return a < b ? a : b;
    }
}

template <typename T>
__global__ void HostTsReduceKernel(T *__restrict__ dst, const T *__restrict__ src, uint64_t count, int op)
{
    using A = typename Acc<T>::type;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; i < count; i += stride) dst[i] = (T)OpApply<A>(op, (A)dst[i], (A)src[i]);
}

template <typename T>
__global__ void HostTsScaleKernel(T *__restrict__ buf, uint64_t count, float scale)
{
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; i < count; i += stride) buf[i] = (T)((typename Acc<T>::type)buf[i] * (typename Acc<T>::type)scale);
}

__global__ void FlagAddKernel(uint64_t *flag, uint64_t v)
{
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(flag), "l"(v) : "memory");
}

__global__ void FlagWaitGeKernel(const uint64_t *flag, uint64_t expected, uint64_t timeoutNs, HcclDeviceWaitStatus *status,
                                 uint32_t *abortWord, uint32_t rank, uint32_t peer, uint32_t kind, uint32_t slot, uint64_t seq)
{
    uint64_t start, now, seen;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
    for (uint32_t it = 0;; ++it) {
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(flag) : "memory");
        if (seen >= expected) return;
        if (abortWord && *(volatile uint32_t *)abortWord) return;
        if ((it & 15) == 15) {
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - start > timeoutNs) break;
            __nanosleep(200);
        }
    }
    // Gave up: leave a record for the host and make later waits of this operator return at once.
    if (status && atomicExch_system(&status->valid, 1u) == 0u) {
        status->rank = rank; status->peer = peer; status->kind = kind; status->slot = slot; status->block = 0;
        status->expected = expected; status->seen = seen; status->seq = seq;
    }
    if (abortWord) *(volatile uint32_t *)abortWord = 1u;
    __threadfence_system();
}

thread_local int t_dev = -1;

class CudaPlatform : public Platform {
    std::mutex peekMu_;
    std::map<int, cudaStream_t> peekStreams_;

public:
    PlatKind kind() const override { return PlatKind::CUDA; }
    const char *name() const override { return "cuda-sm100"; }
    int DeviceCount() override { int n = 0; if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; } return n; }
    HcclResult SetDevice(int dev) override { CUDA_CHK(cudaSetDevice(dev)); t_dev = dev; CUDA_CHK(cudaFree(0)); return HCCL_SUCCESS; }
    int CurrentDevice() override { int d = 0; cudaGetDevice(&d); return d; }

    size_t Granularity() override
    {
        if (gran_) return gran_;
        CUmemAllocationProp prop = Prop(CurrentDevice());
        size_t g = 2u << 20;
        if (g_drv.p_cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) g = 2u << 20;
        if (MulticastSupported()) {
            CUmulticastObjectProp mp;
            memset(&mp, 0, sizeof(mp));
            mp.numDevices = 2; mp.size = g; mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
            size_t mg = 0;
            if (g_drv.p_cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > g) g = mg;
        }
        gran_ = g;
        return g;
    }
    HcclResult PhysAlloc(size_t bytes, PhysMem *out) override
    {
        CUmemAllocationProp prop = Prop(CurrentDevice());
        CUmemGenericAllocationHandle h;
        DRV_CHK(g_drv.p_cuMemCreate(&h, bytes, &prop, 0));
        out->handle = (uint64_t)h; out->bytes = bytes; out->imported = false;
        return HCCL_SUCCESS;
    }
    HcclResult PhysExportFd(const PhysMem &m, int *fd) override
    {
        int f = -1;
        DRV_CHK(g_drv.p_cuMemExportToShareableHandle(&f, (CUmemGenericAllocationHandle)m.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        *fd = f;
        return HCCL_SUCCESS;
    }
    HcclResult PhysImportFd(int fd, size_t bytes, PhysMem *out) override
    {
        CUmemGenericAllocationHandle h;
        DRV_CHK(g_drv.p_cuMemImportFromShareableHandle(&h, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
        out->handle = (uint64_t)h; out->bytes = bytes; out->imported = true;
        return HCCL_SUCCESS;
    }
    HcclResult PhysRelease(PhysMem *m) override
    {
        if (m->bytes) DRV_CHK(g_drv.p_cuMemRelease((CUmemGenericAllocationHandle)m->handle));
        *m = PhysMem();
        return HCCL_SUCCESS;
    }
    HcclResult VaReserve(size_t bytes, void **base) override
    {
        CUdeviceptr p = 0;
        DRV_CHK(g_drv.p_cuMemAddressReserve(&p, bytes, Granularity(), 0, 0));
        *base = (void *)p;
        return HCCL_SUCCESS;
    }
    HcclResult VaFree(void *base, size_t bytes) override { DRV_CHK(g_drv.p_cuMemAddressFree((CUdeviceptr)base, bytes)); return HCCL_SUCCESS; }
    HcclResult Map(void *va, const PhysMem &m, size_t bytes) override
    {
        DRV_CHK(g_drv.p_cuMemMap((CUdeviceptr)va, bytes, 0, (CUmemGenericAllocationHandle)m.handle, 0));
        CUmemAccessDesc acc;
        memset(&acc, 0, sizeof(acc));
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = CurrentDevice();
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        DRV_CHK(g_drv.p_cuMemSetAccess((CUdeviceptr)va, bytes, &acc, 1));
        return HCCL_SUCCESS;
    }
    HcclResult Unmap(void *va, size_t bytes) override { DRV_CHK(g_drv.p_cuMemUnmap((CUdeviceptr)va, bytes)); return HCCL_SUCCESS; }
    HcclResult RetainPhys(void *ptr, PhysMem *out, void **allocBase, size_t *allocBytes) override
    {
        CUmemGenericAllocationHandle h;
        if (g_drv.p_cuMemRetainAllocationHandle(&h, ptr) != CUDA_SUCCESS) return HCCL_E_NOT_FOUND;
        CUdeviceptr base = 0;
        size_t size = 0;
        if (g_drv.p_cuMemGetAddressRange(&base, &size, (CUdeviceptr)ptr) != CUDA_SUCCESS) { g_drv.p_cuMemRelease(h); return HCCL_E_NOT_FOUND; }
        out->handle = (uint64_t)h; out->bytes = size; out->imported = true;
        *allocBase = (void *)base; *allocBytes = size;
        return HCCL_SUCCESS;
    }
    HcclResult IpcExport(void *ptr, std::vector<uint8_t> *token, size_t *offsetInAlloc) override
    {
        CUdeviceptr base = 0;
        size_t size = 0;
        if (g_drv.p_cuMemGetAddressRange(&base, &size, (CUdeviceptr)ptr) != CUDA_SUCCESS) return HCCL_E_PARA;
        cudaIpcMemHandle_t h;
        CUDA_CHK(cudaIpcGetMemHandle(&h, (void *)base));
        token->assign((uint8_t *)&h, (uint8_t *)&h + sizeof(h));
        uint64_t sz = size;
        token->insert(token->end(), (uint8_t *)&sz, (uint8_t *)&sz + 8);
        *offsetInAlloc = (size_t)((CUdeviceptr)ptr - base);
        return HCCL_SUCCESS;
    }
    HcclResult IpcImport(const std::vector<uint8_t> &token, void **base) override
    {
        if (token.size() < sizeof(cudaIpcMemHandle_t)) return HCCL_E_PARA;
        cudaIpcMemHandle_t h;
        memcpy(&h, token.data(), sizeof(h));
        CUDA_CHK(cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess));
        return HCCL_SUCCESS;
    }
    HcclResult IpcClose(void *base) override { CUDA_CHK(cudaIpcCloseMemHandle(base)); return HCCL_SUCCESS; }

    bool MulticastSupported() override
    {
        if (mcChecked_) return mcOk_;
        int v = 0;
        mcOk_ = g_drv.p_cuDeviceGetAttribute && g_drv.p_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, CurrentDevice()) == CUDA_SUCCESS && v != 0;
        mcChecked_ = true;
        return mcOk_;
    }
    HcclResult McCreate(size_t bytes, int numDevices, PhysMem *mc) override
    {
        CUmulticastObjectProp mp;
        memset(&mp, 0, sizeof(mp));
        mp.numDevices = (unsigned)numDevices; mp.size = bytes; mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        CUmemGenericAllocationHandle h;
        DRV_CHK(g_drv.p_cuMulticastCreate(&h, &mp));
        mc->handle = (uint64_t)h; mc->bytes = bytes; mc->imported = false;
        return HCCL_SUCCESS;
    }
    HcclResult McAddDevice(const PhysMem &mc) override
    {
        DRV_CHK(g_drv.p_cuMulticastAddDevice((CUmemGenericAllocationHandle)mc.handle, CurrentDevice()));
        return HCCL_SUCCESS;
    }
    HcclResult McBind(const PhysMem &mc, size_t mcOffset, const PhysMem &phys, size_t bytes) override
    {
        DRV_CHK(g_drv.p_cuMulticastBindMem((CUmemGenericAllocationHandle)mc.handle, mcOffset, (CUmemGenericAllocationHandle)phys.handle, 0, bytes, 0));
        return HCCL_SUCCESS;
    }
    HcclResult McUnbind(const PhysMem &mc, size_t mcOffset, size_t bytes) override
    {
        DRV_CHK(g_drv.p_cuMulticastUnbind((CUmemGenericAllocationHandle)mc.handle, CurrentDevice(), mcOffset, bytes));
        return HCCL_SUCCESS;
    }

    HcclResult DevAlloc(size_t bytes, void **ptr) override { CUDA_CHK(cudaMalloc(ptr, bytes ? bytes : 1)); return HCCL_SUCCESS; }
    HcclResult DevFree(void *ptr) override { CUDA_CHK(cudaFree(ptr)); return HCCL_SUCCESS; }
    HcclResult HostAlloc(size_t bytes, void **ptr) override { CUDA_CHK(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocMapped | cudaHostAllocPortable)); return HCCL_SUCCESS; }
    HcclResult HostFree(void *ptr) override { CUDA_CHK(cudaFreeHost(ptr)); return HCCL_SUCCESS; }
    HcclResult MemsetSync(void *ptr, int v, size_t bytes) override { CUDA_CHK(cudaMemset(ptr, v, bytes)); CUDA_CHK(cudaDeviceSynchronize()); return HCCL_SUCCESS; }
    HcclResult MemcpySync(void *dst, const void *src, size_t bytes) override { CUDA_CHK(cudaMemcpy(dst, src, bytes, cudaMemcpyDefault)); return HCCL_SUCCESS; }

    HcclResult PeekSync(void *hostDst, const void *devSrc, size_t bytes) override
    {
        std::lock_guard<std::mutex> lk(peekMu_);
        cudaStream_t &st = peekStreams_[CurrentDevice()];
        if (!st) CUDA_CHK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
        CUDA_CHK(cudaMemcpyAsync(hostDst, devSrc, bytes, cudaMemcpyDeviceToHost, st));
        CUDA_CHK(cudaStreamSynchronize(st));
        return HCCL_SUCCESS;
    }
    HcclResult StreamCreate(Stream *s) override { cudaStream_t st; CUDA_CHK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking)); *s = st; return HCCL_SUCCESS; }
    HcclResult StreamDestroy(Stream s) override { CUDA_CHK(cudaStreamDestroy((cudaStream_t)s)); return HCCL_SUCCESS; }
    HcclResult StreamSync(Stream s) override { CUDA_CHK(cudaStreamSynchronize((cudaStream_t)s)); return HCCL_SUCCESS; }
    HcclResult StreamOrder(Stream before, Stream after) override
    {
        cudaEvent_t ev;
        CUDA_CHK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        CUDA_CHK(cudaEventRecord(ev, (cudaStream_t)before));
        CUDA_CHK(cudaStreamWaitEvent((cudaStream_t)after, ev, 0));
        CUDA_CHK(cudaEventDestroy(ev));   // released by the runtime once the wait has consumed it
        return HCCL_SUCCESS;
    }
    bool StreamCapturing(Stream s) override
    {
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing((cudaStream_t)s, &st) != cudaSuccess) { cudaGetLastError(); return false; }
        return st != cudaStreamCaptureStatusNone;
    }

    HcclResult MemcpyAsync(void *dst, const void *src, size_t bytes, Stream s) override
    {
        CUDA_CHK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, (cudaStream_t)s));
        return HCCL_SUCCESS;
    }
    HcclResult ReduceAsync(void *dst, const void *src, uint64_t count, HcclDataType t, HcclReduceOp op, Stream s) override
    {
        if (count == 0) return HCCL_SUCCESS;
        int threads = 256;
        uint64_t want = (count + threads - 1) / threads;
        int blocks = (int)(want > 1184 ? 1184 : want);   // 8 CTAs per SM on 148 SMs
        cudaStream_t st = (cudaStream_t)s;
#define HC_LAUNCH(E, T) case E: HostTsReduceKernel<T><<<blocks, threads, 0, st>>>((T *)dst, (const T *)src, count, (int)op); break;
        switch (t) {
            HC_LAUNCH(HCCL_DATA_TYPE_INT8, int8_t) HC_LAUNCH(HCCL_DATA_TYPE_INT16, int16_t) HC_LAUNCH(HCCL_DATA_TYPE_INT32, int32_t)
            HC_LAUNCH(HCCL_DATA_TYPE_INT64, long long) HC_LAUNCH(HCCL_DATA_TYPE_UINT8, uint8_t) HC_LAUNCH(HCCL_DATA_TYPE_UINT16, uint16_t)
            HC_LAUNCH(HCCL_DATA_TYPE_UINT32, uint32_t) HC_LAUNCH(HCCL_DATA_TYPE_UINT64, unsigned long long)
            HC_LAUNCH(HCCL_DATA_TYPE_FP32, float) HC_LAUNCH(HCCL_DATA_TYPE_FP64, double)
            HC_LAUNCH(HCCL_DATA_TYPE_FP16, __half) HC_LAUNCH(HCCL_DATA_TYPE_BFP16, __nv_bfloat16)
            default: return HCCL_E_NOT_SUPPORT;
        }
#undef HC_LAUNCH
        CUDA_CHK(cudaGetLastError());
        return HCCL_SUCCESS;
    }
    HcclResult ScaleAsync(void *buf, uint64_t count, HcclDataType t, float scale, Stream s) override
    {
        if (count == 0) return HCCL_SUCCESS;
        const int threads = 256;
        uint64_t want = (count + threads - 1) / threads;
        int blocks = (int)(want > 1184 ? 1184 : want);
        cudaStream_t st = (cudaStream_t)s;
        switch (t) {
            case HCCL_DATA_TYPE_FP32: HostTsScaleKernel<float><<<blocks, threads, 0, st>>>((float *)buf, count, scale); break;
            case HCCL_DATA_TYPE_FP64: HostTsScaleKernel<double><<<blocks, threads, 0, st>>>((double *)buf, count, scale); break;
            case HCCL_DATA_TYPE_FP16: HostTsScaleKernel<__half><<<blocks, threads, 0, st>>>((__half *)buf, count, scale); break;
            case HCCL_DATA_TYPE_BFP16: HostTsScaleKernel<__nv_bfloat16><<<blocks, threads, 0, st>>>((__nv_bfloat16 *)buf, count, scale); break;
            default: return HCCL_E_NOT_SUPPORT;
        }
        CUDA_CHK(cudaGetLastError());
        return HCCL_SUCCESS;
    }
    HcclResult FlagAddAsync(uint64_t *flag, uint64_t v, Stream s) override
    {
        FlagAddKernel<<<1, 1, 0, (cudaStream_t)s>>>(flag, v);
        CUDA_CHK(cudaGetLastError());
        return HCCL_SUCCESS;
    }
    HcclResult FlagWaitGeAsync(uint64_t *flag, uint64_t expected, uint32_t timeoutMs, const WaitReport &rep, Stream s) override
    {
        FlagWaitGeKernel<<<1, 1, 0, (cudaStream_t)s>>>(flag, expected, (uint64_t)timeoutMs * 1000000ull, rep.status, rep.abortWord,
                                                        rep.rank, rep.peer, rep.kind, rep.slot, rep.seq);
        CUDA_CHK(cudaGetLastError());
        return HCCL_SUCCESS;
    }
    HcclResult HostFuncAsync(std::function<void()> fn, Stream s) override
    {
        auto *heapFn = new std::function<void()>(std::move(fn));
        cudaError_t e = cudaLaunchHostFunc((cudaStream_t)s, [](void *p) {
            auto *f = (std::function<void()> *)p;
            (*f)();
            delete f;
        }, heapFn);
        if (e != cudaSuccess) { delete heapFn; HCCL_ERROR("cudaLaunchHostFunc: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
        return HCCL_SUCCESS;
    }

private:
    static CUmemAllocationProp Prop(int dev)
    {
        CUmemAllocationProp prop;
        memset(&prop, 0, sizeof(prop));
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = dev;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        return prop;
    }
    size_t gran_ = 0;
    bool mcChecked_ = false, mcOk_ = false;
};

}  // namespace

// Forces the helper kernels of the stream engine to be loaded on the current device.  A wait kernel may be spinning
// when the host issues the first reduce; with lazy loading that first launch could have to wait for the spinning
// kernel, whose partner may be stuck the same way on the other side.
void PreloadPlatformKernels()
{
    cudaFuncAttributes a;
    cudaFuncGetAttributes(&a, FlagAddKernel);
    cudaFuncGetAttributes(&a, FlagWaitGeKernel);
    cudaFuncGetAttributes(&a, HostTsScaleKernel<float>); cudaFuncGetAttributes(&a, HostTsScaleKernel<double>);
    cudaFuncGetAttributes(&a, HostTsScaleKernel<__half>); cudaFuncGetAttributes(&a, HostTsScaleKernel<__nv_bfloat16>);
#define HC_PRELOAD(T) cudaFuncGetAttributes(&a, HostTsReduceKernel<T>);
    HC_PRELOAD(int8_t) HC_PRELOAD(int16_t) HC_PRELOAD(int32_t) HC_PRELOAD(long long) HC_PRELOAD(uint8_t) HC_PRELOAD(uint16_t) HC_PRELOAD(uint32_t)
    HC_PRELOAD(unsigned long long) HC_PRELOAD(float) HC_PRELOAD(double) HC_PRELOAD(__half) HC_PRELOAD(__nv_bfloat16)
#undef HC_PRELOAD
    cudaGetLastError();
}

Platform *CudaInstance()
{
    static std::once_flag once;
    static CudaPlatform *inst = nullptr;
    std::call_once(once, [] {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { cudaGetLastError(); return; }
        g_drv.Load();
        if (!g_drv.ok) { HCCL_WARNING("CUDA driver lacks the virtual-memory API; CUDA platform disabled"); return; }
        inst = new CudaPlatform();
    });
    return inst;
}

}  // namespace hc
