// sim_platform.cc - host implementation of Platform.
//
// Physical blocks are memfd files, address ranges are PROT_NONE reservations and Map() is a
// MAP_FIXED shared mapping, so a block imported from another process (or another thread-rank of
// this process) aliases the same pages - the property the CUDA VMM path provides on the GPU.
// A stream is a worker thread draining a FIFO of closures; the null stream runs work inline.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <thread>

#include "../core/dtype.h"
#include "../core/log.h"
#include "../core/net.h"
#include "platform.h"

namespace hc {
namespace {
std::atomic<int> g_withhold{0};     // flag writes still to be dropped (tests)


class SimStream {
public:
    SimStream() : th_([this] { Loop(); }) {}
    ~SimStream()
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        th_.join();
    }
    void Push(std::function<void()> fn)
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            q_.push_back(std::move(fn));
            ++pushed_;
        }
        cv_.notify_all();
    }
    void Sync()
    {
        std::unique_lock<std::mutex> lk(mu_);
        uint64_t target = pushed_;
        done_cv_.wait(lk, [&] { return done_ >= target; });
    }
    // Ticket of everything enqueued so far, and a wait for it from another thread.
    uint64_t Ticket()
    {
        std::lock_guard<std::mutex> lk(mu_);
        return pushed_;
    }
    void WaitTicket(uint64_t t)
    {
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [&] { return done_ >= t; });
    }

private:
    void Loop()
    {
        for (;;) {
            std::function<void()> fn;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return stop_ || !q_.empty(); });
                if (q_.empty()) return;
                fn = std::move(q_.front());
                q_.pop_front();
            }
            fn();
            {
                std::lock_guard<std::mutex> lk(mu_);
                ++done_;
            }
            done_cv_.notify_all();
        }
    }
    std::mutex mu_;
    std::condition_variable cv_, done_cv_;
    std::deque<std::function<void()>> q_;
    uint64_t pushed_ = 0, done_ = 0;
    bool stop_ = false;
    std::thread th_;
};

thread_local int t_simDevice = 0;

class SimPlatform : public Platform {
public:
    PlatKind kind() const override { return PlatKind::SIM; }
    const char *name() const override { return "host-sim"; }
    int DeviceCount() override { return 64; }
    HcclResult SetDevice(int dev) override { t_simDevice = dev; return HCCL_SUCCESS; }
    int CurrentDevice() override { return t_simDevice; }

    size_t Granularity() override { return (size_t)sysconf(_SC_PAGESIZE); }

    HcclResult PhysAlloc(size_t bytes, PhysMem *out) override
    {
        int fd = memfd_create("hccl-sim", MFD_CLOEXEC);
        if (fd < 0) return HCCL_E_SYSCALL;
        if (ftruncate(fd, (off_t)bytes) != 0) { ::close(fd); return HCCL_E_OOM; }
        out->handle = (uint64_t)fd;
        out->bytes = bytes;
        out->imported = false;
        return HCCL_SUCCESS;
    }
    HcclResult PhysExportFd(const PhysMem &m, int *fd) override
    {
        int d = fcntl((int)m.handle, F_DUPFD_CLOEXEC, 0);
        if (d < 0) return HCCL_E_SYSCALL;
        *fd = d;
        return HCCL_SUCCESS;
    }
    HcclResult PhysImportFd(int fd, size_t bytes, PhysMem *out) override
    {
        struct stat st;
        if (fstat(fd, &st) != 0 || (size_t)st.st_size < bytes) return HCCL_E_PARA;
        int d = fcntl(fd, F_DUPFD_CLOEXEC, 0);
        if (d < 0) return HCCL_E_SYSCALL;
        out->handle = (uint64_t)d;
        out->bytes = bytes;
        out->imported = true;
        return HCCL_SUCCESS;
    }
    HcclResult PhysRelease(PhysMem *m) override
    {
        if (m->bytes) ::close((int)m->handle);
        *m = PhysMem();
        return HCCL_SUCCESS;
    }
    HcclResult VaReserve(size_t bytes, void **base) override
    {
        void *p = mmap(nullptr, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
        if (p == MAP_FAILED) return HCCL_E_MEMORY;
        *base = p;
        return HCCL_SUCCESS;
    }
    HcclResult VaFree(void *base, size_t bytes) override { return munmap(base, bytes) == 0 ? HCCL_SUCCESS : HCCL_E_MEMORY; }
    HcclResult Map(void *va, const PhysMem &m, size_t bytes) override
    {
        void *p = mmap(va, bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, (int)m.handle, 0);
        if (p == MAP_FAILED) return HCCL_E_MEMORY;
        std::lock_guard<std::mutex> lk(mu_);
        maps_[(uintptr_t)va] = {bytes, (int)m.handle};
        return HCCL_SUCCESS;
    }
    HcclResult Unmap(void *va, size_t bytes) override
    {
        void *p = mmap(va, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
        std::lock_guard<std::mutex> lk(mu_);
        maps_.erase((uintptr_t)va);
        return p == MAP_FAILED ? HCCL_E_MEMORY : HCCL_SUCCESS;
    }
    HcclResult RetainPhys(void *ptr, PhysMem *out, void **allocBase, size_t *allocBytes) override
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = maps_.upper_bound((uintptr_t)ptr);
        if (it == maps_.begin()) return HCCL_E_NOT_FOUND;
        --it;
        if ((uintptr_t)ptr >= it->first + it->second.bytes) return HCCL_E_NOT_FOUND;
        int d = fcntl(it->second.fd, F_DUPFD_CLOEXEC, 0);
        if (d < 0) return HCCL_E_SYSCALL;
        out->handle = (uint64_t)d;
        out->bytes = it->second.bytes;
        out->imported = true;
        *allocBase = (void *)it->first;
        *allocBytes = it->second.bytes;
        return HCCL_SUCCESS;
    }
    HcclResult IpcExport(void *, std::vector<uint8_t> *, size_t *) override { return HCCL_E_NOT_SUPPORT; }
    HcclResult IpcImport(const std::vector<uint8_t> &, void **) override { return HCCL_E_NOT_SUPPORT; }
    HcclResult IpcClose(void *) override { return HCCL_E_NOT_SUPPORT; }

    bool MulticastSupported() override { return false; }
    HcclResult McCreate(size_t, int, PhysMem *) override { return HCCL_E_NOT_SUPPORT; }
    HcclResult McAddDevice(const PhysMem &) override { return HCCL_E_NOT_SUPPORT; }
    HcclResult McBind(const PhysMem &, size_t, const PhysMem &, size_t) override { return HCCL_E_NOT_SUPPORT; }
    HcclResult McUnbind(const PhysMem &, size_t, size_t) override { return HCCL_E_NOT_SUPPORT; }

    HcclResult DevAlloc(size_t bytes, void **ptr) override
    {
        if (posix_memalign(ptr, 256, bytes ? bytes : 1) != 0) return HCCL_E_OOM;
        return HCCL_SUCCESS;
    }
    HcclResult DevFree(void *ptr) override { free(ptr); return HCCL_SUCCESS; }
    HcclResult HostAlloc(size_t bytes, void **ptr) override { return DevAlloc(bytes, ptr); }
    HcclResult HostFree(void *ptr) override { free(ptr); return HCCL_SUCCESS; }
    HcclResult MemsetSync(void *ptr, int v, size_t bytes) override { memset(ptr, v, bytes); return HCCL_SUCCESS; }
    HcclResult MemcpySync(void *dst, const void *src, size_t bytes) override { memmove(dst, src, bytes); return HCCL_SUCCESS; }

    HcclResult PeekSync(void *hostDst, const void *devSrc, size_t bytes) override { memcpy(hostDst, devSrc, bytes); return HCCL_SUCCESS; }
    HcclResult StreamCreate(Stream *s) override { *s = new SimStream(); return HCCL_SUCCESS; }
    HcclResult StreamDestroy(Stream s) override { delete (SimStream *)s; return HCCL_SUCCESS; }
    HcclResult StreamSync(Stream s) override { if (s) ((SimStream *)s)->Sync(); return HCCL_SUCCESS; }
    HcclResult StreamOrder(Stream before, Stream after) override
    {
        if (!before) return HCCL_SUCCESS;   // inline work has already finished
        SimStream *b = (SimStream *)before;
        uint64_t t = b->Ticket();
        Run(after, [b, t] { b->WaitTicket(t); });
        return HCCL_SUCCESS;
    }
    bool StreamCapturing(Stream) override { return false; }

    HcclResult MemcpyAsync(void *dst, const void *src, size_t bytes, Stream s) override
    {
        Run(s, [=] {
            memmove(dst, src, bytes);
            std::atomic_thread_fence(std::memory_order_release);
        });
        return HCCL_SUCCESS;
    }
    HcclResult ReduceAsync(void *dst, const void *src, uint64_t count, HcclDataType t, HcclReduceOp op, Stream s) override
    {
        if (!DtypeReducible(t)) return HCCL_E_NOT_SUPPORT;
        Run(s, [=] { HostReduce(dst, src, count, t, op); });
        return HCCL_SUCCESS;
    }
    HcclResult ScaleAsync(void *buf, uint64_t count, HcclDataType t, float scale, Stream s) override
    {
        if (t != HCCL_DATA_TYPE_FP32 && t != HCCL_DATA_TYPE_FP64 && t != HCCL_DATA_TYPE_FP16 && t != HCCL_DATA_TYPE_BFP16) return HCCL_E_NOT_SUPPORT;
        Run(s, [=] {
            for (uint64_t i = 0; i < count; ++i) {
                switch (t) {
                    case HCCL_DATA_TYPE_FP32: ((float *)buf)[i] *= scale; break;
                    case HCCL_DATA_TYPE_FP64: ((double *)buf)[i] *= (double)scale; break;
                    case HCCL_DATA_TYPE_FP16: ((uint16_t *)buf)[i] = FloatToHalf(HalfToFloat(((uint16_t *)buf)[i]) * scale); break;
                    default: ((uint16_t *)buf)[i] = FloatToBf16(Bf16ToFloat(((uint16_t *)buf)[i]) * scale); break;
                }
            }
        });
        return HCCL_SUCCESS;
    }
    HcclResult FlagAddAsync(uint64_t *flag, uint64_t v, Stream s) override
    {
        // host-side fault injection for tests: the next g_withhold flag writes of this process are lost
        int left = g_withhold.load();
        while (left > 0 && !g_withhold.compare_exchange_weak(left, left - 1)) {}
        if (left > 0) return HCCL_SUCCESS;
        Run(s, [=] { __atomic_fetch_add(flag, v, __ATOMIC_RELEASE); });
        return HCCL_SUCCESS;
    }
    HcclResult FlagWaitGeAsync(uint64_t *flag, uint64_t expected, uint32_t timeoutMs, const WaitReport &rep, Stream s) override
    {
        Run(s, [=] {
            int64_t deadline = net::NowMs() + (int64_t)timeoutMs;
            uint32_t spins = 0;
            for (;;) {
                uint64_t seen = __atomic_load_n(flag, __ATOMIC_ACQUIRE);
                if (seen >= expected) return;
                if (rep.abortWord && __atomic_load_n(rep.abortWord, __ATOMIC_ACQUIRE)) return;
                if ((++spins & 0x3f) == 0) {
                    if (net::NowMs() >= deadline) {
                        if (rep.status && !__atomic_exchange_n(&rep.status->valid, 1u, __ATOMIC_ACQ_REL)) {
                            rep.status->rank = rep.rank; rep.status->peer = rep.peer; rep.status->kind = rep.kind;
                            rep.status->slot = rep.slot; rep.status->block = 0; rep.status->expected = expected;
                            rep.status->seen = seen; rep.status->seq = rep.seq;
                        }
                        if (rep.abortWord) __atomic_store_n(rep.abortWord, 1u, __ATOMIC_RELEASE);
                        return;
                    }
                    std::this_thread::yield();
                }
            }
        });
        return HCCL_SUCCESS;
    }
    HcclResult HostFuncAsync(std::function<void()> fn, Stream s) override { Run(s, std::move(fn)); return HCCL_SUCCESS; }

private:
    static void Run(Stream s, std::function<void()> fn)
    {
        if (s) ((SimStream *)s)->Push(std::move(fn));
        else fn();
    }
    struct MapRec { size_t bytes; int fd; };
    std::mutex mu_;
    std::map<uintptr_t, MapRec> maps_;
};

}  // namespace

void SimWithholdFlagWrites(int n) { g_withhold.store(n > 0 ? n : 0); }

Platform *SimInstance()
{
    static SimPlatform *p = new SimPlatform();
    return p;
}

}  // namespace hc
