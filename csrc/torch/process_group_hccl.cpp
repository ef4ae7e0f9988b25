// process_group_hccl.cpp - torch.distributed backend "hccl" on top of the C API.
//
// One communicator per backend object, created lazily by the first operator (all ranks call operators in the
// same order, so they meet in HcclCommInitRootInfoConfig; the root info travels through the c10d store).
// CUDA tensors: every operator runs on a dedicated communication stream that first waits for the caller's
// current stream; the returned Work carries an event recorded behind the operator, wait() makes the caller's
// current stream wait for it (no host blocking), and the future is completed under the communication stream so
// that continuations are stream-ordered too.  CPU tensors are served when the library runs on its CPU simulator
// platform (HCCL_SIM=1): operators are synchronous there and the Work is complete on return.
//
// The role matches the reference's torch_npu "hccl" process group, which drives the same C API
// (reference: python/hccl, docs/zh/user_guide: HcclAllReduce & friends called per bucket).
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/chrono.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <optional>
#include <string>
#include <vector>

#include "hccl/hccl.h"
#include "hccl/hccl_comm.h"
#include "hccl/hccl_types.h"

namespace hcomm_torch {

namespace {

void Check(HcclResult r, const char *what)
{
    TORCH_CHECK(r == HCCL_SUCCESS, "hccl backend: ", what, " failed with ", (int)r, " (", HcclGetErrorString(r), ")");
}

HcclDataType DtypeOf(const at::Tensor &t)
{
    switch (t.scalar_type()) {
        case at::kFloat: return HCCL_DATA_TYPE_FP32;
        case at::kHalf: return HCCL_DATA_TYPE_FP16;
        case at::kBFloat16: return HCCL_DATA_TYPE_BFP16;
        case at::kDouble: return HCCL_DATA_TYPE_FP64;
        case at::kChar: return HCCL_DATA_TYPE_INT8;
        case at::kByte: case at::kBool: return HCCL_DATA_TYPE_UINT8;
        case at::kShort: return HCCL_DATA_TYPE_INT16;
        case at::kInt: return HCCL_DATA_TYPE_INT32;
        case at::kLong: return HCCL_DATA_TYPE_INT64;
        default: TORCH_CHECK(false, "hccl backend: dtype ", t.scalar_type(), " is not supported");
    }
}

bool IsFloating(const at::Tensor &t) { return at::isFloatingType(t.scalar_type()); }

// SUM/PROD/MIN/MAX map directly; AVG is a SUM followed by (or fused with) a scale; the rest is refused.
HcclReduceOp ReduceOpOf(const c10d::ReduceOp &op, bool *avg)
{
    *avg = false;
    switch (op.op_) {
        case c10d::ReduceOp::SUM: return HCCL_REDUCE_SUM;
        case c10d::ReduceOp::PRODUCT: return HCCL_REDUCE_PROD;
        case c10d::ReduceOp::MIN: return HCCL_REDUCE_MIN;
        case c10d::ReduceOp::MAX: return HCCL_REDUCE_MAX;
        case c10d::ReduceOp::AVG: *avg = true; return HCCL_REDUCE_SUM;
        default: TORCH_CHECK(false, "hccl backend: reduce op not supported (sum, product, min, max, avg are)");
    }
}

void CheckDense(const at::Tensor &t, const char *what)
{
    TORCH_CHECK(t.is_contiguous(), "hccl backend: ", what, " must be contiguous");
    TORCH_CHECK(!t.is_sparse(), "hccl backend: sparse tensors are not supported");
}

}  // namespace

class WorkHccl : public c10d::Work {
public:
    WorkHccl(int rank, c10d::OpType op, std::vector<at::Tensor> outputs, std::optional<at::Device> device)
        : c10d::Work(rank, op), outputs_(std::move(outputs)), device_(device)
    {
        if (device_ && device_->is_cuda()) {
            future_ = c10::make_intrusive<at::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), std::vector<at::Device>{*device_});
        } else {
            future_ = c10::make_intrusive<at::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
        }
    }
    // Called with the communication stream current, right behind the operator.
    void Seal()
    {
        if (device_ && device_->is_cuda()) {
            done_ = std::make_shared<at::cuda::CUDAEvent>(cudaEventDisableTiming);
            done_->record(c10::cuda::getCurrentCUDAStream(device_->index()));
        }
        future_->markCompleted(at::IValue(outputs_));
    }
    bool isCompleted() override { return !done_ || done_->query(); }
    bool isSuccess() const override { return true; }
    bool wait(std::chrono::milliseconds = kNoTimeout) override
    {
        if (done_) done_->block(c10::cuda::getCurrentCUDAStream(device_->index()));
        return true;
    }
    void synchronize() override { wait(); }
    void blockCurrentStream() override { wait(); }
    std::vector<at::Tensor> result() override { return outputs_; }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

private:
    std::vector<at::Tensor> outputs_;
    std::optional<at::Device> device_;
    std::shared_ptr<at::cuda::CUDAEvent> done_;
    c10::intrusive_ptr<at::ivalue::Future> future_;
};

class ProcessGroupHccl : public c10d::Backend {
public:
    ProcessGroupHccl(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size, std::chrono::milliseconds timeout)
        : c10d::Backend(rank, size), store_(store), timeout_(timeout)
    {
    }
    ~ProcessGroupHccl() override { Shutdown(); }

    const std::string getBackendName() const override { return "hccl"; }
    void setSequenceNumberForGroup() override {}
    uint64_t getSequenceNumberForGroup() override { return seq_; }
    void shutdown() override { Shutdown(); }
    void abort() override { Shutdown(); }

    // Native handle (HcclComm) for code that calls the C API or the fused kernels on the same communicator.
    uint64_t CommHandle(const at::Device &device)
    {
        EnsureComm(device);
        return (uint64_t)(uintptr_t)comm_;
    }

    c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor> &tensors, const c10d::AllreduceOptions &opts) override
    {
        TORCH_CHECK(tensors.size() == 1, "hccl backend: one tensor per allreduce");
        at::Tensor &t = tensors[0];
        CheckDense(t, "allreduce tensor");
        bool avg = false;
        HcclReduceOp op = ReduceOpOf(opts.reduceOp, &avg);
        return Run(c10d::OpType::ALLREDUCE, {t}, {t}, [=](void *stream) mutable {
            if (avg && IsFloating(t))
                Check(HcclAllReduceScaled(t.data_ptr(), t.data_ptr(), (uint64_t)t.numel(), DtypeOf(t), DtypeOf(t), 1.0f / (float)getSize(), comm_, stream), "HcclAllReduceScaled");
            else {
                Check(HcclAllReduce(t.data_ptr(), t.data_ptr(), (uint64_t)t.numel(), DtypeOf(t), op, comm_, stream), "HcclAllReduce");
                if (avg) t.div_(getSize(), "trunc");
            }
        });
    }

    // out = cast(scale * sum over ranks of in): the gradient hook's single-kernel reduction (in and out may alias).
    c10::intrusive_ptr<c10d::Work> AllreduceScaled(at::Tensor in, at::Tensor out, double scale)
    {
        CheckDense(in, "allreduce_scaled input");
        CheckDense(out, "allreduce_scaled output");
        TORCH_CHECK(in.numel() == out.numel(), "hccl backend: allreduce_scaled sizes differ");
        return Run(c10d::OpType::ALLREDUCE, {in}, {out}, [=](void *stream) {
            Check(HcclAllReduceScaled(in.data_ptr(), out.data_ptr(), (uint64_t)in.numel(), DtypeOf(in), DtypeOf(out), (float)scale, comm_, stream), "HcclAllReduceScaled");
        });
    }

    c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor> &tensors, const c10d::AllreduceCoalescedOptions &opts) override
    {
        TORCH_CHECK(!tensors.empty(), "hccl backend: empty tensor list");
        bool avg = false;
        HcclReduceOp op = ReduceOpOf(opts.reduceOp, &avg);
        for (auto &t : tensors) CheckDense(t, "allreduce_coalesced tensor");
        std::vector<at::Tensor> ts = tensors;
        return Run(c10d::OpType::ALLREDUCE_COALESCED, ts, ts, [=](void *stream) {
            for (auto t : ts) {
                if (avg && IsFloating(t))
                    Check(HcclAllReduceScaled(t.data_ptr(), t.data_ptr(), (uint64_t)t.numel(), DtypeOf(t), DtypeOf(t), 1.0f / (float)getSize(), comm_, stream), "HcclAllReduceScaled");
                else {
                    Check(HcclAllReduce(t.data_ptr(), t.data_ptr(), (uint64_t)t.numel(), DtypeOf(t), op, comm_, stream), "HcclAllReduce");
                    if (avg) t.div_(getSize(), "trunc");
                }
            }
        });
    }

    c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor> &tensors, const c10d::BroadcastOptions &opts) override
    {
        TORCH_CHECK(tensors.size() == 1, "hccl backend: one tensor per broadcast");
        at::Tensor t = tensors[0];
        CheckDense(t, "broadcast tensor");
        const uint32_t root = (uint32_t)opts.rootRank;
        return Run(c10d::OpType::BROADCAST, {t}, {t}, [=](void *stream) {
            Check(HcclBroadcast(t.data_ptr(), (uint64_t)t.numel(), DtypeOf(t), root, comm_, stream), "HcclBroadcast");
        });
    }

    c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor> &tensors, const c10d::ReduceOptions &opts) override
    {
        TORCH_CHECK(tensors.size() == 1, "hccl backend: one tensor per reduce");
        at::Tensor t = tensors[0];
        CheckDense(t, "reduce tensor");
        bool avg = false;
        HcclReduceOp op = ReduceOpOf(opts.reduceOp, &avg);
        const uint32_t root = (uint32_t)opts.rootRank;
        return Run(c10d::OpType::REDUCE, {t}, {t}, [=](void *stream) mutable {
            at::Tensor src = t.clone();      // the root's output aliases its input in the c10d contract
            Check(HcclReduce(src.data_ptr(), t.data_ptr(), (uint64_t)t.numel(), DtypeOf(t), op, root, comm_, stream), "HcclReduce");
            Retain(src, stream);
            if (avg && (uint32_t)getRank() == root) t.div_(getSize());
        });
    }

    c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor &out, at::Tensor &in, const c10d::AllgatherOptions &) override
    {
        CheckDense(in, "all_gather input");
        CheckDense(out, "all_gather output");
        TORCH_CHECK(out.numel() == in.numel() * getSize(), "hccl backend: all_gather output must hold world_size inputs");
        at::Tensor i = in, o = out;
        return Run(c10d::OpType::_ALLGATHER_BASE, {i}, {o}, [=](void *stream) {
            Check(HcclAllGather(i.data_ptr(), o.data_ptr(), (uint64_t)i.numel(), DtypeOf(i), comm_, stream), "HcclAllGather");
        });
    }

    c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>> &outs, std::vector<at::Tensor> &ins, const c10d::AllgatherOptions &) override
    {
        TORCH_CHECK(ins.size() == 1 && outs.size() == 1 && (int)outs[0].size() == getSize(), "hccl backend: all_gather takes one input and world_size outputs");
        at::Tensor in = ins[0];
        CheckDense(in, "all_gather input");
        std::vector<at::Tensor> o = outs[0];
        bool sameSize = true;
        for (auto &t : o) sameSize = sameSize && t.numel() == in.numel();
        TORCH_CHECK(sameSize, "hccl backend: all_gather outputs must match the input size");
        return Run(c10d::OpType::ALLGATHER, {in}, o, [=](void *stream) {
            at::Tensor flat = at::empty({(int64_t)getSize(), in.numel()}, in.options());
            Check(HcclAllGather(in.data_ptr(), flat.data_ptr(), (uint64_t)in.numel(), DtypeOf(in), comm_, stream), "HcclAllGather");
            for (int r = 0; r < getSize(); ++r) o[r].copy_(flat[r].view_as(o[r]), true);
            Retain(flat, stream);
        });
    }

    c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor> &outs, std::vector<at::Tensor> &ins, const c10d::AllgatherOptions &) override
    {
        TORCH_CHECK(outs.size() == ins.size() && !ins.empty(), "hccl backend: all_gather_into_tensor_coalesced list sizes differ");
        std::vector<at::Tensor> i = ins, o = outs;
        for (size_t k = 0; k < i.size(); ++k) { CheckDense(i[k], "all_gather input"); CheckDense(o[k], "all_gather output"); }
        return Run(c10d::OpType::COALESCED, i, o, [=](void *stream) {
            for (size_t k = 0; k < i.size(); ++k)
                Check(HcclAllGather(i[k].data_ptr(), o[k].data_ptr(), (uint64_t)i[k].numel(), DtypeOf(i[k]), comm_, stream), "HcclAllGather");
        });
    }

    c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor &out, at::Tensor &in, const c10d::ReduceScatterOptions &opts) override
    {
        CheckDense(in, "reduce_scatter input");
        CheckDense(out, "reduce_scatter output");
        TORCH_CHECK(in.numel() == out.numel() * getSize(), "hccl backend: reduce_scatter input must hold world_size outputs");
        bool avg = false;
        HcclReduceOp op = ReduceOpOf(opts.reduceOp, &avg);
        at::Tensor i = in, o = out;
        return Run(c10d::OpType::_REDUCE_SCATTER_BASE, {i}, {o}, [=](void *stream) mutable {
            Check(HcclReduceScatter(i.data_ptr(), o.data_ptr(), (uint64_t)o.numel(), DtypeOf(i), op, comm_, stream), "HcclReduceScatter");
            if (avg) o.div_(getSize());
        });
    }

    c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor> &outs, std::vector<std::vector<at::Tensor>> &ins, const c10d::ReduceScatterOptions &opts) override
    {
        TORCH_CHECK(outs.size() == 1 && ins.size() == 1 && (int)ins[0].size() == getSize(), "hccl backend: reduce_scatter takes world_size inputs and one output");
        at::Tensor out = outs[0];
        CheckDense(out, "reduce_scatter output");
        std::vector<at::Tensor> i = ins[0];
        bool avg = false;
        HcclReduceOp op = ReduceOpOf(opts.reduceOp, &avg);
        return Run(c10d::OpType::REDUCE_SCATTER, i, {out}, [=](void *stream) mutable {
            at::Tensor flat = at::empty({(int64_t)getSize(), out.numel()}, out.options());
            for (int r = 0; r < getSize(); ++r) flat[r].copy_(i[r].reshape({-1}), true);
            Check(HcclReduceScatter(flat.data_ptr(), out.data_ptr(), (uint64_t)out.numel(), DtypeOf(out), op, comm_, stream), "HcclReduceScatter");
            if (avg) out.div_(getSize());
            Retain(flat, stream);
        });
    }

    c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor> &outs, std::vector<at::Tensor> &ins, const c10d::ReduceScatterOptions &opts) override
    {
        TORCH_CHECK(outs.size() == ins.size() && !ins.empty(), "hccl backend: reduce_scatter_tensor_coalesced list sizes differ");
        bool avg = false;
        HcclReduceOp op = ReduceOpOf(opts.reduceOp, &avg);
        std::vector<at::Tensor> i = ins, o = outs;
        for (size_t k = 0; k < i.size(); ++k) { CheckDense(i[k], "reduce_scatter input"); CheckDense(o[k], "reduce_scatter output"); }
        return Run(c10d::OpType::COALESCED, i, o, [=](void *stream) mutable {
            for (size_t k = 0; k < i.size(); ++k) {
                Check(HcclReduceScatter(i[k].data_ptr(), o[k].data_ptr(), (uint64_t)o[k].numel(), DtypeOf(i[k]), op, comm_, stream), "HcclReduceScatter");
                if (avg) o[k].div_(getSize());
            }
        });
    }

    c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor &out, at::Tensor &in, std::vector<int64_t> &outSplits, std::vector<int64_t> &inSplits,
                                                 const c10d::AllToAllOptions &) override
    {
        CheckDense(in, "all_to_all input");
        CheckDense(out, "all_to_all output");
        at::Tensor i = in, o = out;
        const int n = getSize();
        if (outSplits.empty() && inSplits.empty()) {
            TORCH_CHECK(i.numel() % n == 0 && o.numel() == i.numel(), "hccl backend: all_to_all_single without splits needs equal, divisible sizes");
            return Run(c10d::OpType::ALLTOALL_BASE, {i}, {o}, [=](void *stream) {
                const uint64_t per = (uint64_t)(i.numel() / n);
                Check(HcclAlltoAll(i.data_ptr(), per, DtypeOf(i), o.data_ptr(), per, DtypeOf(o), comm_, stream), "HcclAlltoAll");
            });
        }
        TORCH_CHECK((int)outSplits.size() == n && (int)inSplits.size() == n, "hccl backend: split lists must have world_size entries");
        const int64_t inRow = i.dim() ? i.numel() / std::max<int64_t>(1, i.size(0)) : 1, outRow = o.dim() ? o.numel() / std::max<int64_t>(1, o.size(0)) : 1;
        std::vector<uint64_t> sc(n), sd(n), rc(n), rd(n);
        uint64_t so = 0, ro = 0;
        for (int r = 0; r < n; ++r) {
            sc[r] = (uint64_t)(inSplits[r] * inRow); sd[r] = so; so += sc[r];
            rc[r] = (uint64_t)(outSplits[r] * outRow); rd[r] = ro; ro += rc[r];
        }
        return Run(c10d::OpType::ALLTOALL_BASE, {i}, {o}, [=](void *stream) {
            Check(HcclAlltoAllV(i.data_ptr(), sc.data(), sd.data(), DtypeOf(i), o.data_ptr(), rc.data(), rd.data(), DtypeOf(o), comm_, stream), "HcclAlltoAllV");
        });
    }

    c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor> &outs, std::vector<at::Tensor> &ins, const c10d::AllToAllOptions &) override
    {
        const int n = getSize();
        TORCH_CHECK((int)outs.size() == n && (int)ins.size() == n, "hccl backend: all_to_all takes world_size tensors each way");
        std::vector<at::Tensor> i = ins, o = outs;
        return Run(c10d::OpType::ALLTOALL, i, o, [=](void *stream) {
            std::vector<uint64_t> sc(n), sd(n), rc(n), rd(n);
            uint64_t so = 0, ro = 0;
            for (int r = 0; r < n; ++r) {
                sc[r] = (uint64_t)i[r].numel(); sd[r] = so; so += sc[r];
                rc[r] = (uint64_t)o[r].numel(); rd[r] = ro; ro += rc[r];
            }
            at::Tensor sflat = at::empty({(int64_t)std::max<uint64_t>(so, 1)}, i[0].options()), rflat = at::empty({(int64_t)std::max<uint64_t>(ro, 1)}, o[0].options());
            for (int r = 0; r < n; ++r)
                if (sc[r]) sflat.narrow(0, (int64_t)sd[r], (int64_t)sc[r]).copy_(i[r].reshape({-1}), true);
            Check(HcclAlltoAllV(sflat.data_ptr(), sc.data(), sd.data(), DtypeOf(sflat), rflat.data_ptr(), rc.data(), rd.data(), DtypeOf(rflat), comm_, stream), "HcclAlltoAllV");
            for (int r = 0; r < n; ++r)
                if (rc[r]) o[r].copy_(rflat.narrow(0, (int64_t)rd[r], (int64_t)rc[r]).view_as(o[r]), true);
            Retain(sflat, stream);
            Retain(rflat, stream);
        });
    }

    c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>> &outs, std::vector<at::Tensor> &ins, const c10d::GatherOptions &opts) override
    {
        TORCH_CHECK(ins.size() == 1, "hccl backend: one input per gather");
        at::Tensor in = ins[0];
        CheckDense(in, "gather input");
        const uint32_t root = (uint32_t)opts.rootRank;
        std::vector<at::Tensor> o;
        if ((uint32_t)getRank() == root) {
            TORCH_CHECK(outs.size() == 1 && (int)outs[0].size() == getSize(), "hccl backend: the gather root passes world_size outputs");
            o = outs[0];
        }
        return Run(c10d::OpType::GATHER, {in}, o, [=](void *stream) {
            at::Tensor flat = at::empty({(int64_t)getSize(), in.numel()}, in.options());
            Check(HcclGather(in.data_ptr(), flat.data_ptr(), (uint64_t)in.numel(), DtypeOf(in), root, comm_, stream), "HcclGather");
            for (size_t r = 0; r < o.size(); ++r) o[r].copy_(flat[(int64_t)r].view_as(o[r]), true);
            Retain(flat, stream);
        });
    }

    c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor> &outs, std::vector<std::vector<at::Tensor>> &ins, const c10d::ScatterOptions &opts) override
    {
        TORCH_CHECK(outs.size() == 1, "hccl backend: one output per scatter");
        at::Tensor out = outs[0];
        CheckDense(out, "scatter output");
        const uint32_t root = (uint32_t)opts.rootRank;
        std::vector<at::Tensor> i;
        if ((uint32_t)getRank() == root) {
            TORCH_CHECK(ins.size() == 1 && (int)ins[0].size() == getSize(), "hccl backend: the scatter root passes world_size inputs");
            i = ins[0];
        }
        return Run(c10d::OpType::SCATTER, {out}, {out}, [=](void *stream) mutable {
            at::Tensor flat = at::empty({(int64_t)getSize(), out.numel()}, out.options());
            for (size_t r = 0; r < i.size(); ++r) flat[(int64_t)r].copy_(i[r].reshape({-1}), true);
            Check(HcclScatter(flat.data_ptr(), out.data_ptr(), (uint64_t)out.numel(), DtypeOf(out), root, comm_, stream), "HcclScatter");
            Retain(flat, stream);
        });
    }

    c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor> &tensors, int dst, int) override
    {
        TORCH_CHECK(tensors.size() == 1, "hccl backend: one tensor per send");
        at::Tensor t = tensors[0];
        CheckDense(t, "send tensor");
        return Run(c10d::OpType::SEND, {t}, {}, [=](void *stream) {
            Check(HcclSend(t.data_ptr(), (uint64_t)t.numel(), DtypeOf(t), (uint32_t)dst, comm_, stream), "HcclSend");
        });
    }

    c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor> &tensors, int src, int) override
    {
        TORCH_CHECK(tensors.size() == 1, "hccl backend: one tensor per recv");
        at::Tensor t = tensors[0];
        CheckDense(t, "recv tensor");
        return Run(c10d::OpType::RECV, {t}, {t}, [=](void *stream) {
            Check(HcclRecv(t.data_ptr(), (uint64_t)t.numel(), DtypeOf(t), (uint32_t)src, comm_, stream), "HcclRecv");
        });
    }

    c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions &opts) override
    {
        // a barrier carries no tensor: it runs on the device of the last operator (or the one named in the options)
        std::optional<at::Device> dev = lastDevice_;
        if (!opts.device_ids.empty()) dev = at::Device(at::kCUDA, (c10::DeviceIndex)opts.device_ids[0]);
        if (opts.device.has_value()) dev = *opts.device;
        if (!dev) dev = UsesSimulator() ? at::Device(at::kCPU) : at::Device(at::kCUDA, c10::cuda::current_device());
        auto work = RunOn(*dev, c10d::OpType::BARRIER, {}, {}, [=](void *stream) { Check(HcclBarrier(comm_, stream), "HcclBarrier"); });
        if (dev->is_cuda()) {
            c10::cuda::CUDAGuard g(*dev);
            C10_CUDA_CHECK(cudaStreamSynchronize(CommStream(*dev)));   // c10d barriers block the host
        }
        return work;
    }

private:
    static bool UsesSimulator()
    {
        const char *s = std::getenv("HCCL_SIM");
        return s && *s && std::strcmp(s, "0") != 0;
    }

    void Shutdown()
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (comm_) {
            if (commDevice_ && commDevice_->is_cuda()) {
                c10::cuda::CUDAGuard g(*commDevice_);
                cudaDeviceSynchronize();
            }
            HcclCommDestroy(comm_);
            comm_ = nullptr;
        }
    }

    void EnsureComm(const at::Device &device)
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (comm_) {
            TORCH_CHECK(*commDevice_ == device, "hccl backend: this process group is bound to ", *commDevice_, ", got a tensor on ", device);
            return;
        }
        TORCH_CHECK(device.is_cuda() || UsesSimulator(), "hccl backend: CPU tensors are served only on the simulator platform (HCCL_SIM=1)");
        const std::string key = "hccl/rootinfo/" + groupTag_;
        HcclRootInfo info;
        if (getRank() == 0) {
            Check(HcclGetRootInfo(&info), "HcclGetRootInfo");
            std::vector<uint8_t> bytes((const uint8_t *)&info, (const uint8_t *)&info + sizeof(info));
            store_->set(key, bytes);
        } else {
            std::vector<uint8_t> bytes = store_->get(key);
            TORCH_CHECK(bytes.size() == sizeof(info), "hccl backend: malformed root info in the store");
            std::memcpy(&info, bytes.data(), sizeof(info));
        }
        HcclCommConfig cfg;
        HcclCommConfigInit(&cfg);
        if (const char *mb = std::getenv("HCOMM_TORCH_BUFFER_MB")) cfg.hcclBufferSize = (uint32_t)std::max(1, std::atoi(mb));
        std::optional<c10::cuda::CUDAGuard> guard;
        if (device.is_cuda()) guard.emplace(device);
        Check(HcclCommInitRootInfoConfig((uint32_t)getSize(), &info, (uint32_t)getRank(), &cfg, &comm_), "HcclCommInitRootInfoConfig");
        commDevice_ = device;
    }

    cudaStream_t CommStream(const at::Device &device)
    {
        if (!commStream_) commStream_ = c10::cuda::getStreamFromPool(/*isHighPriority=*/true, device.index());
        return commStream_->stream();
    }

    // Keeps a temporary alive until the communication stream has passed the work that uses it.
    static void Retain(const at::Tensor &t, void *stream)
    {
        if (t.is_cuda() && stream) {
            c10::cuda::CUDAStream s = c10::cuda::getCurrentCUDAStream(t.device().index());
            c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), s);
        }
    }

    c10::intrusive_ptr<c10d::Work> Run(c10d::OpType op, const std::vector<at::Tensor> &inputs, const std::vector<at::Tensor> &outputs,
                                       const std::function<void(void *)> &fn)
    {
        const at::Tensor &first = !inputs.empty() ? inputs[0] : outputs[0];
        for (auto &t : inputs) TORCH_CHECK(t.device() == first.device(), "hccl backend: tensors of one operator must share a device");
        for (auto &t : outputs) TORCH_CHECK(t.device() == first.device(), "hccl backend: tensors of one operator must share a device");
        return RunOn(first.device(), op, inputs, outputs, fn);
    }

    c10::intrusive_ptr<c10d::Work> RunOn(const at::Device &device, c10d::OpType op, const std::vector<at::Tensor> &inputs,
                                         const std::vector<at::Tensor> &outputs, const std::function<void(void *)> &fn)
    {
        EnsureComm(device);
        lastDevice_ = device;
        ++seq_;
        auto work = c10::make_intrusive<WorkHccl>(getRank(), op, outputs, device);
        if (!device.is_cuda()) {
            fn(nullptr);
            work->Seal();
            return work;
        }
        c10::cuda::CUDAGuard dg(device);
        c10::cuda::CUDAStream cur = c10::cuda::getCurrentCUDAStream(device.index());
        cudaStream_t cs = CommStream(device);
        at::cuda::CUDAEvent ready(cudaEventDisableTiming);
        ready.record(cur);
        ready.block(*commStream_);
        for (auto &t : inputs) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), *commStream_);
        for (auto &t : outputs) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), *commStream_);
        {
            c10::cuda::CUDAStreamGuard sg(*commStream_);    // helper tensor ops (copies, div_) land on the communication stream
            fn((void *)cs);
            work->Seal();
        }
        return work;
    }

    c10::intrusive_ptr<c10d::Store> store_;
    std::chrono::milliseconds timeout_;
    std::mutex mu_;
    HcclComm comm_ = nullptr;
    std::optional<at::Device> commDevice_, lastDevice_;
    std::optional<c10::cuda::CUDAStream> commStream_;
    std::string groupTag_ = "0";
    uint64_t seq_ = 0;

public:
    void SetGroupTag(const std::string &t) { groupTag_ = t; }
};

c10::intrusive_ptr<c10d::Backend> CreateBackend(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size, const std::chrono::milliseconds &timeout,
                                                const std::string &tag)
{
    auto pg = c10::make_intrusive<ProcessGroupHccl>(store, rank, size, timeout);
    pg->SetGroupTag(tag);
    return pg;
}

}  // namespace hcomm_torch

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    using hcomm_torch::ProcessGroupHccl;
    py::class_<ProcessGroupHccl, c10d::Backend, c10::intrusive_ptr<ProcessGroupHccl>>(m, "ProcessGroupHCCL")
        .def("allreduce_scaled", &ProcessGroupHccl::AllreduceScaled, py::arg("input"), py::arg("output"), py::arg("scale"),
             py::call_guard<py::gil_scoped_release>())
        .def("comm_handle", &ProcessGroupHccl::CommHandle, py::arg("device"));
    m.def("create_backend", &hcomm_torch::CreateBackend, py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"), py::arg("tag") = "0");
}
