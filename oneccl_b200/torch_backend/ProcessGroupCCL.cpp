// torch.distributed backend "ccl": a c10d::Backend on top of the ccl:: C++ API.
//
// The reference repository does not contain its PyTorch binding (its README
// points at an external project); this file is the framework layer of this
// library.  Bootstrap: rank 0 starts the library's KVS and publishes its address
// in the torch Store the process group was created with; every rank then builds
// a ccl::communicator.  CPU tensors take the scheduler path; CUDA tensors run
// the device kernels on a dedicated communication stream per device (the
// current stream is joined in at launch and at wait(), the NCCL backend's
// stream semantics), so collectives overlap with the caller's compute.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/extension.h>
#include <pybind11/chrono.h>

#include <map>
#include <thread>
#include <mutex>

#include "oneapi/ccl.hpp"

namespace c10d {

namespace {

ccl::datatype to_ccl_dtype(at::ScalarType t) {
    switch (t) {
        case at::kChar: return ccl::datatype::int8;
        case at::kByte:
        case at::kBool: return ccl::datatype::uint8;
        case at::kShort: return ccl::datatype::int16;
        case at::kInt: return ccl::datatype::int32;
        case at::kLong: return ccl::datatype::int64;
        case at::kHalf: return ccl::datatype::float16;
        case at::kFloat: return ccl::datatype::float32;
        case at::kDouble: return ccl::datatype::float64;
        case at::kBFloat16: return ccl::datatype::bfloat16;
        case at::kUInt16: return ccl::datatype::uint16;
        case at::kUInt32: return ccl::datatype::uint32;
        case at::kUInt64: return ccl::datatype::uint64;
        default: TORCH_CHECK(false, "ccl backend: unsupported dtype ", t);
    }
}

ccl::reduction to_ccl_op(const ReduceOp& op) {
    switch (op.op_) {
        case ReduceOp::SUM:
        case ReduceOp::AVG: return ccl::reduction::sum;
        case ReduceOp::PRODUCT: return ccl::reduction::prod;
        case ReduceOp::MIN: return ccl::reduction::min;
        case ReduceOp::MAX: return ccl::reduction::max;
        default: TORCH_CHECK(false, "ccl backend: unsupported reduce op");
    }
}

// the library carries its own CUDA runtime whose current device is per thread
void sync_device(const at::Tensor& t) {
    if (t.is_cuda())
        cudaSetDevice(t.device().index());
}

class WorkCCL : public Work {
public:
    WorkCCL(OpType op, std::vector<at::Tensor> outputs, std::vector<at::Tensor> keep)
            : Work(-1, op), outputs_(std::move(outputs)), keep_(std::move(keep)) {}
    void add(ccl::event e) { events_.push_back(std::move(e)); }
    void set_cuda(c10::DeviceIndex dev, cudaEvent_t done) {
        cuda_ = true;
        device_ = dev;
        done_ = done;
    }
    // Host work: a plain future.  Device work: a device-aware future completed while the
    // communication stream is current, so that it records an event there and callbacks
    // (DDP's bucket post-processing) are ordered after the collective.
    void make_future(bool cuda, c10::DeviceIndex dev) {
        auto type = c10::ListType::create(c10::TensorType::get());
        if (cuda)
            future_ = c10::make_intrusive<c10::ivalue::Future>(
                type, std::vector<c10::Device>{ c10::Device(c10::kCUDA, dev) });
        else
            future_ = c10::make_intrusive<c10::ivalue::Future>(type);
    }
    void mark_launched() {
        if (cuda_)
            future_->markCompleted(c10::IValue(outputs_));
    }
    ~WorkCCL() override {
        if (done_)
            cudaEventDestroy(done_);
    }
    bool isCompleted() override {
        if (cuda_) {
            if (cudaEventQuery(done_) != cudaSuccess) {
                (void)cudaGetLastError();
                return false;
            }
            check_device();
            return true;
        }
        for (auto& e : events_)
            if (!e.test())
                return false;
        return true;
    }
    // a device-side failure (bounded wait ran out, abort, argument mismatch) is recorded in the communicator's
    // status word; once the event has fired it is turned into this Work's exception
    void check_device() {
        try {
            for (auto& e : events_)
                (void)e.test();
        }
        catch (...) {
            std::lock_guard<std::mutex> lk(mutex_);
            if (!exception_)
                exception_ = std::current_exception();
        }
    }
    bool isSuccess() const override { return !exception_; }
    bool wait(std::chrono::milliseconds timeout = kNoTimeout) override {
        if (cuda_) {
            if (timeout != kNoTimeout) {
                // a caller that gives a time limit wants to know on the host: poll the event until then
                const auto deadline = std::chrono::steady_clock::now() + timeout;
                while (cudaEventQuery(done_) != cudaSuccess) {
                    (void)cudaGetLastError();
                    TORCH_CHECK(std::chrono::steady_clock::now() < deadline, "ccl backend: operation timed out after ",
                                timeout.count(), " ms");
                    std::this_thread::yield();
                }
                check_device();
                if (exception_)
                    std::rethrow_exception(exception_);
            }
            // stream semantics: later work on the caller's stream is ordered after the collective
            auto cur = c10::cuda::getCurrentCUDAStream(device_);
            C10_CUDA_CHECK(cudaStreamWaitEvent(cur.stream(), done_, 0));
            return true;
        }
        for (auto& e : events_)
            e.wait();
        if (!future_->completed())
            future_->markCompleted(c10::IValue(outputs_));
        return true;
    }
    void synchronize() override { wait(); }
    std::vector<at::Tensor> result() override { return outputs_; }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override {
        if (!cuda_ && !future_->completed()) {
            // host operations: complete the future from the caller's side
            for (auto& e : events_)
                e.wait();
            future_->markCompleted(c10::IValue(outputs_));
        }
        return future_;
    }

private:
    std::vector<ccl::event> events_;
    std::vector<at::Tensor> outputs_, keep_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
    bool cuda_ = false;
    c10::DeviceIndex device_ = 0;
    cudaEvent_t done_ = nullptr;
};

// what endCoalescing hands back: complete when every operation issued inside the batch is
class CoalescedWorkCCL : public Work {
public:
    explicit CoalescedWorkCCL(std::vector<c10::intrusive_ptr<Work>> parts)
            : Work(-1, OpType::COALESCED), parts_(std::move(parts)) {}
    bool isCompleted() override {
        for (auto& p : parts_)
            if (!p->isCompleted())
                return false;
        return true;
    }
    bool isSuccess() const override { return true; }
    bool wait(std::chrono::milliseconds timeout = kNoTimeout) override {
        for (auto& p : parts_)
            p->wait(timeout);
        return true;
    }
    void synchronize() override { wait(); }
    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override {
        // the parts' futures carry the device events; the batch as a whole completes on the host side
        auto f = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
        wait();
        f->markCompleted(c10::IValue(std::vector<at::Tensor>{}));
        return f;
    }

private:
    std::vector<c10::intrusive_ptr<Work>> parts_;
};

std::atomic<int> pg_counter{ 0 };

} // namespace

class ProcessGroupCCL : public Backend {
public:
    ProcessGroupCCL(const c10::intrusive_ptr<Store>& store, int rank, int size) : Backend(rank, size), store_(store) {
        ccl::init();
        const std::string key = "ccl_kvs_addr_" + std::to_string(pg_counter++);
        std::shared_ptr<ccl::kvs> kvs;
        if (rank == 0) {
            kvs = ccl::create_main_kvs();
            auto addr = kvs->get_address();
            store->set(key, std::vector<uint8_t>(addr.begin(), addr.end()));
        }
        else {
            auto bytes = store->get(key);
            ccl::kvs::address_type addr;
            addr.fill(0);
            std::copy_n(bytes.begin(), std::min(bytes.size(), addr.size()), addr.begin());
            kvs = ccl::create_kvs(addr);
        }
        comm_ = ccl::create_communicator(size, rank, kvs);
    }

    ~ProcessGroupCCL() override {
        for (auto& kv : streams_)
            cudaStreamSynchronize(kv.second);
    }

    const std::string getBackendName() const override { return "ccl"; }

    // ---- helpers --------------------------------------------------------------------------
    struct launch_ctx {
        bool cuda = false;
        c10::DeviceIndex dev = 0;
        cudaStream_t comm_stream = nullptr;
        ccl::stream stream;
    };

    launch_ctx begin(const at::Tensor& t) {
        launch_ctx c;
        if (!t.is_cuda())
            return c;
        c.cuda = true;
        c.dev = t.device().index();
        sync_device(t);
        {
            std::lock_guard<std::mutex> lk(mu_);
            auto it = streams_.find(c.dev);
            if (it == streams_.end()) {
                c10::cuda::CUDAGuard g(c.dev);
                // highest priority: a bucket allreduce launched during backward runs beside the GEMM that is on
                // the GPU instead of waiting behind all of its waves
                cudaStream_t s;
                int lo = 0, hi = 0;
                C10_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
                C10_CUDA_CHECK(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, hi));
                it = streams_.emplace(c.dev, s).first;
            }
            c.comm_stream = it->second;
        }
        // the communication stream joins the caller's stream
        auto cur = c10::cuda::getCurrentCUDAStream(c.dev);
        cudaEvent_t ev;
        C10_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        C10_CUDA_CHECK(cudaEventRecord(ev, cur.stream()));
        C10_CUDA_CHECK(cudaStreamWaitEvent(c.comm_stream, ev, 0));
        C10_CUDA_CHECK(cudaEventDestroy(ev));
        c.stream = ccl::create_stream((CUstream_st*)c.comm_stream);
        return c;
    }

    c10::intrusive_ptr<Work> finish(launch_ctx& c, c10::intrusive_ptr<WorkCCL> w) {
        w->make_future(c.cuda, c.dev);
        if (c.cuda) {
            cudaEvent_t done;
            C10_CUDA_CHECK(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
            C10_CUDA_CHECK(cudaEventRecord(done, c.comm_stream));
            w->set_cuda(c.dev, done);
            c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(c.comm_stream, c.dev));
            w->mark_launched();
        }
        if (coalescing_)
            batch_.push_back(w);
        return w;
    }

    static at::Tensor contig(const at::Tensor& t) { return t.is_contiguous() ? t : t.contiguous(); }

    // ---- collectives ------------------------------------------------------------------------
    c10::intrusive_ptr<Work> allreduce(std::vector<at::Tensor>& tensors, const AllreduceOptions& opts) override {
        TORCH_CHECK(tensors.size() == 1, "ccl backend: one tensor per rank");
        at::Tensor t = contig(tensors[0]);
        auto c = begin(t);
        auto w = c10::make_intrusive<WorkCCL>(OpType::ALLREDUCE, tensors, std::vector<at::Tensor>{ t });
        ccl::allreduce_attr attr;
        const bool avg = opts.reduceOp.op_ == ReduceOp::AVG;
        TORCH_CHECK(!avg || at::isFloatingType(t.scalar_type()), "ccl backend: ReduceOp.AVG needs a floating-point tensor");
        if (avg && c.cuda)
            attr.set<ccl::device_attr_ext_id::scale>(1.0f / (float)getSize());
        if (c.cuda)
            w->add(ccl::allreduce(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()),
                                  to_ccl_op(opts.reduceOp), comm_, c.stream, attr));
        else {
            ccl::allreduce(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()),
                           to_ccl_op(opts.reduceOp), comm_, attr)
                .wait();
            if (avg)
                t.div_(getSize());
        }
        if (!t.is_same(tensors[0])) {
            copy_back(c, tensors[0], t);
        }
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                 const AllreduceCoalescedOptions& opts) override {
        TORCH_CHECK(!tensors.empty(), "ccl backend: empty tensor list");
        bool one_kind = tensors[0].is_cuda();
        for (auto& t : tensors)
            one_kind = one_kind && t.is_cuda() && t.device() == tensors[0].device() &&
                       t.scalar_type() == tensors[0].scalar_type() && t.is_contiguous();
        if (one_kind) {
            // CUDA tensors of one dtype: ONE fused operation (pack kernel, one allreduce on a buffer of the
            // symmetric heap, unpack kernel) and one Work that covers every tensor
            auto c = begin(tensors[0]);
            auto w = c10::make_intrusive<WorkCCL>(OpType::ALLREDUCE_COALESCED, tensors, tensors);
            ccl::allreduce_attr attr;
            if (opts.reduceOp.op_ == ReduceOp::AVG)
                attr.set<ccl::device_attr_ext_id::scale>(1.0f / (float)getSize());
            std::vector<void*> bufs;
            std::vector<size_t> counts;
            for (auto& t : tensors) {
                bufs.push_back(t.data_ptr());
                counts.push_back((size_t)t.numel());
            }
            w->add(ccl::preview::allreduce_coalesced(bufs, counts, to_ccl_dtype(tensors[0].scalar_type()),
                                                     to_ccl_op(opts.reduceOp), comm_, c.stream, attr));
            return finish(c, w);
        }
        // mixed lists: one operation per tensor; the returned Work completes when all of them have
        std::vector<c10::intrusive_ptr<Work>> parts;
        AllreduceOptions o;
        o.reduceOp = opts.reduceOp;
        for (auto& t : tensors) {
            std::vector<at::Tensor> one{ t };
            parts.push_back(allreduce(one, o));
        }
        return c10::make_intrusive<CoalescedWorkCCL>(std::move(parts));
    }

    c10::intrusive_ptr<Work> broadcast(std::vector<at::Tensor>& tensors, const BroadcastOptions& opts) override {
        TORCH_CHECK(tensors.size() == 1, "ccl backend: one tensor per rank");
        at::Tensor t = contig(tensors[0]);
        auto c = begin(t);
        auto w = c10::make_intrusive<WorkCCL>(OpType::BROADCAST, tensors, std::vector<at::Tensor>{ t });
        const int root = (int)opts.rootRank;
        if (c.cuda)
            w->add(ccl::broadcast(t.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()), root, comm_,
                                  c.stream));
        else
            ccl::broadcast(t.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()), root, comm_).wait();
        if (!t.is_same(tensors[0]))
            copy_back(c, tensors[0], t);
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> reduce(std::vector<at::Tensor>& tensors, const ReduceOptions& opts) override {
        TORCH_CHECK(tensors.size() == 1, "ccl backend: one tensor per rank");
        at::Tensor t = contig(tensors[0]);
        auto c = begin(t);
        auto w = c10::make_intrusive<WorkCCL>(OpType::REDUCE, tensors, std::vector<at::Tensor>{ t });
        const int root = (int)opts.rootRank;
        at::Tensor out = getRank() == root ? at::empty_like(t) : t;
        if (c.cuda) {
            c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(c.comm_stream, c.dev));
            w->add(ccl::reduce(t.data_ptr(), out.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()),
                               to_ccl_op(opts.reduceOp), root, comm_, c.stream));
            if (getRank() == root)
                tensors[0].copy_(out, true);
        }
        else {
            ccl::reduce(t.data_ptr(), out.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()),
                        to_ccl_op(opts.reduceOp), root, comm_)
                .wait();
            if (getRank() == root)
                tensors[0].copy_(out);
        }
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                             const AllgatherOptions& = AllgatherOptions()) override {
        TORCH_CHECK(output.is_contiguous(), "ccl backend: output must be contiguous");
        at::Tensor in = contig(input);
        auto c = begin(in);
        auto w = c10::make_intrusive<WorkCCL>(OpType::_ALLGATHER_BASE, std::vector<at::Tensor>{ output },
                                              std::vector<at::Tensor>{ in });
        if (c.cuda)
            w->add(ccl::allgather(in.data_ptr(), output.data_ptr(), (size_t)in.numel(),
                                  to_ccl_dtype(in.scalar_type()), comm_, c.stream));
        else
            w->add(ccl::allgather(in.data_ptr(), output.data_ptr(), (size_t)in.numel(),
                                  to_ccl_dtype(in.scalar_type()), comm_));
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                       const AllgatherOptions& = AllgatherOptions()) override {
        TORCH_CHECK(inputs.size() == 1 && outputs.size() == 1, "ccl backend: one tensor per rank");
        at::Tensor in = contig(inputs[0]);
        auto& outs = outputs[0];
        TORCH_CHECK((int)outs.size() == getSize(), "allgather: need one output per rank");
        auto c = begin(in);
        // gather into one flat buffer, then scatter into the list (sizes may differ per rank)
        std::vector<size_t> counts;
        size_t total = 0;
        for (auto& o : outs) {
            counts.push_back((size_t)o.numel());
            total += (size_t)o.numel();
        }
        at::Tensor flat;
        std::vector<at::Tensor> keep{ in };
        auto w = c10::make_intrusive<WorkCCL>(OpType::ALLGATHER, outs, keep);
        if (c.cuda) {
            c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(c.comm_stream, c.dev));
            flat = at::empty({ (int64_t)total }, in.options());
            w->add(ccl::allgatherv(in.data_ptr(), (size_t)in.numel(), flat.data_ptr(), counts,
                                   to_ccl_dtype(in.scalar_type()), comm_, c.stream));
            size_t off = 0;
            for (size_t i = 0; i < outs.size(); i++) {
                outs[i].copy_(flat.narrow(0, (int64_t)off, (int64_t)counts[i]).view_as(outs[i]), true);
                off += counts[i];
            }
        }
        else {
            flat = at::empty({ (int64_t)total }, in.options());
            ccl::allgatherv(in.data_ptr(), (size_t)in.numel(), flat.data_ptr(), counts,
                            to_ccl_dtype(in.scalar_type()), comm_)
                .wait();
            size_t off = 0;
            for (size_t i = 0; i < outs.size(); i++) {
                outs[i].copy_(flat.narrow(0, (int64_t)off, (int64_t)counts[i]).view_as(outs[i]));
                off += counts[i];
            }
        }
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> allgather_coalesced(std::vector<std::vector<at::Tensor>>& output_lists,
                                                 std::vector<at::Tensor>& inputs,
                                                 const AllgatherOptions& opts = AllgatherOptions()) override {
        TORCH_CHECK(output_lists.size() == inputs.size(), "ccl backend: one output list per input tensor");
        std::vector<c10::intrusive_ptr<Work>> parts;
        for (size_t i = 0; i < inputs.size(); i++) {
            std::vector<std::vector<at::Tensor>> outs{ output_lists[i] };
            std::vector<at::Tensor> in{ inputs[i] };
            parts.push_back(allgather(outs, in, opts));
        }
        return c10::make_intrusive<CoalescedWorkCCL>(std::move(parts));
    }

    c10::intrusive_ptr<Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outputs,
                                                             std::vector<at::Tensor>& inputs,
                                                             const AllgatherOptions& opts) override {
        c10::intrusive_ptr<Work> last;
        for (size_t i = 0; i < inputs.size(); i++)
            last = _allgather_base(outputs[i], inputs[i], opts);
        return last;
    }

    c10::intrusive_ptr<Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                  const ReduceScatterOptions& opts) override {
        TORCH_CHECK(output.is_contiguous(), "ccl backend: output must be contiguous");
        at::Tensor in = contig(input);
        auto c = begin(in);
        auto w = c10::make_intrusive<WorkCCL>(OpType::_REDUCE_SCATTER_BASE, std::vector<at::Tensor>{ output },
                                              std::vector<at::Tensor>{ in });
        ccl::reduce_scatter_attr attr;
        const bool avg = opts.reduceOp.op_ == ReduceOp::AVG;
        TORCH_CHECK(!avg || at::isFloatingType(in.scalar_type()), "ccl backend: ReduceOp.AVG needs a floating-point tensor");
        if (avg && c.cuda)
            attr.set<ccl::device_attr_ext_id::scale>(1.0f / (float)getSize());
        if (c.cuda)
            w->add(ccl::reduce_scatter(in.data_ptr(), output.data_ptr(), (size_t)output.numel(),
                                       to_ccl_dtype(in.scalar_type()), to_ccl_op(opts.reduceOp), comm_, c.stream,
                                       attr));
        else {
            ccl::reduce_scatter(in.data_ptr(), output.data_ptr(), (size_t)output.numel(),
                                to_ccl_dtype(in.scalar_type()), to_ccl_op(opts.reduceOp), comm_, attr)
                .wait();
            if (avg)
                output.div_(getSize());
        }
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> reduce_scatter(std::vector<at::Tensor>& outputs,
                                            std::vector<std::vector<at::Tensor>>& inputs,
                                            const ReduceScatterOptions& opts) override {
        TORCH_CHECK(outputs.size() == 1 && inputs.size() == 1, "ccl backend: one tensor per rank");
        at::Tensor flat = at::cat(inputs[0]).contiguous().view({ -1 });
        at::Tensor out = contig(outputs[0]);
        auto work = _reduce_scatter_base(out, flat, opts);
        if (!out.is_same(outputs[0])) {
            work->wait();
            outputs[0].copy_(out);
        }
        return work;
    }

    c10::intrusive_ptr<Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outputs,
                                                             std::vector<at::Tensor>& inputs,
                                                             const ReduceScatterOptions& opts) override {
        c10::intrusive_ptr<Work> last;
        for (size_t i = 0; i < inputs.size(); i++)
            last = _reduce_scatter_base(outputs[i], inputs[i], opts);
        return last;
    }

    c10::intrusive_ptr<Work> alltoall_base(at::Tensor& output, at::Tensor& input, std::vector<int64_t>& outSplits,
                                           std::vector<int64_t>& inSplits, const AllToAllOptions&) override {
        TORCH_CHECK(output.is_contiguous(), "ccl backend: output must be contiguous");
        at::Tensor in = contig(input);
        auto c = begin(in);
        auto w = c10::make_intrusive<WorkCCL>(OpType::ALLTOALL_BASE, std::vector<at::Tensor>{ output },
                                              std::vector<at::Tensor>{ in });
        const int N = getSize();
        const size_t row_in = in.dim() > 0 && in.size(0) > 0 ? (size_t)(in.numel() / in.size(0)) : 1;
        const size_t row_out = output.dim() > 0 && output.size(0) > 0 ? (size_t)(output.numel() / output.size(0)) : 1;
        std::vector<size_t> sc(N), rc(N);
        for (int i = 0; i < N; i++) {
            sc[i] = inSplits.empty() ? (size_t)in.numel() / N : (size_t)inSplits[i] * row_in;
            rc[i] = outSplits.empty() ? (size_t)output.numel() / N : (size_t)outSplits[i] * row_out;
        }
        if (c.cuda)
            w->add(ccl::alltoallv(in.data_ptr(), sc, output.data_ptr(), rc, to_ccl_dtype(in.scalar_type()), comm_,
                                  c.stream));
        else
            w->add(ccl::alltoallv(in.data_ptr(), sc, output.data_ptr(), rc, to_ccl_dtype(in.scalar_type()), comm_));
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> alltoall(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
                                      const AllToAllOptions& opts) override {
        const int N = getSize();
        TORCH_CHECK((int)outputs.size() == N && (int)inputs.size() == N, "alltoall: need one tensor per rank");
        std::vector<int64_t> ins, outs;
        for (auto& t : inputs)
            ins.push_back(t.numel());
        for (auto& t : outputs)
            outs.push_back(t.numel());
        std::vector<at::Tensor> flat_in_parts;
        for (auto& t : inputs)
            flat_in_parts.push_back(t.contiguous().view({ -1 }));
        at::Tensor in = at::cat(flat_in_parts);
        int64_t total = 0;
        for (auto v : outs)
            total += v;
        at::Tensor out = at::empty({ total }, in.options());
        auto work = alltoall_base(out, in, outs, ins, opts);
        work->wait();
        if (out.is_cuda())
            c10::cuda::getCurrentCUDAStream(out.device().index()).synchronize();
        int64_t off = 0;
        for (size_t i = 0; i < outputs.size(); i++) {
            outputs[i].copy_(out.narrow(0, off, outs[i]).view_as(outputs[i]));
            off += outs[i];
        }
        return work;
    }

    c10::intrusive_ptr<Work> gather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                    const GatherOptions& opts) override {
        // gather = allgather restricted to the root (collective sizes are identical)
        at::Tensor in = contig(inputs[0]);
        at::Tensor flat = at::empty({ in.numel() * getSize() }, in.options());
        auto work = _allgather_base(flat, in);
        work->wait();
        if (getRank() == (int)opts.rootRank) {
            if (flat.is_cuda())
                c10::cuda::getCurrentCUDAStream(flat.device().index()).synchronize();
            for (int i = 0; i < getSize(); i++)
                outputs[0][i].copy_(flat.narrow(0, i * in.numel(), in.numel()).view_as(outputs[0][i]));
        }
        return work;
    }

    c10::intrusive_ptr<Work> scatter(std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
                                     const ScatterOptions& opts) override {
        // scatter = alltoall in which only the root contributes
        at::Tensor out = contig(outputs[0]);
        const int N = getSize();
        std::vector<int64_t> ins(N, 0), outs(N, 0);
        at::Tensor in;
        if (getRank() == (int)opts.rootRank) {
            std::vector<at::Tensor> parts;
            for (auto& t : inputs[0])
                parts.push_back(t.contiguous().view({ -1 }));
            in = at::cat(parts);
            for (int i = 0; i < N; i++)
                ins[i] = out.numel();
        }
        else
            in = at::empty({ 0 }, out.options());
        outs[(int)opts.rootRank] = out.numel();
        at::Tensor flat_out = out.view({ -1 });
        AllToAllOptions o;
        auto work = alltoall_base(flat_out, in, outs, ins, o);
        if (!out.is_same(outputs[0])) {
            work->wait();
            outputs[0].copy_(out);
        }
        return work;
    }

    c10::intrusive_ptr<Work> send(std::vector<at::Tensor>& tensors, int dstRank, int /*tag*/) override {
        at::Tensor t = contig(tensors[0]);
        auto c = begin(t);
        auto w = c10::make_intrusive<WorkCCL>(OpType::SEND, tensors, std::vector<at::Tensor>{ t });
        if (c.cuda)
            w->add(ccl::send(t.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()), dstRank, comm_, c.stream));
        else
            w->add(ccl::send(t.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()), dstRank, comm_));
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> recv(std::vector<at::Tensor>& tensors, int srcRank, int /*tag*/) override {
        TORCH_CHECK(tensors[0].is_contiguous(), "ccl backend: recv tensor must be contiguous");
        at::Tensor t = tensors[0];
        auto c = begin(t);
        auto w = c10::make_intrusive<WorkCCL>(OpType::RECV, tensors, std::vector<at::Tensor>{ t });
        if (c.cuda)
            w->add(ccl::recv(t.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()), srcRank, comm_, c.stream));
        else
            w->add(ccl::recv(t.data_ptr(), (size_t)t.numel(), to_ccl_dtype(t.scalar_type()), srcRank, comm_));
        return finish(c, w);
    }

    c10::intrusive_ptr<Work> barrier(const BarrierOptions& opts = BarrierOptions()) override {
        auto w = c10::make_intrusive<WorkCCL>(OpType::BARRIER, std::vector<at::Tensor>{}, std::vector<at::Tensor>{});
        // drain device work first, then meet on the host transport
        for (auto& kv : streams_)
            cudaStreamSynchronize(kv.second);
        (void)opts;
        ccl::barrier(comm_).wait();
        w->make_future(false, 0);
        return w;
    }

    void startCoalescing() override {
        ccl::group_start();
        coalescing_ = true;
    }
    c10::intrusive_ptr<Work> endCoalescing() override {
        ccl::group_end();
        coalescing_ = false;
        auto w = c10::make_intrusive<CoalescedWorkCCL>(std::move(batch_));
        batch_.clear();
        return w;
    }
    bool supportsCoalescing() const override { return true; }

    static c10::intrusive_ptr<Backend> create(const c10::intrusive_ptr<Store>& store, int rank, int size,
                                              const std::chrono::duration<float>& /*timeout*/) {
        return c10::make_intrusive<ProcessGroupCCL>(store, rank, size);
    }

private:
    void copy_back(launch_ctx& c, at::Tensor& dst, const at::Tensor& src) {
        if (c.cuda) {
            c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(c.comm_stream, c.dev));
            dst.copy_(src, true);
        }
        else
            dst.copy_(src);
    }
    c10::intrusive_ptr<Store> store_;
    ccl::communicator comm_;
    std::mutex mu_;
    std::map<c10::DeviceIndex, cudaStream_t> streams_;
    bool coalescing_ = false;
    std::vector<c10::intrusive_ptr<Work>> batch_; // operations issued since startCoalescing
};

} // namespace c10d

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("create_backend", &c10d::ProcessGroupCCL::create, "creates the ccl process group backend");
}
