#include "fusion/fusion.hpp"

#include <cstring>

#include "coll/algorithms.hpp"
#include "core/datatype.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "sched/entries.hpp"

namespace cclx {

struct fusion_manager::fused_event : public event_impl {
    std::atomic<bool> done{ false };
    std::atomic<bool> launched{ false };
    host_comm* comm = nullptr;
    std::shared_ptr<master_sched> master; // the batch this operation travels in (host buffers)
    uint64_t ticket = 0;
    event_ptr device_done; // device buffers: the event recorded behind the batch's unpack kernel
    void wait() override {
        if (!launched.load(std::memory_order_acquire))
            fusion_manager::get().flush(comm);
        if (device_done)
            device_done->wait();
        else
            executor::get().wait(master.get(), ticket);
    }
    bool test() override {
        if (!launched.load(std::memory_order_acquire))
            fusion_manager::get().flush(comm);
        return device_done ? device_done->test() : executor::get().test(master.get(), ticket);
    }
    void* native() override { return device_done ? device_done->native() : nullptr; }
};

fusion_manager& fusion_manager::get() {
    static fusion_manager inst;
    return inst;
}

event_ptr fusion_manager::try_add(host_comm& comm, const coll_param& p, const coll_attr& attr) {
    const env_data& env = env_data::get();
    const size_t bytes = p.count * dtype_size(p.dtype);
    // device buffers are fusable too: the batch then becomes one pack kernel, one allreduce on a buffer of
    // the symmetric heap and one unpack kernel on the operations' stream
    const bool fusable = bytes > 0 && bytes <= env.fusion_bytes_threshold && !attr.reduction_fn &&
                         p.reduction != red_custom && p.deps.empty() && p.dtype <= dt_last_predefined &&
                         (!p.device || (attr.out_dtype < 0 && attr.gpu_algo.empty()));
    if (!fusable) {
        flush(&comm); // keep the operation order of this communicator
        return nullptr;
    }
    std::vector<pending> batch;
    std::shared_ptr<fused_event> ev = std::make_shared<fused_event>();
    ev->comm = &comm;
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (!queue_.empty()) {
            const pending& f = queue_.front();
            const bool compatible = f.comm == &comm && f.p.dtype == p.dtype && f.p.reduction == p.reduction &&
                                    f.p.device == p.device && f.p.stream == p.stream && f.scale == attr.scale &&
                                    f.do_scale == attr.do_scale;
            if (!compatible || queue_.size() >= env.fusion_count_threshold ||
                queued_bytes_ + bytes > env.fusion_bytes_threshold * env.fusion_count_threshold) {
                batch.assign(queue_.begin(), queue_.end());
                queue_.clear();
                queued_bytes_ = 0;
            }
        }
        queue_.push_back(pending{ &comm, p, ev, attr.scale, attr.do_scale });
        queued_bytes_ += bytes;
        if (queue_.size() >= env.fusion_count_threshold) {
            if (!batch.empty()) {
                // two full batches back to back: start the older one first
                launch(batch);
                batch.clear();
            }
            batch.assign(queue_.begin(), queue_.end());
            queue_.clear();
            queued_bytes_ = 0;
        }
    }
    if (!batch.empty())
        launch(batch);
    return ev;
}

void fusion_manager::flush(host_comm* comm) {
    std::vector<pending> batch;
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (queue_.empty() || (comm && queue_.front().comm != comm))
            return;
        batch.assign(queue_.begin(), queue_.end());
        queue_.clear();
        queued_bytes_ = 0;
    }
    launch(batch);
}

void fusion_manager::launch(std::vector<pending>& batch) {
    host_comm* comm = batch[0].comm;
    const int dtype = batch[0].p.dtype, op = batch[0].p.reduction;
    const size_t esz = dtype_size(dtype);
    if (batch[0].p.device) {
        std::vector<const void*> send;
        std::vector<void*> recv;
        std::vector<size_t> counts;
        for (auto& b : batch) {
            send.push_back(b.p.send_buf);
            recv.push_back(b.p.recv_buf);
            counts.push_back(b.p.count);
        }
        coll_attr a;
        a.scale = batch[0].scale;
        a.do_scale = batch[0].do_scale;
        event_ptr done = coll_allreduce_coalesced(*comm, send, recv, counts, dtype, op, a, batch[0].p.stream, true);
        for (auto& b : batch) {
            b.ev->device_done = done;
            b.ev->launched.store(true, std::memory_order_release);
        }
        fused_ops += batch.size();
        batches++;
        stats().fused_ops += batch.size();
        stats().fused_batches++;
        LOG_DEBUG("fusion: ", batch.size(), " device allreduces in one launch sequence");
        return;
    }
    size_t total = 0;
    for (auto& b : batch)
        total += b.p.count;
    auto master = std::make_shared<master_sched>(comm, comm->next_sched_id(true));
    sched* s = master->add_partial(0);
    char* fused = (char*)s->alloc_tmp(total * esz + 64);
    // pack
    size_t off = 0;
    for (auto& b : batch) {
        s->add<copy_entry>(b.p.send_buf, fused + off * esz, b.p.count * esz);
        off += b.p.count;
    }
    s->add_barrier();
    // one allreduce over the packed buffer
    algo::buf_desc d{ nullptr, fused, total, dtype, op, nullptr };
    const size_t bytes = total * esz;
    if (bytes <= 8192)
        algo::allreduce_recursive_doubling(*s, d);
    else if (bytes <= (512u << 10))
        algo::allreduce_nreduce(*s, d);
    else
        algo::allreduce_ring(*s, d);
    s->add_barrier();
    // unpack
    off = 0;
    for (auto& b : batch) {
        s->add<copy_entry>(fused + off * esz, b.p.recv_buf, b.p.count * esz);
        off += b.p.count;
    }
    const uint64_t ticket = executor::get().start(master.get());
    for (auto& b : batch) {
        b.ev->master = master;
        b.ev->ticket = ticket;
        b.ev->launched.store(true, std::memory_order_release);
    }
    fused_ops += batch.size();
    batches++;
    stats().fused_ops += batch.size();
    stats().fused_batches++;
    LOG_DEBUG("fusion: ", batch.size(), " allreduces, ", bytes, " bytes in one schedule");
}

} // namespace cclx
