// Fusion of small allreduce operations into one buffer and one collective.
//
// Same purpose and knobs as the reference's fusion manager
// (src/fusion/fusion.cpp:129-466; CCL_FUSION, CCL_FUSION_BYTES_THRESHOLD = 16384,
// CCL_FUSION_COUNT_THRESHOLD = 256): allreduces below the byte threshold with the
// same communicator / datatype / reduction and no custom function are queued,
// then packed into one buffer, reduced by a single schedule, and unpacked, with
// every user's event completed from the schedule's last entry.
//
// Design difference: the reference flushes on a timer in its service worker,
// so ranks may cut batches at different places.  Here a batch is cut only at
// points that are the same in every rank's program order (count or byte limit
// reached, an operation that cannot be fused arrives on the communicator, a
// fused event is waited on or tested), which keeps the fused message identical
// on all ranks without an agreement round.
#pragma once
#include <deque>
#include <memory>
#include <mutex>

#include "coll/coll.hpp"

namespace cclx {

class fusion_manager {
public:
    static fusion_manager& get();
    // returns nullptr when the operation is not fusable (caller runs it normally)
    event_ptr try_add(host_comm& comm, const coll_param& p, const coll_attr& attr);
    // cut the current batch of `comm` (all communicators when null) and start it
    void flush(host_comm* comm = nullptr);
    uint64_t fused_ops = 0, batches = 0;

private:
    struct fused_event;
    struct pending {
        host_comm* comm;
        coll_param p;
        std::shared_ptr<fused_event> ev;
        float scale = 1.0f; // device operations: fused output scale of the operation
        bool do_scale = false;
    };
    void launch(std::vector<pending>& batch);
    std::mutex mu_;
    std::deque<pending> queue_;
    size_t queued_bytes_ = 0;
};

} // namespace cclx
