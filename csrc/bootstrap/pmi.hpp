// Process-management layer on top of a key-value store: rank-scoped put/get,
// barrier, allgather and broadcast of small blobs.
//
// Plays the part of the reference's pmi_resizable_simple(_internal)
// (src/atl/util/pm/pmi_resizable_rt/pmi_resizable_simple_internal.cpp:151-337):
// every communicator creation gets its own key namespace ("CCL_POD_ADDR<id>"),
// keys are "<name>-<rank>", barriers are counted on the server.  Works over any
// ikvs; the counted barrier of the internal server is used when available and
// replaced by a set/get rendezvous on user-supplied stores.
#pragma once
#include <memory>
#include <string>

#include "bootstrap/kvs.hpp"
#include "gpu/symm_heap.hpp"

namespace cclx {

class pmi : public gpu::bootstrap_if {
public:
    pmi(std::shared_ptr<kvs::ikvs> store, int rank, int size);
    ~pmi() override = default;

    int rank() const override { return rank_; }
    int size() const override { return size_; }
    void put(const std::string& name, const kvs::bytes& v);
    kvs::bytes get(const std::string& name, int from_rank);
    void barrier() override;
    void allgather(const void* send, void* recv, size_t bytes_per_rank) override;
    void bcast(void* buf, size_t bytes, int root);
    std::string job_id() override;
    const std::string& ns() const { return ns_; }
    std::shared_ptr<kvs::ikvs> store() const { return store_; }
    // liveness: heartbeat keys under the namespace
    void heartbeat();
    bool peer_alive(int r, int max_age_ms);

private:
    std::shared_ptr<kvs::ikvs> store_;
    kvs::internal_kvs* internal_ = nullptr;
    int rank_, size_;
    std::string ns_;
    unsigned seq_ = 0;
    std::string job_id_;
    int timeout_ms_;
};

} // namespace cclx
