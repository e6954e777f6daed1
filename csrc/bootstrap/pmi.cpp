#include "bootstrap/pmi.hpp"

#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <random>

#include "core/env.hpp"
#include "core/log.hpp"

namespace cclx {

namespace {
std::mutex id_mu;
// per store address: how many process groups this process created on it.  All
// ranks create their communicators in the same order, so the counter names the
// same namespace everywhere (the reference's local_id).
std::map<std::string, unsigned> local_ids;
} // namespace

pmi::pmi(std::shared_ptr<kvs::ikvs> store, int rank, int size) : store_(std::move(store)), rank_(rank), size_(size) {
    CCL_THROW_IF_NOT(size > 0 && rank >= 0 && rank < size, "invalid rank ", rank, " / size ", size);
    internal_ = dynamic_cast<kvs::internal_kvs*>(store_.get());
    timeout_ms_ = env_data::get().kvs_get_timeout_sec * 1000;
    unsigned id;
    {
        std::lock_guard<std::mutex> lk(id_mu);
        id = local_ids[store_->get_address().str() + "#" + std::to_string(size)]++;
    }
    ns_ = "CCL_POD_ADDR" + std::to_string(id) + "_" + std::to_string(size);
}

void pmi::put(const std::string& name, const kvs::bytes& v) {
    store_->set(ns_ + "/" + name + "-" + std::to_string(rank_), v);
}

kvs::bytes pmi::get(const std::string& name, int from_rank) {
    return store_->get(ns_ + "/" + name + "-" + std::to_string(from_rank), timeout_ms_);
}

void pmi::barrier() {
    const unsigned s = seq_++;
    if (size_ == 1)
        return;
    if (internal_) {
        internal_->raw().barrier(ns_ + "/CCL_BARRIER" + std::to_string(s), (uint32_t)size_, timeout_ms_);
        return;
    }
    // generic store: everybody checks in, rank 0 releases
    const std::string base = ns_ + "/bar" + std::to_string(s);
    store_->set(base + "-in-" + std::to_string(rank_), kvs::bytes(1, '1'));
    if (rank_ == 0) {
        for (int r = 0; r < size_; r++)
            store_->get(base + "-in-" + std::to_string(r), timeout_ms_);
        store_->set(base + "-out", kvs::bytes(1, '1'));
    }
    else
        store_->get(base + "-out", timeout_ms_);
}

void pmi::allgather(const void* send, void* recv, size_t n) {
    const unsigned s = seq_++;
    const std::string name = "ag" + std::to_string(s);
    put(name, kvs::bytes((const char*)send, (const char*)send + n));
    for (int r = 0; r < size_; r++) {
        if (r == rank_) {
            std::memcpy((char*)recv + (size_t)r * n, send, n);
            continue;
        }
        kvs::bytes b = get(name, r);
        CCL_THROW_IF_NOT(b.size() == n, "bootstrap allgather size mismatch from rank ", r);
        std::memcpy((char*)recv + (size_t)r * n, b.data(), n);
    }
}

void pmi::bcast(void* buf, size_t n, int root) {
    const unsigned s = seq_++;
    const std::string name = "bc" + std::to_string(s);
    if (rank_ == root)
        put(name, kvs::bytes((const char*)buf, (const char*)buf + n));
    else {
        kvs::bytes b = get(name, root);
        CCL_THROW_IF_NOT(b.size() == n, "bootstrap bcast size mismatch");
        std::memcpy(buf, b.data(), n);
    }
}

std::string pmi::job_id() {
    if (job_id_.empty()) {
        char id[17] = { 0 };
        if (rank_ == 0) {
            std::random_device rd;
            static const char* hex = "0123456789abcdef";
            for (int i = 0; i < 16; i++)
                id[i] = hex[rd() & 15];
        }
        bcast(id, 16, 0);
        job_id_ = std::string(id, 16);
    }
    return job_id_;
}

void pmi::heartbeat() {
    using namespace std::chrono;
    long long now = duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
    std::string v = std::to_string(now);
    store_->set(ns_ + "/hb-" + std::to_string(rank_), kvs::bytes(v.begin(), v.end()));
}

bool pmi::peer_alive(int r, int max_age_ms) {
    using namespace std::chrono;
    kvs::bytes b;
    if (!store_->try_get(ns_ + "/hb-" + std::to_string(r), b))
        return false;
    long long then = std::atoll(std::string(b.begin(), b.end()).c_str());
    long long now = duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
    // steady_clock is per host; the heartbeat check is meant for ranks of one node
    return now - then <= max_age_ms;
}

} // namespace cclx
