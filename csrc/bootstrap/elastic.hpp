// Elastic membership on top of the key-value store: processes ("pods") may join and leave a job
// while it runs; the survivors agree on a new rank assignment and re-form their communicator.
//
// Covers the reference's resizable process manager (src/atl/util/pm/pmi_resizable_rt/pmi_resizable/
// resizable_pmi.cpp:36-404: pod list in the KVS, liveness tracking, a user `resize_fn` that answers
// wait / run / finalize for a proposed size; pmi_listener.cpp:43-242 for the liveness side) with a
// smaller protocol:
//   * every pod registers "pods/<id>" with a join ticket (atomic counter: a total order) and a
//     thread bumps its heartbeat counter "hb/<id>";
//   * a pod is alive for an observer while its counter keeps changing (no clocks are compared
//     across hosts);
//   * to form generation g every live pod publishes the member list it sees under
//     "view/<g>/<id>"; the view is adopted when all listed members published the same list and
//     the resize function accepts its size;
//   * ranks follow the join tickets, and the communicator of generation g bootstraps through a
//     store view whose keys are prefixed with "elastic/<g>/", so old and new pods agree on every
//     key although they have created different numbers of communicators before.
// The store itself (the process that created the main KVS) is the one fixed point, as in the reference.
#pragma once
#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "bootstrap/kvs.hpp"

namespace cclx {

enum class resize_action : int { wait = 0, run = 1, finalize = 2 };

// store view with prefixed keys and its own identity (address string carries the prefix)
class scoped_kvs : public kvs::ikvs {
public:
    scoped_kvs(std::shared_ptr<kvs::ikvs> base, std::string prefix);
    void set(const std::string& key, const kvs::bytes& val) override { base_->set(prefix_ + key, val); }
    bool try_get(const std::string& key, kvs::bytes& out) override { return base_->try_get(prefix_ + key, out); }
    kvs::address get_address() const override { return addr_; }

private:
    std::shared_ptr<kvs::ikvs> base_;
    std::string prefix_;
    kvs::address addr_{};
};

class elastic_group {
public:
    struct view {
        int rank = -1;
        int size = 0;
        uint64_t generation = 0;
        std::vector<std::string> members; // in rank order
    };

    elastic_group(std::shared_ptr<kvs::internal_kvs> store, std::string pod_id, int heartbeat_ms, int dead_after_ms);
    ~elastic_group();

    // answer for a proposed size; default: run as soon as `min_size` pods are present
    void set_resize_fn(std::function<resize_action(size_t)> fn) { resize_fn_ = std::move(fn); }
    void set_min_size(size_t n) { min_size_ = n; }

    // registers this pod (first call) and agrees on the next generation with the live pods;
    // throws on timeout or when the resize function answers finalize
    view form(int timeout_ms);
    const view& current() const { return view_; }
    // true when the set of live pods differs from the current view (someone died, left or joined)
    bool changed();
    // withdraws this pod: the others see the change at their next check
    void leave();
    // store view the communicator of the current generation bootstraps through
    std::shared_ptr<kvs::ikvs> generation_store();
    const std::string& id() const { return id_; }
    // called by form() after this pod published its list for a generation and before it looks at the others'
    // (a test makes a third pod register inside that window)
    void set_window_hook(std::function<void(uint64_t)> fn) { window_hook_ = std::move(fn); }

private:
    std::vector<std::string> live_pods(int settle_ms);
    void beat_loop();
    std::shared_ptr<kvs::internal_kvs> store_;
    std::string id_;
    int hb_ms_, dead_ms_;
    size_t min_size_ = 1;
    std::function<resize_action(size_t)> resize_fn_;
    bool registered_ = false;
    view view_;
    uint64_t floor_ = 0; // generations below this one failed here
    std::function<void(uint64_t)> window_hook_;
    std::thread beat_;
    std::atomic<bool> stop_{ false };
    // last observed heartbeat value and when it last changed (local steady clock, ms)
    struct seen {
        long long value = -1;
        long long changed_at = 0;
    };
    std::map<std::string, seen> seen_;
    std::map<std::string, long long> ticket_;
};

} // namespace cclx
