// CPU scheduler: schedule objects made of entries, progressed by worker threads.
//
// Behavioural model taken from the reference (src/sched/sched.hpp:59-319,
// src/sched/entry/entry.hpp:56-129, src/sched/queue/queue.hpp:38-257,
// src/exec/exec.hpp:40-178, src/exec/thread/worker.cpp:62-379): a collective is
// compiled once into a schedule - a list of small state machines (send, recv,
// recv+reduce, local reduce, copy, sync, nested schedule, ...) with barrier
// points - split into per-worker partial schedules, queued into priority bins
// and progressed cooperatively until the request counter reaches zero.  Cached
// schedules are re-armed instead of rebuilt; a relaunch of a schedule that is
// still running is queued behind it.
//
// The implementation is this library's own and much smaller: entries are plain
// C++ objects owning their requests, tags are (comm, schedule, step) triples
// matched FIFO per source by the transport, temporary memory comes from a
// size-bucketed cache, and workers sleep on a condition variable when idle.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "core/types.hpp"
#include "transport/atl.hpp"

namespace cclx {

class host_comm;
class sched;
class executor;

// ---- request ------------------------------------------------------------------------
// Counts the partial schedules of one launch.  The partial that finishes last
// runs on_last (on its worker thread).  What a user waits for is a launch
// ticket of the master schedule (master_sched::issued / done), not this counter,
// so that a cached schedule can be relaunched from on_last.
class request {
public:
    void arm(int parts) { counter_.store(parts, std::memory_order_release); }
    void part_done() {
        if (counter_.fetch_sub(1, std::memory_order_acq_rel) == 1 && on_last)
            on_last();
    }
    std::function<void()> on_last;
    void set_error(const std::string& e);
    bool has_error() const { return failed_.load(std::memory_order_acquire); }
    std::string error() const;
    std::atomic<bool> urgent{ false }; // a user thread is waiting (fusion flushes early)

private:
    std::atomic<int> counter_{ 0 };
    std::atomic<bool> failed_{ false };
    mutable std::mutex mu_;
    std::string error_;
};

// ---- temporary memory ---------------------------------------------------------------
// process-wide size-bucketed cache of host buffers (reference buffer_cache.hpp:35-101)
class buffer_cache {
public:
    static buffer_cache& get();
    void* take(size_t bytes);
    void give(void* p, size_t bytes);
    void clear();
    size_t cached_bytes() const { return cached_; }
    uint64_t hits = 0, misses = 0;

private:
    std::mutex mu_;
    std::multimap<size_t, void*> free_;
    size_t cached_ = 0;
};

// ---- entries ------------------------------------------------------------------------
enum class entry_status { not_started, again, started, complete };

class sched_entry {
public:
    explicit sched_entry(sched* s) : owner_(s) {}
    virtual ~sched_entry() = default;
    virtual const char* name() const = 0;
    virtual void start() = 0;
    virtual void update() {}
    virtual void reset() { status_ = entry_status::not_started; }
    void do_progress();
    entry_status status() const { return status_; }
    bool is_complete() const { return status_ == entry_status::complete; }
    // entries that inject data into the transport take a flow-control credit while in flight
    virtual bool uses_credit() const { return false; }
    void make_barrier() { barrier_ = true; }
    bool is_barrier() const { return barrier_; }
    // profile (CCL_SCHED_PROFILE)
    uint64_t total_ns = 0, update_calls = 0;

protected:
    sched* owner_;
    entry_status status_ = entry_status::not_started;
    bool barrier_ = false;
    uint64_t started_at_ns_ = 0;
};

// ---- schedule -----------------------------------------------------------------------
class sched {
public:
    sched(host_comm* comm, uint64_t sched_id, int ep);
    ~sched();

    host_comm* comm() const { return comm_; }
    int ep() const { return ep_; }
    uint64_t sched_id() const { return sched_id_; }
    void set_sched_id(uint64_t id) { sched_id_ = id; }
    uint64_t tag(uint64_t step) const;

    // building
    template <class E, class... Args>
    E* add(Args&&... args) {
        E* e = new E(this, std::forward<Args>(args)...);
        entries_.emplace_back(e);
        return e;
    }
    void add_barrier(); // entries added later start only when everything before is complete
    void* alloc_tmp(size_t bytes);
    size_t entry_count() const { return entries_.size(); }

    // running
    bool do_progress(); // true when every entry is complete
    void reset(); // re-arm for another launch (cached schedules)
    void dump(std::string& out) const;
    void profile(std::string& out) const;
    size_t flow_high_water = 0; // most entries of this schedule ever in flight together

    int priority = 0;
    request* req = nullptr; // request of the master schedule this partial belongs to
    uint64_t op_base = 0; // partial schedules of one master use disjoint step ranges
    std::function<void()> on_complete; // runs on the worker thread after the last entry

private:
    host_comm* comm_;
    uint64_t sched_id_;
    int ep_;
    std::deque<std::unique_ptr<sched_entry>> entries_;
    size_t first_incomplete_ = 0;
    std::vector<std::pair<void*, size_t>> tmp_;
};

// A master schedule: what one API call creates.  Owns the partial schedules and the request.
class master_sched {
public:
    master_sched(host_comm* comm, uint64_t sched_id);
    ~master_sched();
    sched* add_partial(int ep);
    request& req() { return req_; }
    std::vector<std::unique_ptr<sched>>& partials() { return partials_; }
    uint64_t sched_id() const { return sched_id_; }
    host_comm* comm() const { return comm_; }
    // A cached schedule takes a new id on every launch (reference sched.cpp: the id is updated at each
    // commit).  Ranks may disagree on which calls hit their caches (a key made of buffer addresses hits
    // on one rank and misses on another), but they agree on the order of calls, so the id drawn per
    // call is the same everywhere while an id kept from build time would not be.
    void renew_id(uint64_t id);
    std::deque<uint64_t> pending_ids; // ids of launches queued behind the running one (under launch_mu)

    // launch tickets: launch k is complete when done >= k
    std::atomic<uint64_t> issued{ 0 }, done{ 0 };
    bool ticket_complete(uint64_t t) const { return done.load(std::memory_order_acquire) >= t || req_.has_error(); }
    // every partial of launch t has left the workers' queues: only then may the object go away (a failed
    // launch is complete for its waiter before that)
    bool ticket_retired(uint64_t t) const { return done.load(std::memory_order_acquire) >= t; }
    // cached-schedule relaunch protocol (reference sched_restart_manager.cpp:19-146):
    // a launch requested while the schedule runs is queued and started by the
    // worker that completes the current one
    std::mutex launch_mu;
    std::atomic<bool> in_flight{ false }; // written under launch_mu; the schedule cache reads it without
    // true when no launch is running or queued and the worker that finished the last one is done with this object
    bool idle() const {
        return !in_flight.load(std::memory_order_acquire) &&
               done.load(std::memory_order_acquire) == issued.load(std::memory_order_acquire);
    }
    int delayed_launches = 0;
    bool cached = false;
    int priority = 0;
    std::function<void()> user_complete; // e.g. unpack / finalise of a fused operation
    std::string cache_key;

private:
    host_comm* comm_;
    uint64_t sched_id_;
    request req_;
    std::vector<std::unique_ptr<sched>> partials_;
};

// ---- queue, workers, executor ---------------------------------------------------------
class sched_queue {
public:
    void add(sched* s);
    // progress the highest-priority bin (every bin once in a while); returns the number of schedules touched
    size_t progress(uint64_t iteration, bool strict_order);
    bool empty();
    size_t size();
    void dump(std::string& out);

private:
    std::mutex mu_;
    std::map<int, std::vector<sched*>, std::greater<int>> bins_;
    std::deque<sched*> incoming_;
};

class worker {
public:
    worker(executor* ex, int idx);
    ~worker();
    void start();
    void stop();
    void add(sched* s);
    size_t do_work(); // one progress iteration (also callable from a user thread)
    int index() const { return idx_; }
    bool on_worker_thread() const;

private:
    void loop();
    executor* ex_;
    int idx_;
    sched_queue queue_;
    std::thread thread_;
    std::atomic<bool> stop_{ false };
    std::mutex mu_;
    std::mutex work_mu_; // one thread progresses a worker's queue at a time
    std::condition_variable cv_;
    uint64_t iteration_ = 0;
    std::thread::id tid_;
};

class executor {
public:
    static executor& get();
    // lets the calling thread drive the schedules when there are no worker threads
    void progress();
    void ensure_started(std::shared_ptr<atl_transport> tr);
    void shutdown();
    int worker_count() const { return (int)workers_.size(); }
    // returns the launch ticket
    static constexpr uint64_t KEEP_ID = ~0ull;
    // `new_id`: schedule id of this launch (KEEP_ID: the one the schedule was built with)
    uint64_t start(master_sched* m, uint64_t new_id = KEEP_ID);
    void wait(master_sched* m, uint64_t ticket);
    bool test(master_sched* m, uint64_t ticket);
    void launch_now(master_sched* m); // arm + enqueue (internal)
    // service hook run by worker 0 every iteration (fusion flush)
    std::function<void()> service_hook;
    // hold every worker outside its progress loop (datatype table changes, resize)
    void lock_workers();
    void unlock_workers();

    ~executor();

private:
    friend class worker;
    executor() = default;
    std::vector<std::unique_ptr<worker>> workers_;
    // every transport with a live communicator is polled; the executor does not keep them alive
    typedef std::vector<std::weak_ptr<atl_transport>> transport_list;
    std::shared_ptr<const transport_list> transports_;
    std::atomic<unsigned> rr_{ 0 };
    std::mutex mu_;
    std::mutex freeze_mu_;
    std::atomic<bool> frozen_{ false };
};

// ---- schedule cache -------------------------------------------------------------------
class sched_cache {
public:
    // The schedule stays alive while the caller holds the pointer, whatever the cache does meanwhile.
    std::shared_ptr<master_sched> find(const std::string& key);
    // At most CCL_SCHED_CACHE_MAX_ENTRIES schedules are kept: a program that reuses a match_id with new
    // buffers every time (keys contain the buffer addresses) would otherwise grow the cache without
    // bound.  The least recently used schedule that is not running makes room.
    void insert(const std::string& key, std::shared_ptr<master_sched> m);
    void flush(); // drops schedules that are not in flight
    size_t size();
    uint64_t hits = 0, misses = 0, evictions = 0;

private:
    struct slot {
        std::shared_ptr<master_sched> m;
        uint64_t last_use = 0;
    };
    std::mutex mu_;
    uint64_t clock_ = 0;
    std::unordered_map<std::string, slot> map_;
};

uint64_t now_ns();

} // namespace cclx
