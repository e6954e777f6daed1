#include "sched/sched.hpp"
#include "topo/numa.hpp"

#include <pthread.h>
#include <sched.h>

#include <chrono>
#include <cstdlib>
#include <sstream>

#include "comm/host_comm.hpp"
#include "core/datatype.hpp"
#include "core/env.hpp"
#include "core/trace.hpp"
#include "core/log.hpp"
#include "sched/entries.hpp"

namespace cclx {

uint64_t now_ns() {
    using namespace std::chrono;
    return (uint64_t)duration_cast<nanoseconds>(steady_clock::now().time_since_epoch()).count();
}

// ---- request --------------------------------------------------------------------------
void request::set_error(const std::string& e) {
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (error_.empty())
            error_ = e;
    }
    failed_.store(true, std::memory_order_release);
}

std::string request::error() const {
    std::lock_guard<std::mutex> lk(mu_);
    return error_;
}

// ---- buffer cache ---------------------------------------------------------------------
buffer_cache& buffer_cache::get() {
    // never destroyed: schedules that outlive static destruction still hand their buffers back
    static buffer_cache* inst = new buffer_cache();
    return *inst;
}

static size_t bucket_of(size_t bytes) {
    size_t b = 4096;
    while (b < bytes)
        b <<= 1;
    return b;
}

void* buffer_cache::take(size_t bytes) {
    const size_t b = bucket_of(bytes);
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = free_.find(b);
        if (it != free_.end()) {
            void* p = it->second;
            free_.erase(it);
            cached_ -= b;
            hits++;
            return p;
        }
        misses++;
    }
    void* p = nullptr;
    if (posix_memalign(&p, 4096, b) != 0 || !p)
        CCL_THROW("out of host memory allocating ", b, " bytes");
    return p;
}

void buffer_cache::give(void* p, size_t bytes) {
    const size_t b = bucket_of(bytes);
    std::lock_guard<std::mutex> lk(mu_);
    if (!env_data::get().buffer_cache || cached_ + b > env_data::get().buffer_cache_max_bytes) {
        std::free(p);
        return;
    }
    free_.emplace(b, p);
    cached_ += b;
}

void buffer_cache::clear() {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& kv : free_)
        std::free(kv.second);
    free_.clear();
    cached_ = 0;
}

// ---- entry ----------------------------------------------------------------------------
void sched_entry::do_progress() {
    const env_data& env = env_data::get();
    const bool timed = env.sched_profile || env.entry_max_update_time_sec > 0;
    uint64_t t0 = timed ? now_ns() : 0;
    if (status_ == entry_status::not_started || status_ == entry_status::again) {
        if (status_ == entry_status::not_started && timed)
            started_at_ns_ = t0;
        status_ = entry_status::started;
        trace_range tr(2, name()); // entries are state machines: the range covers the start call, marks the end
        start();
    }
    else if (status_ == entry_status::started) {
        update_calls++;
        update();
        if (status_ == entry_status::complete && trace_level() >= 2)
            trace_mark(name());
    }
    if (timed) {
        uint64_t t1 = now_ns();
        total_ns += t1 - t0;
        if (env.entry_max_update_time_sec > 0 && status_ == entry_status::started &&
            (double)(t1 - started_at_ns_) * 1e-9 > env.entry_max_update_time_sec) {
            CCL_THROW("entry ", name(), " made no progress for ", env.entry_max_update_time_sec,
                      " s (CCL_ENTRY_MAX_UPDATE_TIME_SEC): a peer is missing or stalled");
        }
    }
}

// ---- concrete entries -----------------------------------------------------------------
namespace {
// a transport request that ended because the peer is gone turns into the schedule's error
inline entry_status request_status(const atl_req& req, const char* what, int peer) {
    if (!req.is_done())
        return entry_status::started;
    if (req.error)
        CCL_THROW(what, ": rank ", peer, " of the communicator has left the job (process gone or connection closed)");
    return entry_status::complete;
}
} // namespace

void send_entry::start() {
    owner_->comm()->atl().send(owner_->ep(), buf_, bytes_, dst_, owner_->tag(step_), &req_, one_way_);
    update();
}
void send_entry::update() {
    status_ = request_status(req_, "send", dst_);
}

void register_entry::start() {
    *out_ = owner_->comm()->atl().mr_reg(buf_, bytes_);
    status_ = entry_status::complete;
}
void deregister_entry::start() {
    owner_->comm()->atl().mr_dereg(*mr_);
    status_ = entry_status::complete;
}
void write_entry::start() {
    owner_->comm()->atl().rma_write(owner_->ep(), buf_, bytes_, *mr_, offset_, &req_);
    update();
}
void write_entry::update() {
    status_ = request_status(req_, "one-sided write", mr_->owner);
}

void recv_entry::start() {
    owner_->comm()->atl().recv(owner_->ep(), buf_, bytes_, src_, owner_->tag(step_), &req_);
    update();
}
void recv_entry::update() {
    status_ = request_status(req_, "recv", src_);
}

recv_reduce_entry::recv_reduce_entry(sched* s, void* inout, size_t count, int dtype, int op, int src, uint64_t step,
                                     reduction_fn_t fn, void* tmp, const void* local)
        : sched_entry(s), inout_(inout), count_(count), dtype_(dtype), op_(op), src_(src), step_(step), fn_(fn),
          tmp_(tmp), local_(local) {
    if (!tmp_ && !local_)
        tmp_ = s->alloc_tmp(count * dtype_size(dtype));
}
void recv_reduce_entry::start() {
    owner_->comm()->atl().recv(owner_->ep(), local_ ? inout_ : tmp_, count_ * dtype_size(dtype_), src_,
                               owner_->tag(step_), &req_);
    update();
}
void recv_reduce_entry::update() {
    if (request_status(req_, "recv", src_) != entry_status::complete) {
        status_ = entry_status::started;
        return;
    }
    comp_reduce(local_ ? local_ : tmp_, count_, inout_, dtype_, op_, fn_);
    status_ = entry_status::complete;
}

void reduce_local_entry::start() {
    comp_reduce(in_, count_, inout_, dtype_, op_, fn_);
    status_ = entry_status::complete;
}

void copy_entry::start() {
    if (bytes_ && src_ != dst_)
        std::memmove(dst_, src_, bytes_);
    status_ = entry_status::complete;
}

void sync_entry::start() {
    obj_->counter.fetch_sub(1, std::memory_order_acq_rel);
    update();
}
void sync_entry::update() {
    if (obj_->counter.load(std::memory_order_acquire) <= 0) {
        status_ = entry_status::complete;
        // the last visitor re-arms the object for the next launch of a cached schedule
        if (obj_->visited.fetch_add(1) + 1 == obj_->initial) {
            obj_->visited.store(0);
            obj_->counter.store(obj_->initial, std::memory_order_release);
        }
    }
    else
        status_ = entry_status::started;
}
void sync_entry::reset() {
    sched_entry::reset();
}

void probe_entry::update() {
    size_t len = 0;
    if (owner_->comm()->atl().transport().probe(owner_->ep(), owner_->comm()->atl().world_rank_of(src_),
                                                owner_->tag(step_), &len)) {
        if (out_)
            *out_ = len;
        status_ = entry_status::complete;
    }
    else
        status_ = entry_status::started;
}

subsched_entry::subsched_entry(sched* s, std::function<void(sched&)> builder, const char* label, host_comm* other)
        : sched_entry(s), builder_(std::move(builder)), label_(label), other_(other) {}

void subsched_entry::start() {
    if (!sub_) {
        sub_.reset(new sched(other_ ? other_ : owner_->comm(), owner_->sched_id(), owner_->ep()));
        sub_->op_base = owner_->op_base;
        builder_(*sub_);
    }
    sub_->set_sched_id(owner_->sched_id()); // a cached owner runs under a new id every time
    update();
}
void subsched_entry::update() {
    status_ = sub_->do_progress() ? entry_status::complete : entry_status::started;
}
void subsched_entry::reset() {
    sched_entry::reset();
    if (sub_)
        sub_->reset();
}

// ---- sched ----------------------------------------------------------------------------
sched::sched(host_comm* comm, uint64_t sched_id, int ep) : comm_(comm), sched_id_(sched_id), ep_(ep) {}

sched::~sched() {
    for (auto& t : tmp_)
        buffer_cache::get().give(t.first, t.second);
}

uint64_t sched::tag(uint64_t step) const {
    return atl_tag::make(comm_->id(), sched_id_, op_base + step);
}

void sched::add_barrier() {
    if (!entries_.empty())
        entries_.back()->make_barrier();
}

void* sched::alloc_tmp(size_t bytes) {
    void* p = buffer_cache::get().take(bytes ? bytes : 1);
    tmp_.emplace_back(p, bytes ? bytes : 1);
    return p;
}

bool sched::do_progress() {
    // Entries run concurrently until a barrier entry: nothing after a barrier
    // starts before everything up to and including it is complete.
    const size_t n = entries_.size();
    while (first_incomplete_ < n && entries_[first_incomplete_]->is_complete())
        first_incomplete_++;
    // flow control (reference src/sched/queue/flow_control.cpp:21-65): at most CCL_MAX_FLOW_CREDITS
    // sends of one schedule are in flight; the others start as credits come back.  Receives never
    // wait for a credit: a rank that posted only receives could otherwise starve every sender.
    const size_t credits = (size_t)std::max(1, env_data::get().max_flow_credits);
    size_t in_flight = 0;
    for (size_t i = first_incomplete_; i < n; i++) {
        sched_entry& e = *entries_[i];
        if (!e.is_complete()) {
            if (!e.uses_credit() || e.status() != entry_status::not_started || in_flight < credits)
                e.do_progress();
            if (e.uses_credit() && !e.is_complete() && e.status() != entry_status::not_started)
                in_flight++;
        }
        if (in_flight > flow_high_water)
            flow_high_water = in_flight;
        if (e.is_barrier()) {
            bool all_done = true;
            for (size_t k = first_incomplete_; k <= i; k++)
                if (!entries_[k]->is_complete()) {
                    all_done = false;
                    break;
                }
            if (!all_done)
                break;
        }
    }
    while (first_incomplete_ < n && entries_[first_incomplete_]->is_complete())
        first_incomplete_++;
    return first_incomplete_ == n;
}

void sched::reset() {
    for (auto& e : entries_)
        e->reset();
    first_incomplete_ = 0;
}

void sched::dump(std::string& out) const {
    std::ostringstream ss;
    ss << "sched " << sched_id_ << " ep " << ep_ << " entries " << entries_.size() << ":";
    for (size_t i = 0; i < entries_.size(); i++) {
        static const char* st[] = { "not_started", "again", "started", "complete" };
        ss << "\n  [" << i << "] " << entries_[i]->name() << (entries_[i]->is_barrier() ? " |barrier|" : "") << " "
           << st[(int)entries_[i]->status()];
    }
    out += ss.str();
}

void sched::profile(std::string& out) const {
    std::ostringstream ss;
    for (size_t i = 0; i < entries_.size(); i++)
        ss << "\n  [" << i << "] " << entries_[i]->name() << ": total " << entries_[i]->total_ns / 1000.0
           << " us, updates " << entries_[i]->update_calls;
    out += ss.str();
}

// ---- master ---------------------------------------------------------------------------
master_sched::master_sched(host_comm* comm, uint64_t sched_id) : comm_(comm), sched_id_(sched_id) {}
master_sched::~master_sched() = default;

void master_sched::renew_id(uint64_t id) {
    sched_id_ = id;
    for (auto& p : partials_)
        p->set_sched_id(id); // nested schedules take the id of their owner when they start
}

sched* master_sched::add_partial(int ep) {
    partials_.emplace_back(new sched(comm_, sched_id_, ep));
    sched* s = partials_.back().get();
    s->op_base = (uint64_t)(partials_.size() - 1) << 16;
    s->req = &req_;
    s->priority = priority;
    return s;
}

// ---- queue ----------------------------------------------------------------------------
void sched_queue::add(sched* s) {
    std::lock_guard<std::mutex> lk(mu_);
    incoming_.push_back(s);
}

bool sched_queue::empty() {
    std::lock_guard<std::mutex> lk(mu_);
    return incoming_.empty() && bins_.empty();
}

size_t sched_queue::size() {
    std::lock_guard<std::mutex> lk(mu_);
    size_t n = incoming_.size();
    for (auto& b : bins_)
        n += b.second.size();
    return n;
}

void sched_queue::dump(std::string& out) {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& b : bins_)
        for (sched* s : b.second) {
            out += "\n priority " + std::to_string(b.first) + ": ";
            s->dump(out);
        }
}

static void finish_sched(sched* s, const std::string* err) {
    request* r = s->req;
    if (err) {
        // The failed partial has left its queue like a finished one: it is counted, so that the launch is
        // retired (and its master may be destroyed or relaunched) only when every sibling partial, possibly
        // still queued on another worker, has left too.  Waiters are released at once by the error flag.
        if (r) {
            r->set_error(*err);
            r->part_done();
        }
        return;
    }
    if (env_data::get().sched_profile) {
        std::string p;
        s->profile(p);
        LOG_INFO("sched ", s->sched_id(), " profile:", p);
    }
    if (s->on_complete)
        s->on_complete();
    if (r)
        r->part_done();
}

size_t sched_queue::progress(uint64_t iteration, bool strict_order) {
    {
        std::lock_guard<std::mutex> lk(mu_);
        while (!incoming_.empty()) {
            sched* s = incoming_.front();
            incoming_.pop_front();
            bins_[s->priority].push_back(s);
        }
        if (bins_.empty())
            return 0;
    }
    // bins_ is only touched by the progressing thread from here on (adds go through incoming_)
    size_t touched = 0;
    const bool all_bins = (iteration & 4095) == 0;
    for (auto bit = bins_.begin(); bit != bins_.end();) {
        auto& vec = bit->second;
        for (size_t i = 0; i < vec.size();) {
            sched* s = vec[i];
            bool done = false;
            try {
                done = s->do_progress();
            }
            catch (const std::exception& e) {
                std::string msg = e.what();
                LOG_ERROR("schedule failed: ", msg);
                finish_sched(s, &msg);
                vec.erase(vec.begin() + i);
                continue;
            }
            touched++;
            if (done) {
                vec.erase(vec.begin() + i);
                finish_sched(s, nullptr);
                continue;
            }
            if (strict_order)
                break; // the head of the bin must finish first
            i++;
        }
        if (vec.empty())
            bit = bins_.erase(bit);
        else
            ++bit;
        if (!all_bins && touched)
            break; // highest-priority non-empty bin only
    }
    return touched;
}

// ---- worker ---------------------------------------------------------------------------
worker::worker(executor* ex, int idx) : ex_(ex), idx_(idx) {}

worker::~worker() {
    stop();
}

void worker::start() {
    stop_ = false;
    thread_ = std::thread([this] { loop(); });
}

void worker::stop() {
    if (!thread_.joinable())
        return;
    stop_ = true;
    cv_.notify_all();
    thread_.join();
}

void worker::add(sched* s) {
    queue_.add(s);
    cv_.notify_one();
}

bool worker::on_worker_thread() const {
    return std::this_thread::get_id() == tid_;
}

size_t worker::do_work() {
    std::unique_lock<std::mutex> work(work_mu_, std::try_to_lock);
    if (!work.owns_lock())
        return 0;
    if (ex_->frozen_.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lk(ex_->freeze_mu_); // parked while the executor is locked
    }
    iteration_++;
    if (auto list = std::atomic_load(&ex_->transports_))
        for (auto& w : *list)
            if (auto tr = w.lock())
                tr->poll(idx_);
    if (idx_ == 0 && ex_->service_hook)
        ex_->service_hook();
    size_t n = queue_.progress(iteration_, env_data::get().strict_order);
    if (env_data::get().queue_dump && (iteration_ & 0xfffff) == 0 && !queue_.empty()) {
        std::string d;
        queue_.dump(d);
        LOG_INFO("worker ", idx_, " queue:", d);
    }
    return n;
}

void worker::loop() {
    tid_ = std::this_thread::get_id();
    const env_data& env = env_data::get();
    {
        std::string nm = "ccl_worker_" + std::to_string(idx_);
        pthread_setname_np(pthread_self(), nm.c_str());
        trace_name_thread(nm.c_str());
    }
    int cpu = -1;
    if ((size_t)idx_ < env.worker_affinity.size())
        cpu = env.worker_affinity[idx_];
    else if (env.worker_affinity_auto) {
        const numa_info& numa = numa_info::get();
        const auto cpus = numa_info::auto_worker_cpus(numa.allowed_cpus(), env.local_rank, env.local_size,
                                                      env.worker_count);
        if ((size_t)idx_ < cpus.size())
            cpu = cpus[idx_];
    }
    if (cpu >= 0) {
        cpu_set_t set;
        CPU_ZERO(&set);
        CPU_SET(cpu, &set);
        if (pthread_setaffinity_np(pthread_self(), sizeof(set), &set) != 0)
            LOG_WARN("can not pin worker ", idx_, " to core ", cpu);
        else
            LOG_DEBUG("worker ", idx_, " pinned to core ", cpu);
    }
    // staging memory the worker touches first lands on its own NUMA node
    int node = (size_t)idx_ < env.worker_mem_affinity.size() ? env.worker_mem_affinity[idx_]
                                                              : (cpu >= 0 ? numa_info::get().node_of_cpu(cpu) : -1);
    if (node >= 0 && numa_info::get().node_count() > 1 && !numa_info::get().bind_thread_memory(node))
        LOG_DEBUG("worker ", idx_, ": memory policy for node ", node, " not applied");
    int idle_spins = 0;
    while (!stop_) {
        size_t n = 0;
        try {
            n = do_work();
        }
        catch (const std::exception& e) {
            if (!stop_)
                LOG_ERROR("worker ", idx_, ": ", e.what());
            std::this_thread::sleep_for(std::chrono::milliseconds(10));
        }
        if (n > 0) {
            idle_spins = 0;
            continue;
        }
        if (++idle_spins < env.spin_count) {
            switch (env.yield) {
                case yield_t::pause:
#if defined(__x86_64__)
                    __builtin_ia32_pause();
#endif
                    break;
                case yield_t::sched_yield: ::sched_yield(); break;
                case yield_t::sleep: std::this_thread::sleep_for(std::chrono::microseconds(1)); break;
                default: break;
            }
            continue;
        }
        idle_spins = 0;
        if (env.worker_wait && queue_.empty()) {
            // nothing queued: sleep until work arrives (bounded, so that the service hook keeps its cadence)
            std::unique_lock<std::mutex> lk(mu_);
            cv_.wait_for(lk, std::chrono::microseconds(idx_ == 0 && ex_->service_hook ? 200 : 2000));
        }
    }
}

// ---- executor -------------------------------------------------------------------------
executor& executor::get() {
    static executor inst;
    return inst;
}

void executor::ensure_started(std::shared_ptr<atl_transport> tr) {
    std::lock_guard<std::mutex> lk(mu_);
    if (tr) {
        // copy-on-write list: workers read a snapshot without taking a lock; dead entries are dropped here
        auto next = std::make_shared<transport_list>();
        bool known = false;
        if (auto cur = std::atomic_load(&transports_))
            for (auto& w : *cur)
                if (auto live = w.lock()) {
                    next->push_back(w);
                    known = known || live == tr;
                }
        if (!known)
            next->push_back(tr);
        std::atomic_store(&transports_, std::shared_ptr<const transport_list>(next));
    }
    if (!workers_.empty())
        return;
    const env_data& env = env_data::get();
    for (int i = 0; i < env.worker_count; i++)
        workers_.emplace_back(new worker(this, i));
    if (env.worker_offload)
        for (auto& w : workers_)
            w->start();
    LOG_DEBUG("executor started: ", env.worker_count, " worker(s), offload=", env.worker_offload);
}

executor::~executor() {
    // workers poll the transport: stop them before the transport goes away
    shutdown();
}

void executor::shutdown() {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& w : workers_)
        w->stop();
    workers_.clear();
    std::atomic_store(&transports_, std::shared_ptr<const transport_list>());
    service_hook = nullptr;
}

void executor::launch_now(master_sched* m) {
    auto& parts = m->partials();
    m->req().arm((int)parts.size());
    for (auto& p : parts) // a partial built for endpoint e runs on worker e
        workers_[p->ep() % workers_.size()]->add(p.get());
}

uint64_t executor::start(master_sched* m, uint64_t new_id) {
    CCL_THROW_IF_NOT(!workers_.empty(), "executor is not running");
    if (!m->req().on_last) {
        m->req().on_last = [this, m] {
            if (m->user_complete && !m->req().has_error())
                m->user_complete();
            bool again = false;
            uint64_t next_id = KEEP_ID;
            {
                std::lock_guard<std::mutex> lk(m->launch_mu);
                if (m->delayed_launches > 0) {
                    m->delayed_launches--;
                    again = true;
                    next_id = m->pending_ids.front();
                    m->pending_ids.pop_front();
                }
                else
                    m->in_flight = false;
            }
            if (again) {
                for (auto& p : m->partials())
                    p->reset();
                if (next_id != KEEP_ID)
                    m->renew_id(next_id);
            }
            m->done.fetch_add(1, std::memory_order_acq_rel);
            if (again)
                launch_now(m);
        };
    }
    const uint64_t ticket = m->issued.fetch_add(1) + 1;
    bool now = false;
    {
        std::lock_guard<std::mutex> lk(m->launch_mu);
        if (m->in_flight) {
            m->delayed_launches++;
            m->pending_ids.push_back(new_id);
        }
        else {
            m->in_flight = true;
            now = true;
        }
    }
    if (now) {
        if (ticket > 1)
            for (auto& p : m->partials())
                p->reset();
        if (new_id != KEEP_ID)
            m->renew_id(new_id);
        launch_now(m);
    }
    return ticket;
}

bool executor::test(master_sched* m, uint64_t ticket) {
    if (m->ticket_complete(ticket))
        return true;
    if (!env_data::get().worker_offload)
        for (auto& w : workers_)
            w->do_work();
    return m->ticket_complete(ticket);
}

void executor::wait(master_sched* m, uint64_t ticket) {
    const env_data& env = env_data::get();
    m->req().urgent.store(true, std::memory_order_release);
    int spins = 0;
    while (!m->ticket_complete(ticket)) {
        if (!env.worker_offload) {
            for (auto& w : workers_)
                w->do_work();
            continue;
        }
        if (++spins > env.spin_count) {
            std::this_thread::yield();
            spins = 0;
        }
    }
    m->req().urgent.store(false, std::memory_order_release);
    if (m->req().has_error())
        CCL_THROW("collective failed: ", m->req().error());
}

void executor::progress() {
    if (!env_data::get().worker_offload)
        for (auto& w : workers_)
            w->do_work();
    else
        std::this_thread::yield();
}

void executor::lock_workers() {
    freeze_mu_.lock();
    frozen_.store(true, std::memory_order_release);
}

void executor::unlock_workers() {
    frozen_.store(false, std::memory_order_release);
    freeze_mu_.unlock();
}

// ---- cache ----------------------------------------------------------------------------
std::shared_ptr<master_sched> sched_cache::find(const std::string& key) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = map_.find(key);
    if (it == map_.end()) {
        misses++;
        return nullptr;
    }
    hits++;
    it->second.last_use = ++clock_;
    return it->second.m;
}

void sched_cache::insert(const std::string& key, std::shared_ptr<master_sched> m) {
    std::lock_guard<std::mutex> lk(mu_);
    const size_t cap = std::max<size_t>(env_data::get().sched_cache_max_entries, 1);
    while (map_.size() >= cap) {
        auto victim = map_.end();
        for (auto it = map_.begin(); it != map_.end(); ++it)
            if (it->second.m->idle() && (victim == map_.end() || it->second.last_use < victim->second.last_use))
                victim = it;
        if (victim == map_.end())
            break; // everything is running: exceed the bound rather than wait
        map_.erase(victim);
        evictions++;
    }
    m->cached = true;
    m->cache_key = key;
    slot& s = map_[key];
    s.m = std::move(m);
    s.last_use = ++clock_;
}

void sched_cache::flush() {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto it = map_.begin(); it != map_.end();) {
        if (it->second.m->idle())
            it = map_.erase(it);
        else
            ++it;
    }
}

size_t sched_cache::size() {
    std::lock_guard<std::mutex> lk(mu_);
    return map_.size();
}

} // namespace cclx
