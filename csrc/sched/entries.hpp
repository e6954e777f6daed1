// Concrete schedule entries.  Each is a small state machine: start() posts the
// operation, update() polls it.  Counterparts in the reference:
// send/recv/recv_reduce/recv_copy (src/sched/entry/send_entry.hpp:73-131,
// recv_entry.hpp:55-85, recv_reduce_entry.hpp:80-135), reduce_local
// (reduce_local_entry.cpp:98-125), copy (copy/copy_entry.cpp), sync
// (sync_entry.hpp:25-75), function (function_entry.hpp:20-49), subsched
// (subsched_entry.hpp:22-202), deps (deps_entry.cpp:24-43), wait_value, probe,
// register / deregister / write (one-sided).
#pragma once
#include <cstring>
#include <functional>
#include <memory>
#include <vector>

#include "core/comp.hpp"
#include "sched/sched.hpp"

namespace cclx {

class send_entry : public sched_entry {
public:
    send_entry(sched* s, const void* buf, size_t bytes, int dst, uint64_t step, bool one_way = false)
            : sched_entry(s), buf_(buf), bytes_(bytes), dst_(dst), step_(step), one_way_(one_way) {}
    const char* name() const override { return "SEND"; }
    bool uses_credit() const override { return true; }
    void start() override;
    void update() override;
    // the buffer may be bound late (address known only when an earlier entry ran)
    void set_buf(const void* b) { buf_ = b; }

private:
    const void* buf_;
    size_t bytes_;
    int dst_;
    uint64_t step_;
    bool one_way_; // a user's point-to-point send: nothing comes back from dst_ meanwhile
    atl_req req_;
};

class recv_entry : public sched_entry {
public:
    recv_entry(sched* s, void* buf, size_t bytes, int src, uint64_t step)
            : sched_entry(s), buf_(buf), bytes_(bytes), src_(src), step_(step) {}
    const char* name() const override { return "RECV"; }
    void start() override;
    void update() override;

private:
    void* buf_;
    size_t bytes_;
    int src_;
    uint64_t step_;
    atl_req req_;
};

// receive `count` elements into a temporary, then inout = op(tmp, inout).  With a `local` operand the
// message lands in `inout` itself and inout = op(local, inout): an out-of-place reduction needs neither
// the temporary nor a copy of the local contribution into the result buffer first.
class recv_reduce_entry : public sched_entry {
public:
    recv_reduce_entry(sched* s, void* inout, size_t count, int dtype, int op, int src, uint64_t step,
                      reduction_fn_t fn = nullptr, void* tmp = nullptr, const void* local = nullptr);
    const char* name() const override { return "RECV_REDUCE"; }
    void start() override;
    void update() override;

private:
    void* inout_;
    size_t count_;
    int dtype_, op_, src_;
    uint64_t step_;
    reduction_fn_t fn_;
    void* tmp_;
    const void* local_;
    atl_req req_;
};

class reduce_local_entry : public sched_entry {
public:
    reduce_local_entry(sched* s, const void* in, void* inout, size_t count, int dtype, int op,
                       reduction_fn_t fn = nullptr)
            : sched_entry(s), in_(in), inout_(inout), count_(count), dtype_(dtype), op_(op), fn_(fn) {}
    const char* name() const override { return "REDUCE_LOCAL"; }
    void start() override;

private:
    const void* in_;
    void* inout_;
    size_t count_;
    int dtype_, op_;
    reduction_fn_t fn_;
};

class copy_entry : public sched_entry {
public:
    copy_entry(sched* s, const void* src, void* dst, size_t bytes) : sched_entry(s), src_(src), dst_(dst), bytes_(bytes) {}
    const char* name() const override { return "COPY"; }
    void start() override;

private:
    const void* src_;
    void* dst_;
    size_t bytes_;
};

class function_entry : public sched_entry {
public:
    function_entry(sched* s, std::function<void()> fn) : sched_entry(s), fn_(std::move(fn)) {}
    const char* name() const override { return "FUNCTION"; }
    void start() override {
        fn_();
        status_ = entry_status::complete;
    }

private:
    std::function<void()> fn_;
};

// Barrier across the partial schedules of one master: complete when every
// partial reached it.
struct sync_object {
    explicit sync_object(int n) : initial(n), counter(n) {}
    int initial;
    std::atomic<int> counter;
    std::atomic<int> visited{ 0 };
};

class sync_entry : public sched_entry {
public:
    sync_entry(sched* s, std::shared_ptr<sync_object> o) : sched_entry(s), obj_(std::move(o)) {}
    const char* name() const override { return "SYNC"; }
    void start() override;
    void update() override;
    void reset() override;

private:
    std::shared_ptr<sync_object> obj_;
};

// waits until *ptr (host memory) reaches a value: used to chain on device events polled by the host
class wait_value_entry : public sched_entry {
public:
    wait_value_entry(sched* s, const volatile uint64_t* ptr, uint64_t value, bool ge = true)
            : sched_entry(s), ptr_(ptr), value_(value), ge_(ge) {}
    const char* name() const override { return "WAIT_VALUE"; }
    void start() override { update(); }
    void update() override {
        uint64_t v = *ptr_;
        status_ = (ge_ ? v >= value_ : v == value_) ? entry_status::complete : entry_status::started;
    }

private:
    const volatile uint64_t* ptr_;
    uint64_t value_;
    bool ge_;
};

// One-sided operations (reference src/sched/entry/{register,deregister,write}_entry.hpp).  A region is
// registered when the entry runs, so a cached schedule registers anew on every run and the description
// it sends to its writers is always current.
class register_entry : public sched_entry {
public:
    register_entry(sched* s, void* buf, size_t bytes, atl_mr* out) : sched_entry(s), buf_(buf), bytes_(bytes), out_(out) {}
    const char* name() const override { return "REGISTER"; }
    void start() override;

private:
    void* buf_;
    size_t bytes_;
    atl_mr* out_;
};

class deregister_entry : public sched_entry {
public:
    deregister_entry(sched* s, atl_mr* mr) : sched_entry(s), mr_(mr) {}
    const char* name() const override { return "DEREGISTER"; }
    void start() override;

private:
    atl_mr* mr_;
};

// writes `bytes` from `buf`, or one 64-bit value, at `offset` of the region *mr; the region
// description is read when the entry starts (an earlier entry received it)
class write_entry : public sched_entry {
public:
    write_entry(sched* s, const void* buf, size_t bytes, const atl_mr* mr, uint64_t offset)
            : sched_entry(s), buf_(buf), bytes_(bytes), mr_(mr), offset_(offset) {}
    write_entry(sched* s, uint64_t value, const atl_mr* mr, uint64_t offset)
            : sched_entry(s), buf_(&value_), bytes_(sizeof(uint64_t)), mr_(mr), offset_(offset), value_(value) {}
    const char* name() const override { return "WRITE"; }
    bool uses_credit() const override { return true; }
    void start() override;
    void update() override;

private:
    const void* buf_;
    size_t bytes_;
    const atl_mr* mr_;
    uint64_t offset_;
    uint64_t value_ = 0;
    atl_req req_;
};

// dependency on caller-provided predicates (events of earlier operations)
class deps_entry : public sched_entry {
public:
    deps_entry(sched* s, std::vector<std::function<bool()>> deps) : sched_entry(s), deps_(std::move(deps)) {}
    const char* name() const override { return "DEPS"; }
    void start() override { update(); }
    void update() override {
        for (auto& d : deps_)
            if (!d()) {
                status_ = entry_status::started;
                return;
            }
        status_ = entry_status::complete;
    }

private:
    std::vector<std::function<bool()>> deps_;
};

class probe_entry : public sched_entry {
public:
    probe_entry(sched* s, int src, uint64_t step, size_t* out_len)
            : sched_entry(s), src_(src), step_(step), out_(out_len) {}
    const char* name() const override { return "PROBE"; }
    void start() override { update(); }
    void update() override;

private:
    int src_;
    uint64_t step_;
    size_t* out_;
};

// nested schedule built lazily by `builder` the first time the entry starts
class subsched_entry : public sched_entry {
public:
    // `other`: run the nested schedule on another communicator (sub-communicator phases)
    subsched_entry(sched* s, std::function<void(sched&)> builder, const char* label = "SUBSCHED",
                   host_comm* other = nullptr);
    const char* name() const override { return label_; }
    void start() override;
    void update() override;
    void reset() override;

private:
    std::function<void(sched&)> builder_;
    const char* label_;
    host_comm* other_;
    std::unique_ptr<sched> sub_;
};

} // namespace cclx
