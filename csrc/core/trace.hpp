// Tracing ranges for profilers (NVTX v3, header-only: free unless a tool injects itself).
//
// Marks the same points the reference annotates with ITT (domain "oneCCL::API":
// one task per API call carrying the payload size, src/coll/coll.cpp:136-150; one
// event per schedule entry, src/sched/entry/entry.cpp:60-63,108-111), gated by the
// same level knob: CCL_ITT_LEVEL=1 API calls, 2 also schedule entries.
#pragma once
#include <cstdint>

namespace cclx {

int trace_level();
void trace_push(const char* name, uint64_t payload);
void trace_pop();
void trace_mark(const char* name);
void trace_name_thread(const char* name);

class trace_range {
public:
    trace_range(int level, const char* name, uint64_t payload = 0) : on_(trace_level() >= level) {
        if (on_)
            trace_push(name, payload);
    }
    ~trace_range() {
        if (on_)
            trace_pop();
    }
    trace_range(const trace_range&) = delete;
    trace_range& operator=(const trace_range&) = delete;

private:
    bool on_;
};

} // namespace cclx
