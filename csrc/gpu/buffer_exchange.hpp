// Automatic sharing of ordinary device buffers between the ranks of one node.
//
// Role in the layer map: the reference's per-operation handle exchange and its caches
// (ze_handle_exchange_entry: src/sched/entry/ze/ze_handle_exchange_entry.cpp:95-257; pointer -> allocation
// base + offset and the cache of opened handles: src/sched/ze/ze_handle_manager.cpp:292-335,
// src/sched/entry/ze/cache/ze_cache.hpp:212-262).  A collective on buffers that were not allocated from
// the symmetric heap first tells the peers where its buffers live: the allocation they belong to
// (CUDA buffer id, IPC handle of the allocation's base) and the offset inside it.  The exchange goes
// through a small shared-memory mailbox (one record per rank and call, a sequence number written last),
// so it costs a few memory accesses once the peers have arrived.  Every rank then maps the peers'
// allocations it has not seen yet (cudaIpcOpenMemHandle, kept in an LRU keyed by rank and buffer id) and
// ends up with one pointer per peer; all ranks take the same decision because all of them see the same
// records.  Unlike the symmetric heap, offsets may differ between ranks.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <list>
#include <map>
#include <string>
#include <vector>

#include "gpu/device/layout.hpp"
#include "gpu/symm_heap.hpp"

namespace cclx {
namespace gpu {

class device_comm;

// how one rank's buffer can be reached by its peers
enum buf_kind : uint32_t {
    bk_none = 0, // not shareable (null, unaligned, managed / virtual-memory allocation without IPC support)
    bk_heap = 1, // inside the symmetric heap: `off` is the heap offset
    bk_registered = 2, // inside an explicit registration: `reg_id`, `off` inside it
    bk_ipc = 3 // ordinary cudaMalloc allocation: `buffer_id`, `handle` of its base, `off` inside it
};

struct buf_desc {
    uint32_t kind;
    uint32_t reg_id;
    uint64_t off;
    uint64_t buffer_id;
    cudaIpcMemHandle_t handle;
};

// result for one side (send or recv) of a collective
struct shared_view {
    bool ok = false; // every rank's buffer is reachable: ptr[] is valid
    bool heap_equal = false; // all in the symmetric heap at the same offset (multicast window usable)
    size_t heap_off = 0;
    char* ptr[dev::MAX_RANKS] = {};
};

class buffer_exchange {
public:
    buffer_exchange(device_comm& dc, bootstrap_if& bs);
    ~buffer_exchange();
    buffer_exchange(const buffer_exchange&) = delete;

    // Collective among the ranks of the communicator, in call order.  `send` / `recv` may be null (side not
    // asked for).  Blocks until every peer has published its record for the same call.
    void exchange(const void* send, size_t send_bytes, void* recv, size_t recv_bytes, shared_view& in,
                  shared_view& out);

    // observability
    unsigned long long calls = 0, opened = 0, evicted = 0, hits = 0;

private:
    struct record {
        std::atomic<uint64_t> seq;
        buf_desc side[2];
    };
    static constexpr int SLOTS = 4;
    record* slot(int rank, uint64_t seq) { return box_ + (size_t)rank * SLOTS + (seq % SLOTS); }
    buf_desc describe(const void* p, size_t bytes);
    char* resolve(int q, const buf_desc& d);

    device_comm& dc_;
    int rank_, world_;
    record* box_ = nullptr;
    size_t box_bytes_ = 0;
    uint64_t seq_ = 0;
    // my own allocations: buffer id -> handle of the base
    std::map<uint64_t, cudaIpcMemHandle_t> own_handles_;
    // peers' allocations opened here, least recently used first
    struct opened_entry {
        int rank;
        uint64_t buffer_id;
        void* mapped;
    };
    std::list<opened_entry> lru_;
    std::map<std::pair<int, uint64_t>, std::list<opened_entry>::iterator> index_;
};

} // namespace gpu
} // namespace cclx
