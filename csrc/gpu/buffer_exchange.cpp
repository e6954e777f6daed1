#include "gpu/buffer_exchange.hpp"

#include <fcntl.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstring>

#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/device_comm.hpp"

namespace cclx {
namespace gpu {

buffer_exchange::buffer_exchange(device_comm& dc, bootstrap_if& bs) : dc_(dc), rank_(bs.rank()), world_(bs.size()) {
    // rank 0 creates the mailbox, the others attach; the name travels through the bootstrap
    char name[64] = {};
    char all[dev::MAX_RANKS * 64] = {};
    box_bytes_ = (size_t)world_ * SLOTS * sizeof(record);
    int fd = -1;
    if (rank_ == 0) {
        static std::atomic<int> counter{ 0 };
        std::snprintf(name, sizeof(name), "/cclx_bx_%d_%d", (int)getpid(), counter.fetch_add(1));
        fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
        CCL_THROW_IF_NOT(fd >= 0, "shm_open(", name, ") failed: ", strerror(errno));
        CCL_THROW_IF_NOT(ftruncate(fd, (off_t)box_bytes_) == 0, "ftruncate of the buffer mailbox failed");
    }
    bs.allgather(name, all, 64);
    if (rank_ != 0) {
        fd = shm_open(all, O_RDWR, 0600);
        CCL_THROW_IF_NOT(fd >= 0, "shm_open(", all, ") failed: ", strerror(errno));
    }
    void* m = mmap(nullptr, box_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    CCL_THROW_IF_NOT(m != MAP_FAILED, "mmap of the buffer mailbox failed");
    box_ = (record*)m; // a fresh segment is zero: sequence numbers start at 0, the first call uses 1
    bs.barrier();
    if (rank_ == 0)
        shm_unlink(all);
}

buffer_exchange::~buffer_exchange() {
    for (auto& e : lru_)
        cudaIpcCloseMemHandle(e.mapped);
    if (box_)
        munmap(box_, box_bytes_);
}

buf_desc buffer_exchange::describe(const void* p, size_t bytes) {
    buf_desc d;
    std::memset(&d, 0, sizeof(d));
    if (!p || (((uintptr_t)p) & 15))
        return d;
    const size_t hoff = dc_.symm_offset(p);
    if (hoff != (size_t)-1) {
        d.kind = bk_heap;
        d.off = hoff;
        return d;
    }
    int id = -1;
    size_t off = 0;
    if (dc_.find_user(p, bytes, -1, id, off)) {
        d.kind = bk_registered;
        d.reg_id = (uint32_t)id;
        d.off = off;
        return d;
    }
    const driver_api& drv = driver();
    if (!drv.PointerGetAttributes)
        return d;
    unsigned long long bid = 0;
    CUdeviceptr start = 0;
    size_t range = 0;
    int ipc_ok = 0;
    unsigned int mtype = 0;
    CUpointer_attribute attrs[5] = { CU_POINTER_ATTRIBUTE_BUFFER_ID, CU_POINTER_ATTRIBUTE_RANGE_START_ADDR,
                                     CU_POINTER_ATTRIBUTE_RANGE_SIZE, CU_POINTER_ATTRIBUTE_IS_LEGACY_CUDA_IPC_CAPABLE,
                                     CU_POINTER_ATTRIBUTE_MEMORY_TYPE };
    void* vals[5] = { &bid, &start, &range, &ipc_ok, &mtype };
    if (drv.PointerGetAttributes(5, attrs, vals, (CUdeviceptr)p) != CUDA_SUCCESS)
        return d;
    if (mtype != CU_MEMORYTYPE_DEVICE || !ipc_ok || bid == 0 || (const char*)p + bytes > (const char*)start + range)
        return d;
    // Small cudaMalloc allocations are carved out of one 2 MiB page by the driver, and the IPC handle names the
    // page: two such buffers would ask the peer to open one handle twice (cudaErrorAlreadyMapped), and the offset
    // of a buffer inside the opened mapping would not be its offset from RANGE_START.  Share only allocations
    // that own their pages: 2 MiB-aligned start, at least 2 MiB long (every block of PyTorch's caching allocator,
    // every cudaMalloc from 2 MiB on).  The others are staged.
    constexpr size_t PAGE = 2u << 20;
    if ((((uintptr_t)start) & (PAGE - 1)) != 0 || range < PAGE)
        return d;
    auto it = own_handles_.find(bid);
    if (it == own_handles_.end()) {
        cudaIpcMemHandle_t h;
        if (cudaIpcGetMemHandle(&h, (void*)start) != cudaSuccess) {
            (void)cudaGetLastError();
            return d;
        }
        if (own_handles_.size() > 4096)
            own_handles_.clear(); // ids of freed allocations pile up: start over, handles are cheap to get again
        it = own_handles_.emplace(bid, h).first;
    }
    d.kind = bk_ipc;
    d.buffer_id = bid;
    d.off = (uint64_t)((const char*)p - (const char*)start);
    d.handle = it->second;
    return d;
}

char* buffer_exchange::resolve(int q, const buf_desc& d) {
    if (d.kind == bk_heap)
        return dc_.heap().base(q) + d.off;
    if (d.kind == bk_registered)
        return dc_.user_base((int)d.reg_id, q) + d.off;
    // bk_ipc
    auto key = std::make_pair(q, (uint64_t)d.buffer_id);
    auto it = index_.find(key);
    if (it != index_.end()) {
        lru_.splice(lru_.end(), lru_, it->second); // most recently used
        hits++;
        return (char*)it->second->mapped + d.off;
    }
    const size_t cap = std::max<size_t>(env_data::get().ipc_cache_entries, 8);
    if (lru_.size() >= cap) {
        // the mapping may still be in use by a kernel in flight: drain the device before closing it
        CUDA_CHECK(cudaDeviceSynchronize());
        opened_entry old = lru_.front();
        cudaIpcCloseMemHandle(old.mapped);
        index_.erase(std::make_pair(old.rank, old.buffer_id));
        lru_.pop_front();
        evicted++;
    }
    void* mapped = nullptr;
    CUDA_CHECK(cudaIpcOpenMemHandle(&mapped, d.handle, cudaIpcMemLazyEnablePeerAccess));
    lru_.push_back({ q, d.buffer_id, mapped });
    index_[key] = std::prev(lru_.end());
    opened++;
    return (char*)mapped + d.off;
}

void buffer_exchange::exchange(const void* send, size_t send_bytes, void* recv, size_t recv_bytes, shared_view& in,
                               shared_view& out) {
    calls++;
    const uint64_t seq = ++seq_;
    record* mine = slot(rank_, seq);
    mine->side[0] = describe(send, send_bytes);
    mine->side[1] = describe(recv, recv_bytes);
    mine->seq.store(seq, std::memory_order_release);

    const auto t0 = std::chrono::steady_clock::now();
    const auto limit = std::chrono::milliseconds(std::max<size_t>(env_data::get().wait_timeout_ms, 1000));
    buf_desc theirs[dev::MAX_RANKS][2];
    for (int q = 0; q < world_; q++) {
        record* r = slot(q, seq);
        for (uint64_t it = 0; r->seq.load(std::memory_order_acquire) != seq; it++) {
            if ((it & 0xff) == 0xff) {
                sched_yield();
                if (std::chrono::steady_clock::now() - t0 > limit)
                    CCL_THROW("rank ", q, " did not join the buffer exchange of collective call ", seq,
                              " (every rank must issue the same collectives in the same order)");
            }
        }
        theirs[q][0] = r->side[0];
        theirs[q][1] = r->side[1];
    }
    // A slot is reused SLOTS calls later; a peer can be at most one call ahead of the slowest reader because
    // it waits for everybody's record of its current call, so the copies above cannot be overwritten early.
    const void* asked[2] = { send, recv };
    shared_view* views[2] = { &in, &out };
    for (int s = 0; s < 2; s++) {
        shared_view& v = *views[s];
        v = shared_view();
        if (!asked[s])
            continue;
        bool all = true, heap = true;
        for (int q = 0; q < world_; q++) {
            all = all && theirs[q][s].kind != bk_none;
            heap = heap && theirs[q][s].kind == bk_heap && theirs[q][s].off == theirs[0][s].off;
        }
        if (!all)
            continue;
        for (int q = 0; q < world_; q++)
            v.ptr[q] = q == rank_ ? (char*)asked[s] : resolve(q, theirs[q][s]);
        v.ok = true;
        v.heap_equal = heap;
        v.heap_off = heap ? (size_t)theirs[0][s].off : 0;
    }
}

} // namespace gpu
} // namespace cclx
