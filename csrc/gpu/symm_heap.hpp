// Symmetric heap: one peer-mapped device allocation per rank, the CUDA
// replacement of the reference's per-collective Level Zero IPC handle exchange
// (src/sched/entry/ze/ze_handle_exchange_entry.cpp:95-257, fd transport modes of
// src/common/global/ze/ze_fd_manager.cpp:330-454).
//
// Design: instead of exchanging handles for user buffers on every collective
// and caching the opened handles, every rank creates ONE cuMem allocation at
// communicator creation, exports it (POSIX fd passed over Unix sockets with
// SCM_RIGHTS, or pidfd_getfd, or a fabric handle through the KVS), and maps
// all peers' allocations into its address space.  Flag arenas, point-to-point
// slots, staging generations and user "symmetric" tensors are carved out of
// that allocation at identical offsets on every rank.  When the GPUs support
// NVLS, the same physical memory is also bound to a multicast object, which
// gives `multimem` instructions a window over all replicas.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "core/env.hpp"

namespace cclx {
namespace gpu {

// out-of-band exchange used while setting up (implemented over the KVS)
class bootstrap_if {
public:
    virtual ~bootstrap_if() = default;
    virtual int rank() const = 0;
    virtual int size() const = 0;
    virtual void allgather(const void* send, void* recv, size_t bytes_per_rank) = 0;
    virtual void barrier() = 0;
    virtual std::string job_id() = 0; // same string on every rank, unique per communicator
};

struct heap_regions {
    size_t flags_off = 0; // barrier slots
    size_t p2p_flags_off = 0;
    size_t aux_flags_off = 0; // per-tile flags of the fused GEMM kernels, MoE counters
    size_t aux_flags_bytes = 0;
    size_t p2p_data_off = 0;
    size_t p2p_slot_bytes = 0;
    size_t staging_off = 0;
    size_t staging_bytes = 0; // one generation
    size_t user_off = 0;
    size_t total = 0;
};

heap_regions plan_regions(int world, size_t heap_bytes, size_t staging_bytes, size_t granularity);

class symm_heap {
public:
    symm_heap() = default;
    ~symm_heap();
    symm_heap(const symm_heap&) = delete;
    symm_heap& operator=(const symm_heap&) = delete;

    // real mode: one process per GPU, current device already selected
    void create(bootstrap_if& bs, size_t heap_bytes, size_t staging_bytes, ipc_exchange_t mode, int nvls);
    // emulation mode: `world` plain device allocations in this process
    void create_emulated(int world, size_t heap_bytes, size_t staging_bytes);
    void destroy();

    int world() const { return world_; }
    int rank() const { return rank_; }
    bool emulated() const { return emulated_; }
    bool has_multicast() const { return mc_base_ != nullptr; }
    const heap_regions& regions() const { return regions_; }
    // base address of rank p's heap as mapped in this process (emulated: heap of emulated rank p)
    char* base(int p) const { return bases_[p]; }
    char* mc_base() const { return mc_base_; }

    // collective (every rank must call in the same order with the same size);
    // returns an offset into the heap, 256-byte aligned
    size_t alloc(size_t bytes);
    void free(size_t off);
    size_t user_bytes_free() const;
    // offset of a local pointer inside my heap, or (size_t)-1
    size_t offset_of(const void* p, int owner_rank) const;

private:
    int rank_ = 0, world_ = 0;
    bool emulated_ = false;
    heap_regions regions_;
    std::vector<char*> bases_;
    char* mc_base_ = nullptr;
    // driver objects (opaque here)
    std::vector<unsigned long long> handles_; // CUmemGenericAllocationHandle per rank
    unsigned long long mc_handle_ = 0;
    bool mc_bound_ = false;
    size_t mapped_bytes_ = 0;
    int device_ = 0;
    // first-fit allocator over [user_off, total)
    std::map<size_t, size_t> free_; // off -> len
    std::map<size_t, size_t> used_; // off -> len
};

// exported for tests: pass `nfds` descriptors between processes over abstract
// Unix datagram sockets; every rank gives one fd and receives world-1
std::vector<int> exchange_fds_sockets(bootstrap_if& bs, int my_fd, const std::string& tag);
std::vector<int> exchange_fds_pidfd(bootstrap_if& bs, int my_fd);

} // namespace gpu
} // namespace cclx
