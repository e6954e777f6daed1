#include "gpu/device_comm.hpp"

#include <cstring>

#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/buffer_exchange.hpp"
#include "gpu/cuda_driver.hpp"

namespace cclx {
namespace gpu {

static const char* algo_names[] = { "auto", "oneshot", "twoshot", "symm", "nvls", "nvls_oneshot",
                                    "push", "pull",    "copy", "pipelined", "ce" };

const char* gpu_algo_name(int a) {
    return (a >= 0 && a < ga_last) ? algo_names[a] : "unknown";
}

int gpu_algo_from_name(const std::string& s) {
    for (int i = 0; i < ga_last; i++)
        if (s == algo_names[i])
            return i;
    return -1;
}

device_comm::~device_comm() {
    try {
        destroy();
    }
    catch (...) {
    }
}

void device_comm::init(bootstrap_if& bs) {
    const env_data& env = env_data::get();
    bs_ = &bs;
    rank_ = bs.rank();
    world_ = bs.size();
    emulated_ = false;
    timeout_ms_ = env.wait_timeout_ms;
    threads_ = env.cuda_block_threads;
    heap_.create(bs, env.symm_heap_bytes, env.tmp_buf_bytes, env.ipc_exchange, env.nvls);
    build_tables();
    if (env.auto_register && world_ > 1)
        exch_.reset(new buffer_exchange(*this, bs));
    bs.barrier();
}

void device_comm::init_emulated(int world, size_t heap_bytes, size_t staging_bytes) {
    const env_data& env = env_data::get();
    rank_ = 0;
    world_ = world;
    emulated_ = true;
    timeout_ms_ = env.wait_timeout_ms;
    threads_ = env.cuda_block_threads;
    heap_.create_emulated(world, heap_bytes, staging_bytes);
    build_tables();
}

void device_comm::build_tables() {
    int devid = 0;
    CUDA_CHECK(cudaGetDevice(&devid));
    CUDA_CHECK(cudaDeviceGetAttribute(&sm_count_, cudaDevAttrMultiProcessorCount, devid));
    const int entries = emulated_ ? world_ : 1;
    const heap_regions& R = heap_.regions();

    CUDA_CHECK(cudaMalloc((void**)&state_dev_, entries * dev::STATE_WORDS * sizeof(uint32_t)));
    CUDA_CHECK(cudaMemset(state_dev_, 0, entries * dev::STATE_WORDS * sizeof(uint32_t)));
    CUDA_CHECK(cudaMalloc((void**)&p2p_seq_dev_, entries * dev::P2P_SEQ_WORDS * sizeof(uint32_t)));
    CUDA_CHECK(cudaMemset(p2p_seq_dev_, 0, entries * dev::P2P_SEQ_WORDS * sizeof(uint32_t)));
    const size_t status_words = (size_t)entries * 8 + 8;
    CUDA_CHECK(cudaHostAlloc((void**)&status_host_, status_words * sizeof(uint32_t), cudaHostAllocMapped));
    std::memset(status_host_, 0, status_words * sizeof(uint32_t));
    CUDA_CHECK(cudaHostGetDevicePointer((void**)&status_devptr_, status_host_, 0));
    CUDA_CHECK(cudaMalloc((void**)&emu_args_dev_, dev::MAX_RANKS * sizeof(dev::rank_args)));
    CUDA_CHECK(cudaMalloc((void**)&emu_ops_dev_, dev::MAX_RANKS * sizeof(dev::p2p_ops)));
    device_id_ = devid;

    table_host_.assign(entries, dev::comm_dev{});
    for (int e = 0; e < entries; e++) {
        dev::comm_dev& c = table_host_[e];
        c.rank = emulated_ ? e : rank_;
        c.world = world_;
        for (int p = 0; p < world_; p++) {
            char* b = heap_.base(p);
            c.flags[p] = (uint32_t*)(b + R.flags_off);
            c.p2p_flags[p] = (uint32_t*)(b + R.p2p_flags_off);
            c.staging[p] = b + R.staging_off;
            c.aux[p] = (uint32_t*)(b + R.aux_flags_off);
            c.heap[p] = b;
        }
        c.mc_heap = heap_.mc_base();
        c.mc_staging = heap_.mc_base() ? heap_.mc_base() + R.staging_off : nullptr;
        c.mc_flags = heap_.mc_base() ? (uint32_t*)(heap_.mc_base() + R.flags_off) : nullptr;
        c.heap_bytes = R.total;
        c.staging_bytes = R.staging_bytes;
        c.state = state_dev_ + e * dev::STATE_WORDS;
        c.p2p_seq = p2p_seq_dev_ + e * dev::P2P_SEQ_WORDS;
        c.status = status_devptr_ + e * 8;
        c.abort_flag = status_devptr_ + entries * 8;
        c.timeout_ns = (unsigned long long)timeout_ms_ * 1000000ull;
    }
    CUDA_CHECK(cudaMalloc((void**)&table_dev_, entries * sizeof(dev::comm_dev)));
    CUDA_CHECK(cudaMemcpy(table_dev_, table_host_.data(), entries * sizeof(dev::comm_dev), cudaMemcpyHostToDevice));
    for (int p = 0; p < world_; p++)
        p2p_.data[p] = heap_.base(p) + R.p2p_data_off;
    p2p_.slot_bytes = R.p2p_slot_bytes;
    p2p_.pull = env_data::get().p2p_pull ? 1 : 0;
    p2p_.lanes = std::max(1, std::min(env_data::get().p2p_lanes, (int)dev::P2P_LANES));
    CUDA_CHECK(cudaDeviceSynchronize());
}

void device_comm::set_timeout_ms(size_t ms) {
    timeout_ms_ = ms;
    for (auto& c : table_host_)
        c.timeout_ns = (unsigned long long)ms * 1000000ull;
    if (table_dev_)
        CUDA_CHECK(cudaMemcpy(table_dev_, table_host_.data(), table_host_.size() * sizeof(dev::comm_dev),
                              cudaMemcpyHostToDevice));
}

void device_comm::destroy() {
    if (!table_dev_)
        return;
    cudaDeviceSynchronize();
    exch_.reset();
    if (fuse_.tab_host) {
        cudaFreeHost(fuse_.tab_host);
        for (auto& e : fuse_.used)
            cudaEventDestroy(e);
        fuse_ = fuse_state();
    }
    for (auto& r : regs_)
        for (void* m : r.opened)
            cudaIpcCloseMemHandle(m);
    regs_.clear();
    cudaFree(table_dev_);
    table_dev_ = nullptr;
    cudaFree(state_dev_);
    cudaFree(p2p_seq_dev_);
    cudaFree(emu_args_dev_);
    cudaFree(emu_ops_dev_);
    cudaFreeHost(status_host_);
    state_dev_ = p2p_seq_dev_ = nullptr;
    status_host_ = nullptr;
    emu_args_dev_ = nullptr;
    heap_.destroy();
}

int device_comm::max_blocks() const {
    const env_data& env = env_data::get();
    int cap = emulated_ ? std::max(1, sm_count_ / world_) : std::min((int)dev::MAX_BLOCKS, sm_count_);
    if (env.cuda_max_blocks > 0)
        cap = std::min(cap, env.cuda_max_blocks);
    return std::min(cap, (int)dev::MAX_BLOCKS);
}

uint32_t device_comm::status_code(int r) const {
    return status_host_ ? ((volatile uint32_t*)status_host_)[r * 8] : 0;
}

void device_comm::check_status() const {
    const int entries = emulated_ ? world_ : 1;
    for (int e = 0; e < entries; e++) {
        volatile uint32_t* s = (volatile uint32_t*)status_host_ + e * 8;
        if (s[0] != dev::ST_OK) {
            static const char* what[] = { "ok",           "barrier timeout", "aborted",
                                          "flag timeout", "mbarrier timeout", "bad arguments",
                                          "NaN or Inf in a reduction result (detail = element index)",
                                          "a peer called this collective with another buffer kind, offset or count "
                                          "(zero-copy collectives need the same symmetric offset on every rank)" };
            const char* w = s[0] < 8 ? what[s[0]] : "unknown";
            CCL_THROW("device communicator error on rank ", table_host_[e].rank, ": ", w, " (block ", s[1],
                      ", peer ", s[2], ", detail ", s[3], ")");
        }
    }
}

void device_comm::clear_status() {
    const int entries = emulated_ ? world_ : 1;
    std::memset(status_host_, 0, ((size_t)entries * 8 + 8) * sizeof(uint32_t));
}

void device_comm::abort() {
    if (status_host_) {
        const int entries = emulated_ ? world_ : 1;
        ((volatile uint32_t*)status_host_)[entries * 8] = 1;
    }
}

void* device_comm::symm_alloc(size_t bytes, int emu_rank) {
    // emulation: one allocation call reserves the same offset in every emulated heap
    size_t off = heap_.alloc(bytes);
    return heap_.base(emulated_ ? emu_rank : rank_) + off;
}

void device_comm::symm_free(void* p, int emu_rank) {
    size_t off = heap_.offset_of(p, emulated_ ? emu_rank : rank_);
    CCL_THROW_IF_NOT(off != (size_t)-1, "pointer is not in the symmetric heap");
    heap_.free(off);
}

// ---- registration of ordinary allocations ---------------------------------------------------
// Reference counterpart: ze_handle_exchange_entry + ipc_handle_manager (src/sched/entry/ze/
// ze_handle_exchange_entry.cpp:95-257, src/sched/ze/ze_handle_manager.cpp:292-335): the handle of the
// allocation's BASE plus the offset of the buffer inside it travel to the peers, which open the
// handle once.  Here the exchange happens at registration, not per operation.
int device_comm::register_user(void* const* ptrs, const size_t* bytes) {
    // every rank registers and deregisters in the same order, so the count is the same everywhere
    size_t live = 0;
    for (auto& g : regs_)
        live += g.live ? 1 : 0;
    CCL_THROW_IF_NOT(live < env_data::get().ipc_cache_entries, live,
                     " registered allocations are open (CCL_CUDA_IPC_CACHE_ENTRIES); deregister some first");
    user_reg r;
    r.live = true;
    r.base.assign(world_, nullptr);
    r.bytes.assign(world_, 0);
    if (emulated_) {
        for (int q = 0; q < world_; q++) {
            r.base[q] = (char*)ptrs[q];
            r.bytes[q] = bytes[q];
        }
    }
    else {
        CCL_THROW_IF_NOT(bs_ != nullptr, "communicator has no bootstrap for the handle exchange");
        struct wire {
            cudaIpcMemHandle_t handle;
            unsigned long long offset, bytes;
        } mine{}, zero{};
        const driver_api& d = driver();
        CUdeviceptr abase = 0;
        size_t asize = 0;
        CU_CHECK(d.MemGetAddressRange(&abase, &asize, (CUdeviceptr)ptrs[0]));
        CUDA_CHECK(cudaIpcGetMemHandle(&mine.handle, (void*)abase));
        mine.offset = (unsigned long long)((char*)ptrs[0] - (char*)abase);
        mine.bytes = bytes[0];
        std::vector<wire> all(world_, zero);
        bs_->allgather(&mine, all.data(), sizeof(wire));
        for (int q = 0; q < world_; q++) {
            r.bytes[q] = (size_t)all[q].bytes;
            if (q == rank_) {
                r.base[q] = (char*)ptrs[0];
                continue;
            }
            void* mapped = nullptr;
            CUDA_CHECK(cudaIpcOpenMemHandle(&mapped, all[q].handle, cudaIpcMemLazyEnablePeerAccess));
            r.opened.push_back(mapped);
            r.base[q] = (char*)mapped + all[q].offset;
        }
        bs_->barrier();
    }
    for (size_t i = 0; i < regs_.size(); i++)
        if (!regs_[i].live) {
            regs_[i] = std::move(r);
            return (int)i;
        }
    regs_.push_back(std::move(r));
    return (int)regs_.size() - 1;
}

void device_comm::deregister_user(int id) {
    CCL_THROW_IF_NOT(id >= 0 && id < (int)regs_.size() && regs_[id].live, "unknown registration ", id);
    if (!emulated_ && bs_) {
        CUDA_CHECK(cudaDeviceSynchronize());
        bs_->barrier(); // nobody still reads this rank's buffer
    }
    for (void* m : regs_[id].opened)
        cudaIpcCloseMemHandle(m);
    regs_[id] = user_reg();
}

bool device_comm::find_user(const void* p, size_t len, int owner, int& id, size_t& off) const {
    const int q = owner < 0 ? (emulated_ ? 0 : rank_) : owner;
    for (size_t i = 0; i < regs_.size(); i++) {
        const user_reg& r = regs_[i];
        if (!r.live)
            continue;
        const char* b = r.base[q];
        if ((const char*)p >= b && (const char*)p + len <= b + r.bytes[q]) {
            id = (int)i;
            off = (size_t)((const char*)p - b);
            return true;
        }
    }
    return false;
}

size_t device_comm::symm_offset(const void* p, int owner) const {
    if (owner < 0)
        owner = emulated_ ? 0 : rank_;
    return heap_.offset_of(p, owner);
}

} // namespace gpu
} // namespace cclx
