// Host-side owner of one node communicator's device state, and the launch
// entry points of the collective kernels.
//
// Role in the layer map: this is the replacement of the reference's SYCL
// collective runtime (coll_init / invoke_collective / size dispatch,
// src/coll/algorithms/utils/sycl_coll_base.cpp:200-302, sycl_coll_base.hpp:351-408,
// sycl_selection.cpp:18-155): one-time exchange of barrier counters and
// temporary buffers per communicator, then per-call selection by message size
// and a kernel launch on the caller's stream.  Nothing here touches the CPU
// scheduler or worker threads.
#pragma once
#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <vector>

#include "core/types.hpp"
#include "gpu/device/coll_args.hpp"
#include "gpu/device/layout.hpp"
#include "gpu/symm_heap.hpp"

namespace cclx {
namespace gpu {

enum gpu_algo : int {
    ga_auto = 0,
    ga_oneshot, // push + local reduce, staged
    ga_twoshot, // reduce-scatter + allgather through staging
    ga_symm, // zero-copy peer loads/stores on symmetric buffers
    ga_nvls, // multimem on symmetric buffers
    ga_nvls_oneshot, // one-shot with a multimem.st push
    ga_push, // allgather: push into peers' staging
    ga_pull, // allgather: pull from peers' staging
    ga_copy, // single rank / local copy
    ga_pipelined, // allreduce: chunk pipeline through staging (copy in | reduce + broadcast | copy out)
    ga_ce, // allgather on symmetric / registered buffers by the copy engines (no SM time between two barriers)
    ga_last
};
const char* gpu_algo_name(int a);
int gpu_algo_from_name(const std::string& s); // -1 when unknown

class buffer_exchange;

class device_comm {
public:
    device_comm() = default;
    ~device_comm();
    device_comm(const device_comm&) = delete;
    device_comm& operator=(const device_comm&) = delete;

    void init(bootstrap_if& bs); // real: one process per GPU (device already current)
    void init_emulated(int world, size_t heap_bytes, size_t staging_bytes);
    void destroy();

    int rank() const { return rank_; }
    int world() const { return world_; }
    bool emulated() const { return emulated_; }
    bool nvls() const { return heap_.has_multicast(); }
    symm_heap& heap() { return heap_; }
    const dev::comm_dev* table() const { return table_dev_; }
    const dev::comm_dev& host_entry(int r) const { return table_host_[r]; }
    const dev::p2p_layout& p2p() const { return p2p_; }
    int sm_count() const { return sm_count_; }
    int max_blocks() const; // per rank, keeps every block co-resident
    int threads() const { return threads_; }
    dev::rank_args* emu_args_dev() const { return emu_args_dev_; }
    dev::p2p_ops* emu_ops_dev() const { return emu_ops_dev_; }
    int device_id() const { return device_id_; }
    size_t staging_bytes() const { return heap_.regions().staging_bytes; }

    // error status written by kernels (0 = ok); throws with a description when set
    uint32_t status_code(int r = 0) const;
    void check_status() const;
    void clear_status();
    void abort(); // raise the abort flag polled by every device-side wait
    void set_timeout_ms(size_t ms);

    // symmetric allocation helpers (collective in real mode)
    void* symm_alloc(size_t bytes, int emu_rank = 0);
    void symm_free(void* p, int emu_rank = 0);
    // offset of p inside the heap of `owner` (emulated rank or my rank), -1 if not symmetric
    size_t symm_offset(const void* p, int owner = -1) const;

    // Registration of ordinary device allocations (not from the symmetric heap) for zero-copy peer
    // access: collective; every rank passes its own buffer (emulation: one per emulated rank).  The
    // owners' allocations are exported with the CUDA IPC handle of their base allocation and mapped
    // by every peer once; collectives on a registered buffer must use the same offset inside it on
    // every rank.  Returns the registration id.
    int register_user(void* const* ptrs, const size_t* bytes);
    void deregister_user(int id);
    // registration that contains [p, p + len) of `owner` (emulated rank, or this rank when -1)
    bool find_user(const void* p, size_t len, int owner, int& id, size_t& off) const;
    // pointer of rank q's buffer of registration `id`, as mapped in this process
    char* user_base(int id, int q) const { return regs_[id].base[q]; }

    // state of the fused small-message allreduce (launch_allreduce_fused): one buffer in the symmetric heap
    // that the tensors of a batch are packed into, and a ring of pinned pointer / offset tables that the
    // pack kernels read while the host already fills the next one
    struct fuse_state {
        size_t buf_off = (size_t)-1; // heap offset of the fused buffer
        size_t buf_bytes = 0;
        static constexpr int SLOTS = 8, MAX_TENSORS = 1024;
        char* tab_host = nullptr; // SLOTS x entries x MAX_TENSORS x (pointer, offset, byte length)
        char* tab_dev = nullptr;
        cudaEvent_t used[SLOTS] = {};
        int next = 0;
        unsigned long long batches = 0, tensors = 0;
    };
    fuse_state& fuse() { return fuse_; }

    // automatic sharing of ordinary buffers (multi-process mode with CCL_CUDA_AUTO_REGISTER=1), else null
    buffer_exchange* exchange() const { return exch_.get(); }

    // test hook: rank + 1 whose argument signature is falsified in the next collectives (0 = none), so that
    // the cross-rank argument check can be exercised with all ranks emulated on one GPU
    int test_sig_skew = 0;

    // per-algorithm launch counters (observability)
    std::vector<unsigned long long> algo_hits = std::vector<unsigned long long>(ga_last * (int)coll_last, 0);

private:
    void build_tables();
    struct user_reg {
        bool live = false;
        std::vector<char*> base; // per rank, as seen from this process
        std::vector<size_t> bytes;
        std::vector<void*> opened; // IPC mappings this registration holds (closed on deregistration)
    };
    std::vector<user_reg> regs_;
    fuse_state fuse_;
    std::shared_ptr<buffer_exchange> exch_; // shared_ptr: the type is incomplete in this header
    bootstrap_if* bs_ = nullptr;
    int rank_ = 0, world_ = 0;
    bool emulated_ = false;
    symm_heap heap_;
    std::vector<dev::comm_dev> table_host_;
    dev::comm_dev* table_dev_ = nullptr;
    dev::p2p_layout p2p_{};
    uint32_t* state_dev_ = nullptr; // per emulated rank STATE_WORDS
    uint32_t* p2p_seq_dev_ = nullptr;
    uint32_t* status_host_ = nullptr; // pinned + mapped: per rank 8 words, then abort word
    uint32_t* status_devptr_ = nullptr;
    dev::rank_args* emu_args_dev_ = nullptr;
    dev::p2p_ops* emu_ops_dev_ = nullptr;
    int device_id_ = 0;
    int sm_count_ = 0;
    int threads_ = 512;
    size_t timeout_ms_ = 20000;
};

// ---- launchers -------------------------------------------------------------------
// `ra` points at one rank_args in real mode and at world() entries in
// emulation mode.  Counts are in elements of dt_in unless stated.
struct launch_opts {
    int algo = ga_auto;
    int blocks = 0; // 0 = automatic
    float scale = 1.0f;
    bool do_scale = false;
    // alltoall: every rank passes the same single block size (lets the grid follow the size and
    // enables the direct path into symmetric buffers)
    bool uniform = false;
};

void launch_allreduce(device_comm& dc, const dev::rank_args* ra, size_t count, int dt_in, int dt_out, int op,
                      const launch_opts& o, cudaStream_t st);
void launch_reduce_scatter(device_comm& dc, const dev::rank_args* ra, size_t recv_count, int dt_in, int dt_out,
                           int op, const launch_opts& o, cudaStream_t st);
void launch_reduce(device_comm& dc, const dev::rank_args* ra, size_t count, int dt_in, int dt_out, int op,
                   int root, const launch_opts& o, cudaStream_t st);
// scount/sdispl of ra[*] in BYTES: block sizes / offsets inside recv (identical on every rank)
void launch_allgatherv(device_comm& dc, const dev::rank_args* ra, const launch_opts& o, cudaStream_t st);
// debug: scans a floating-point result for NaN / Inf and records ST_NOT_FINITE in the status words
void launch_check_finite(device_comm& dc, const void* buf, size_t count, int dt, cudaStream_t st);
// scount/sdispl/rcount/rdispl of ra[*] in BYTES
void launch_alltoallv(device_comm& dc, const dev::rank_args* ra, const launch_opts& o, cudaStream_t st);
void launch_broadcast(device_comm& dc, const dev::rank_args* ra, size_t bytes, int root, const launch_opts& o,
                      cudaStream_t st);
void launch_barrier(device_comm& dc, cudaStream_t st);
// point to point: `ops` has one entry in real mode and world() entries in emulation mode; all
// operations of a list run in one launch per round (send/recv of a group)
void launch_sendrecv(device_comm& dc, const dev::p2p_ops* ops, cudaStream_t st);
// a wait that nothing satisfies; returns after the device time limit with status ST_FLAG_TIMEOUT
void launch_wait_unset_flag(device_comm& dc, cudaStream_t st);

// local helpers
void launch_reduce_local(const void* in, void* inout, size_t count, int dt, int op, cudaStream_t st);
void launch_transpose_blocks(const void* in, void* out, int rows, int cols, size_t block_bytes, cudaStream_t st);
void launch_pack(const void* const* ptrs_dev, const size_t* offs_dev, const size_t* lens_dev, int n, void* fused,
                 bool unpack, size_t max_tensor_bytes, cudaStream_t st);

// Small-message fusion on the device (the reference's fusion manager builds copy-in -> allreduce -> copy-out
// schedules on the host, src/fusion/fusion.cpp:145-376): `n` tensors per rank are packed into one buffer of
// the symmetric heap by one kernel, reduced by ONE zero-copy allreduce and unpacked by one kernel.  `send` and
// `recv` hold n pointers per entry, tensor-major ([k * entries + e]; entries = world() in emulation mode, else
// 1); `counts` n element counts.  Tensors that do not fit the fused buffer are reduced one by one.
void launch_allreduce_fused(device_comm& dc, const void* const* send, void* const* recv, const size_t* counts, int n,
                            int dt, int op, const launch_opts& o, cudaStream_t st);

int selected_allreduce_algo(const device_comm& dc, size_t bytes, bool symmetric, int dt, int op);

} // namespace gpu
} // namespace cclx
