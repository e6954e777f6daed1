// Environment configuration, parsed once into env_data.
//
// Keeps the portable knob names of the reference (src/common/env/vars.hpp:53-1176,
// defaults src/common/env/env.cpp:77-331) and adds the CUDA-side knobs
// (CCL_CUDA_*) that replace CCL_ZE_* / CCL_SYCL_*.  Parsing is a small typed
// helper per kind (int / size with K,M,G suffix / bool / enum / list), all
// values are printed at first communicator creation when the log level is
// info or higher.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "core/types.hpp"

namespace cclx {

enum class atl_transport_t { tcp, shm, ofi, mpi };
enum class priority_mode_t { none, direct, lifo };
enum class cache_key_t { full, match_id };
enum class yield_t { none, pause, sleep, sched_yield };
enum class launcher_t { hydra, torchrun, pmix, none };
enum class backend_t { native, stub };
enum class ipc_exchange_t { sockets, pidfd, fabric, cudaipc };

struct env_data {
    // logging / debug
    std::string log_level = "warn";
    bool abort_on_throw = false;
    bool sched_profile = false;
    bool sched_dump = false;
    bool queue_dump = false;
    double entry_max_update_time_sec = 0; // 0 = hang detector off
    int itt_level = 0; // NVTX range level (0 off, 1 API calls, 2 entries)

    // backend / launcher
    backend_t backend = backend_t::native;
    launcher_t process_launcher = launcher_t::hydra;
    int local_rank = -1;
    int local_size = -1;

    // workers
    int worker_count = 1;
    bool worker_offload = true;
    bool worker_wait = true;
    std::vector<int> worker_affinity; // explicit core per worker
    bool worker_affinity_auto = false; // CCL_WORKER_AFFINITY=auto: cores from the end of the allowed set
    std::vector<int> worker_mem_affinity;
    int spin_count = 1000;
    yield_t yield = yield_t::pause;

    // transport
    atl_transport_t atl_transport = atl_transport_t::tcp;
    bool atl_shm = true; // same-host pairs use the shared-memory rings
    size_t atl_shm_ring_bytes = 4u << 20;
    bool atl_rma = false; // CCL_ATL_RMA: one-sided writes (the ring_rma allreduce needs them)
    bool atl_cma = true; // CCL_ATL_CMA: cross-memory copies between processes of one host (one-sided writes, long messages)
    size_t atl_cma_threshold = 64u << 10; // messages of at least this size are read out of the sender's memory
    size_t max_short_size = 0;
    size_t chunk_count = 1;
    size_t min_chunk_size = 65536;
    int max_flow_credits = 16;

    // kvs
    std::string kvs_ip_port; // <ip>_<port>
    std::string kvs_ip_exchange = "path"; // env: the main KVS must find its address in CCL_KVS_IP_PORT
    std::string kvs_iface;
    bool kvs_prefer_ipv6 = false;
    int kvs_connection_timeout_sec = 120;
    int kvs_get_timeout_sec = 120;

    // algorithm selection: raw strings, parsed by the selector (coll/selection.cpp)
    std::map<int, std::string> algo_raw; // coll_type -> spec
    std::map<int, std::string> algo_scaleout_raw;
    std::map<int, std::string> algo_gpu_raw; // CCL_CUDA_<COLL>

    // ordering / caching / fusion
    bool unordered_coll = false;
    bool fusion = false;
    size_t fusion_bytes_threshold = 16384;
    size_t fusion_count_threshold = 256;
    priority_mode_t priority_mode = priority_mode_t::none;
    cache_key_t cache_key = cache_key_t::match_id;
    bool cache_flush = false;
    size_t sched_cache_max_entries = 4096; // per communicator
    bool strict_order = false;
    bool op_sync = false;
    bool buffer_cache = true; // CCL_BUFFER_CACHE=0: scratch memory is allocated and freed per schedule
    size_t buffer_cache_max_bytes = 256u << 20;
    bool algo_fallback = true; // CCL_ALGO_FALLBACK=0: an algorithm that cannot run is an error

    // allreduce tuning (CPU)
    size_t ar2d_chunk_count = 1;
    size_t ar2d_min_chunk_size = 65536;
    bool ar2d_switch_dims = false; // first dimension = across nodes
    size_t dtree_partition_count = 1;
    size_t bcast_part_count = 0; // 0 = as many parts as workers
    size_t nreduce_segment_size = 2u << 20;
    bool nreduce_buffering = false;
    size_t rs_chunk_count = 1;
    size_t rs_min_chunk_size = 65536;
    size_t alltoall_scatter_max_ops = 4;
    bool check_inplace_aliasing = true;

    // low precision on CPU: "auto" | "scalar" | "avx512f" | "f16c"
    std::string bf16_impl = "auto";
    std::string fp16_impl = "auto";

    // topology
    std::string topo_color = "fixed"; // fixed | cuda | env
    bool topo_algo = true;
    size_t allreduce_pipe_chunk_count = 0; // parts of a hierarchical device allreduce whose stages overlap (0 / 1: one part)
    std::string topo_p2p_access = "auto"; // auto | 0 | 1
    bool topo_fabric_check = false; // check peer access between all ranks' GPUs before the heap is mapped

    // CUDA device path
    bool cuda_kernels = true; // CCL_ENABLE_CUDA_KERNELS (reference CCL_ENABLE_SYCL_KERNELS)
    ipc_exchange_t ipc_exchange = ipc_exchange_t::sockets;
    size_t symm_heap_bytes = 1ull << 30; // peer-mapped heap per rank
    size_t tmp_buf_bytes = 128ull << 20; // one staging generation; two generations are kept
    int nvls = -1; // -1 auto, 0 off, 1 force
    int nvls_min_ranks = 3; // communicators smaller than this use peer loads even when NVLS exists
    size_t ar_oneshot_threshold = 256u << 10; // <= : one-shot
    size_t ar_pipelined_min = 512u << 10; // >= : ordinary buffers take the chunk pipeline
    int ar_pipelined_blocks = 128; // blocks of the chunk pipeline (few SMs: compute keeps the rest)
    bool cuda_check_nan = false; // debug: scan reduction results for NaN / Inf
    bool ag_gemm_ce = false; // all-gather -> GEMM: the copy engines gather, every SM computes (serial peer copies: pays only when the shards are large)
    bool gemm_rs_ring = true; // GEMM -> reduce-scatter: partial sums ride a ring through the epilogues
    bool gemm_2sm = true; // plain GEMMs run on CTA pairs (tcgen05 cta_group::2) when they have a 256-row tile
    size_t rs_small_threshold = 2u << 20;
    size_t rs_pipelined_min = 16u << 20; // total bytes >= : ordinary send buffers take the chunk pipeline
    size_t ag_small_threshold = 4u << 20; // per-rank block <= : push through staging; above: pull
    int cuda_max_blocks = 0; // 0 = auto (co-resident cap)
    int cuda_block_threads = 512;
    size_t wait_timeout_ms = 20000; // bound of every device-side wait
    bool cuda_copy_engine = false; // large equal-block allgather into symmetric / registered memory goes through the copy engines
    bool cuda_graph_safe = true;
    size_t ipc_cache_entries = 1000; // registered allocations that may be open at once
    std::string ofi_lib_path; // CCL_OFI_LIBRARY_PATH: libfabric.so to open for CCL_ATL_TRANSPORT=ofi
    std::string mpi_lib_path; // CCL_MPI_LIBRARY_PATH: libmpi.so to open for CCL_ATL_TRANSPORT=mpi
    std::string pmix_lib_path; // CCL_PMIX_LIBRARY_PATH: libpmix.so to open for CCL_PROCESS_LAUNCHER=pmix
    std::string pmix_note; // why the PMIx server could not be asked (empty: it was, or was not needed)
    size_t large_msg_size = (size_t)1 << 30; // no single transport message of a split operation exceeds this
    size_t rs_nvls_max_block = 4u << 20; // reduce_scatter: per-rank blocks up to this size use multimem.ld_reduce, larger ones peer loads
    size_t ag_nvls_max_block = 1u << 20; // allgather: blocks up to this size go out as multimem.st, larger ones as peer stores
    bool auto_register = true; // ordinary device buffers are shared with the peers automatically (buffer_exchange)
    int nvls_staged_min_ranks = 5; // from this many ranks on, ordinary buffers of allreduce / reduce_scatter are staged for the in-switch reduction instead of shared
    int p2p_lanes = 64; // independent chunk chains per ordered pair in send / recv (equal on all ranks, <= 128)
    bool p2p_pull = false; // send / recv: the receiver loads from a ring at the sender (else the sender stores into a ring at the receiver)
    int p2p_max_blocks = 0; // upper limit for the blocks of one send / recv operation (0: as many as lanes and the GPU allow)
    size_t auto_register_min = 256 * 1024; // ... for messages of at least this many bytes

    void parse();
    void print(int rank) const;
    static env_data& get();
    static void reload(); // re-parse (tests)
};

// typed helpers (also used by tests through the C API)
bool env_to_size(const char* s, size_t& out); // accepts 4096, 16K, 2M, 1G
bool env_to_bool(const char* s, bool& out);
std::vector<int> env_to_int_list(const char* s); // "1,3,5-7"

} // namespace cclx
