#include "core/env.hpp"

#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>

#include "bootstrap/pmix_client.hpp"
#include "core/log.hpp"

extern char** environ; // POSIX: the process environment

namespace cclx {

static std::string lower(std::string s) {
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
    return s;
}

bool env_to_size(const char* s, size_t& out) {
    if (!s || !*s)
        return false;
    char* end = nullptr;
    double v = std::strtod(s, &end);
    if (end == s || v < 0)
        return false;
    size_t mul = 1;
    if (*end) {
        switch (std::tolower((unsigned char)*end)) {
            case 'k': mul = 1ull << 10; break;
            case 'm': mul = 1ull << 20; break;
            case 'g': mul = 1ull << 30; break;
            default: return false;
        }
        end++;
        if (*end && std::tolower((unsigned char)*end) == 'b')
            end++;
        if (*end)
            return false;
    }
    out = (size_t)(v * (double)mul);
    return true;
}

bool env_to_bool(const char* s, bool& out) {
    if (!s)
        return false;
    std::string v = lower(s);
    if (v == "1" || v == "true" || v == "yes" || v == "on" || v == "enable") {
        out = true;
        return true;
    }
    if (v == "0" || v == "false" || v == "no" || v == "off" || v == "disable") {
        out = false;
        return true;
    }
    return false;
}

std::vector<int> env_to_int_list(const char* s) {
    std::vector<int> out;
    if (!s)
        return out;
    std::stringstream ss(s);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
        if (tok.empty())
            continue;
        size_t dash = tok.find('-', 1);
        if (dash != std::string::npos) {
            int a = std::atoi(tok.substr(0, dash).c_str());
            int b = std::atoi(tok.substr(dash + 1).c_str());
            for (int i = a; i <= b; i++)
                out.push_back(i);
        }
        else
            out.push_back(std::atoi(tok.c_str()));
    }
    return out;
}

namespace {

void get_int(const char* name, int& v) {
    if (const char* s = std::getenv(name))
        v = std::atoi(s);
}
void get_double(const char* name, double& v) {
    if (const char* s = std::getenv(name))
        v = std::atof(s);
}
void get_size(const char* name, size_t& v) {
    if (const char* s = std::getenv(name)) {
        size_t t;
        if (env_to_size(s, t))
            v = t;
        else
            LOG_WARN(name, "=", s, " is not a size, keeping ", v);
    }
}
void get_bool(const char* name, bool& v) {
    if (const char* s = std::getenv(name)) {
        bool t;
        if (env_to_bool(s, t))
            v = t;
        else
            LOG_WARN(name, "=", s, " is not a boolean, keeping ", v);
    }
}
void get_str(const char* name, std::string& v) {
    if (const char* s = std::getenv(name))
        v = s;
}
template <class E>
void get_enum(const char* name, E& v, std::initializer_list<std::pair<const char*, E>> table) {
    const char* s = std::getenv(name);
    if (!s)
        return;
    std::string val = lower(s);
    for (auto& kv : table) {
        if (val == kv.first) {
            v = kv.second;
            return;
        }
    }
    std::string allowed;
    for (auto& kv : table)
        allowed += std::string(kv.first) + " ";
    CCL_THROW(name, "=", s, " is not one of: ", allowed);
}

const char* coll_env_suffix(int c) {
    static const char* names[] = { "ALLGATHER", "ALLGATHERV", "ALLREDUCE", "ALLTOALL",
                                   "ALLTOALLV", "BARRIER",    "BCAST",     "BROADCAST",
                                   "REDUCE",    "REDUCE_SCATTER", "RECV",  "SEND" };
    return names[c];
}

// Names of the reference that a user may carry over and that change nothing here.  Each is
// reported once, with the reason, so that a setting never disappears silently.
void warn_about_names_without_effect() {
    static const std::pair<const char*, const char*> table[] = {
        { "CCL_FUSION_CYCLE_MS", "fused batches are cut at points of the program order, not on a timer" },
        { "CCL_FUSION_CHECK_URGENT", "fused batches are cut at points of the program order, not on a timer" },
        { "CCL_ATL_SYNC_COLL", "it configures the MPI transport" },
        { "CCL_ENABLE_AUTO_CACHE", "it applies to the direct algorithms of the MPI transport" },
        { "CCL_ATL_CACHE", "the mesh transport registers no memory" },
        { "CCL_ATL_HMEM", "device buffers travel through NVLink kernels or pinned staging, not through the transport" },
        { "CCL_USE_HMEM", "device buffers travel through NVLink kernels or pinned staging, not through the transport" },
        { "CCL_ATL_SEND_PROXY", "device buffers are staged by the collective layer, not by the transport" },
        { "CCL_ATL_EXTRA_EP", "every worker already owns an endpoint" },
        { "CCL_STAGING_BUFFER", "staging memory is always pinned host memory" },
        { "CCL_FRAMEWORK", "no framework-specific settings exist" },
        { "CCL_DEBUG_TIMESTAMPS_LEVEL", "use CCL_SCHED_PROFILE or CCL_ITT_LEVEL for timing" },
        { "CCL_MNIC", "one connection per peer and endpoint; interface choice is CCL_KVS_IFACE" },
        { "CCL_MNIC_NAME", "one connection per peer and endpoint; interface choice is CCL_KVS_IFACE" },
        { "CCL_MNIC_COUNT", "one connection per peer and endpoint; interface choice is CCL_KVS_IFACE" },
    };
    for (auto& kv : table)
        if (std::getenv(kv.first))
            LOG_WARN(kv.first, " is set but has no effect: ", kv.second);
    // device knobs of the other backend: point at the CUDA ones
    int reported = 0;
    for (char** e = ::environ; e && *e && reported < 8; e++) {
        const std::string kv(*e);
        if (kv.rfind("CCL_ZE_", 0) == 0 || kv.rfind("CCL_SYCL_", 0) == 0 || kv.rfind("CCL_KERNEL_", 0) == 0) {
            LOG_WARN(kv.substr(0, kv.find('=')), " is set but has no effect: Level Zero / SYCL knobs have no counterpart, the "
                                                  "device path is configured by CCL_CUDA_*");
            reported++;
        }
    }
}

} // namespace

void env_data::parse() {
    get_str("CCL_LOG_LEVEL", log_level);
    logger::get().set_level(lower(log_level));
    get_bool("CCL_ABORT_ON_THROW", abort_on_throw);
    logger::get().set_abort_on_throw(abort_on_throw);
    get_bool("CCL_SCHED_PROFILE", sched_profile);
    get_bool("CCL_SCHED_DUMP", sched_dump);
    get_bool("CCL_QUEUE_DUMP", queue_dump);
    get_double("CCL_ENTRY_MAX_UPDATE_TIME_SEC", entry_max_update_time_sec);
    get_int("CCL_ITT_LEVEL", itt_level);

    get_enum<backend_t>("CCL_BACKEND", backend, { { "native", backend_t::native }, { "stub", backend_t::stub } });
    // default launcher: torchrun exports LOCAL_RANK, hydra exports MPI_LOCALRANKID; otherwise none
    if (std::getenv("MPI_LOCALRANKID"))
        process_launcher = launcher_t::hydra;
    else if (std::getenv("LOCAL_RANK") && std::getenv("LOCAL_WORLD_SIZE"))
        process_launcher = launcher_t::torchrun;
    else
        process_launcher = launcher_t::none;
    get_enum<launcher_t>("CCL_PROCESS_LAUNCHER", process_launcher,
                         { { "hydra", launcher_t::hydra },
                           { "torchrun", launcher_t::torchrun },
                           { "pmix", launcher_t::pmix },
                           { "none", launcher_t::none } });
    get_int("CCL_LOCAL_RANK", local_rank);
    get_int("CCL_LOCAL_SIZE", local_size);
    if (local_rank < 0 || local_size < 0) {
        // what the launcher exports (reference src/common/global/global.cpp:182-220)
        const char* lr = nullptr;
        const char* ls = nullptr;
        if (process_launcher == launcher_t::hydra) {
            lr = std::getenv("MPI_LOCALRANKID");
            ls = std::getenv("MPI_LOCALNRANKS");
        }
        else if (process_launcher == launcher_t::torchrun) {
            lr = std::getenv("LOCAL_RANK");
            ls = std::getenv("LOCAL_WORLD_SIZE");
        }
        else if (process_launcher == launcher_t::pmix) {
            // ask the PMIx server (the library is opened at run time); what some launchers export instead
            get_str("CCL_PMIX_LIBRARY_PATH", pmix_lib_path);
            int plr = -1, pls = -1;
            std::string why;
            if (pmix_local_coord(pmix_lib_path, plr, pls, why)) {
                if (local_rank < 0 && local_size < 0) {
                    local_rank = plr;
                    local_size = pls;
                }
            }
            else {
                pmix_note = why;
                lr = std::getenv("PMIX_LOCAL_RANK");
                ls = std::getenv("PMIX_LOCAL_SIZE");
            }
        }
        if (lr && ls && local_rank < 0 && local_size < 0) {
            local_rank = std::atoi(lr);
            local_size = std::atoi(ls);
        }
    }

    get_int("CCL_WORKER_COUNT", worker_count);
    CCL_THROW_IF_NOT(worker_count >= 1 && worker_count <= 64, "CCL_WORKER_COUNT out of range");
    get_bool("CCL_WORKER_OFFLOAD", worker_offload);
    get_bool("CCL_WORKER_WAIT", worker_wait);
    if (const char* s = std::getenv("CCL_WORKER_AFFINITY")) {
        if (lower(s) != "auto")
            worker_affinity = env_to_int_list(s);
        else
            worker_affinity_auto = true;
    }
    if (const char* s = std::getenv("CCL_WORKER_MEM_AFFINITY")) {
        if (lower(s) != "auto")
            worker_mem_affinity = env_to_int_list(s);
    }
    get_int("CCL_SPIN_COUNT", spin_count);
    get_enum<yield_t>("CCL_YIELD", yield,
                      { { "none", yield_t::none },
                        { "pause", yield_t::pause },
                        { "sleep", yield_t::sleep },
                        { "sched_yield", yield_t::sched_yield } });

    get_enum<atl_transport_t>("CCL_ATL_TRANSPORT", atl_transport,
                              { { "tcp", atl_transport_t::tcp },
                                { "shm", atl_transport_t::shm },
                                { "ofi", atl_transport_t::ofi },
                                { "mpi", atl_transport_t::mpi } });
    get_bool("CCL_ATL_SHM", atl_shm);
    get_size("CCL_ATL_SHM_RING_BYTES", atl_shm_ring_bytes);
    get_bool("CCL_ATL_RMA", atl_rma);
    get_bool("CCL_ATL_CMA", atl_cma);
    get_size("CCL_ATL_CMA_THRESHOLD", atl_cma_threshold);
    get_size("CCL_MAX_SHORT_SIZE", max_short_size);
    get_size("CCL_CHUNK_COUNT", chunk_count);
    get_size("CCL_MIN_CHUNK_SIZE", min_chunk_size);
    get_int("CCL_MAX_FLOW_CREDITS", max_flow_credits);

    if (const char* km = std::getenv("CCL_KVS_MODE")) {
        // the reference chooses between its PMI key-value store and MPI; only the first exists here
        CCL_THROW_IF_NOT(lower(km) == "pmi" || lower(km) == "internal", "CCL_KVS_MODE=", km,
                         ": this build has no MPI, the only mode is pmi");
    }
    get_str("CCL_KVS_IP_PORT", kvs_ip_port);
    get_str("CCL_KVS_IP_EXCHANGE", kvs_ip_exchange);
    kvs_ip_exchange = lower(kvs_ip_exchange);
    CCL_THROW_IF_NOT(kvs_ip_exchange == "path" || kvs_ip_exchange == "env", "CCL_KVS_IP_EXCHANGE=", kvs_ip_exchange,
                     " is not one of: path env");
    get_str("CCL_KVS_IFACE", kvs_iface);
    get_bool("CCL_KVS_PREFER_IPV6", kvs_prefer_ipv6);
    get_int("CCL_KVS_CONNECTION_TIMEOUT", kvs_connection_timeout_sec);
    get_int("CCL_KVS_GET_TIMEOUT", kvs_get_timeout_sec);

    for (int c = 0; c < coll_last; c++) {
        std::string base = std::string("CCL_") + coll_env_suffix(c);
        if (const char* s = std::getenv(base.c_str()))
            algo_raw[c] = s;
        if (const char* s = std::getenv((base + "_SCALEOUT").c_str()))
            algo_scaleout_raw[c] = s;
        std::string gpu = std::string("CCL_CUDA_") + coll_env_suffix(c);
        if (const char* s = std::getenv(gpu.c_str()))
            algo_gpu_raw[c] = s;
    }

    get_bool("CCL_UNORDERED_COLL", unordered_coll);
    get_bool("CCL_FUSION", fusion);
    get_size("CCL_FUSION_BYTES_THRESHOLD", fusion_bytes_threshold);
    get_size("CCL_FUSION_COUNT_THRESHOLD", fusion_count_threshold);
    get_enum<priority_mode_t>("CCL_PRIORITY", priority_mode,
                              { { "none", priority_mode_t::none },
                                { "direct", priority_mode_t::direct },
                                { "lifo", priority_mode_t::lifo } });
    get_enum<cache_key_t>("CCL_CACHE_KEY", cache_key,
                          { { "full", cache_key_t::full }, { "match_id", cache_key_t::match_id } });
    get_bool("CCL_CACHE_FLUSH", cache_flush);
    get_size("CCL_SCHED_CACHE_MAX_ENTRIES", sched_cache_max_entries);
    get_bool("CCL_STRICT_ORDER", strict_order);
    get_bool("CCL_OP_SYNC", op_sync);
    get_bool("CCL_BUFFER_CACHE", buffer_cache);
    get_size("CCL_BUFFER_CACHE_MAX_BYTES", buffer_cache_max_bytes);
    get_bool("CCL_ALGO_FALLBACK", algo_fallback);

    get_size("CCL_ALLREDUCE_2D_CHUNK_COUNT", ar2d_chunk_count);
    CCL_THROW_IF_NOT(ar2d_chunk_count >= 1, "CCL_ALLREDUCE_2D_CHUNK_COUNT must be at least 1");
    get_size("CCL_ALLREDUCE_2D_MIN_CHUNK_SIZE", ar2d_min_chunk_size);
    CCL_THROW_IF_NOT(ar2d_min_chunk_size >= 1, "CCL_ALLREDUCE_2D_MIN_CHUNK_SIZE must be at least 1");
    get_bool("CCL_ALLREDUCE_2D_SWITCH_DIMS", ar2d_switch_dims);
    get_size("CCL_DTREE_PARTITION_COUNT", dtree_partition_count);
    get_size("CCL_BCAST_PART_COUNT", bcast_part_count);
    get_size("CCL_ALLREDUCE_NREDUCE_SEGMENT_SIZE", nreduce_segment_size);
    get_bool("CCL_ALLREDUCE_NREDUCE_BUFFERING", nreduce_buffering);
    get_size("CCL_RS_CHUNK_COUNT", rs_chunk_count);
    get_size("CCL_RS_MIN_CHUNK_SIZE", rs_min_chunk_size);
    get_size("CCL_ALLTOALL_SCATTER_MAX_OPS", alltoall_scatter_max_ops);
    get_bool("CCL_CHECK_INPLACE_ALIASING", check_inplace_aliasing);

    get_str("CCL_BF16", bf16_impl);
    get_str("CCL_FP16", fp16_impl);

    get_str("CCL_TOPO_COLOR", topo_color);
    get_bool("CCL_TOPO_ALGO", topo_algo);
    get_size("CCL_ALLREDUCE_PIPE_CHUNK_COUNT", allreduce_pipe_chunk_count);
    get_str("CCL_TOPO_P2P_ACCESS", topo_p2p_access);
    get_bool("CCL_TOPO_FABRIC_VERTEX_CONNECTION_CHECK", topo_fabric_check);
    get_bool("CCL_TOPO_WA_FABRIC_VERTEX_CONNECTION_CHECK", topo_fabric_check); // the reference's spelling

    get_bool("CCL_ENABLE_CUDA_KERNELS", cuda_kernels);
    get_enum<ipc_exchange_t>("CCL_CUDA_IPC_EXCHANGE", ipc_exchange,
                             { { "sockets", ipc_exchange_t::sockets },
                               { "pidfd", ipc_exchange_t::pidfd },
                               { "fabric", ipc_exchange_t::fabric },
                               { "cudaipc", ipc_exchange_t::cudaipc } });
    get_size("CCL_CUDA_SYMM_HEAP_SIZE", symm_heap_bytes);
    get_size("CCL_CUDA_TMP_BUF_SIZE", tmp_buf_bytes);
    get_int("CCL_CUDA_NVLS", nvls);
    get_int("CCL_CUDA_NVLS_MIN_RANKS", nvls_min_ranks);
    get_size("CCL_CUDA_ALLREDUCE_SMALL_THRESHOLD", ar_oneshot_threshold);
    get_size("CCL_CUDA_ALLREDUCE_PIPELINE_MIN", ar_pipelined_min);
    get_int("CCL_CUDA_ALLREDUCE_PIPELINE_BLOCKS", ar_pipelined_blocks);
    get_bool("CCL_CUDA_GEMM_2SM", gemm_2sm);
    get_bool("CCL_CUDA_GEMM_RS_RING", gemm_rs_ring);
    get_bool("CCL_CUDA_AG_GEMM_CE", ag_gemm_ce);
    get_bool("CCL_CUDA_CHECK_NAN", cuda_check_nan);
    get_size("CCL_CUDA_REDUCE_SCATTER_SMALL_THRESHOLD", rs_small_threshold);
    get_size("CCL_CUDA_REDUCE_SCATTER_PIPELINE_MIN", rs_pipelined_min);
    get_size("CCL_CUDA_ALLGATHERV_SMALL_THRESHOLD", ag_small_threshold);
    get_size("CCL_CUDA_ALLGATHER_NVLS_MAX_BLOCK", ag_nvls_max_block);
    get_size("CCL_CUDA_REDUCE_SCATTER_NVLS_MAX_BLOCK", rs_nvls_max_block);
    get_int("CCL_CUDA_MAX_BLOCKS", cuda_max_blocks);
    get_int("CCL_CUDA_BLOCK_THREADS", cuda_block_threads);
    get_size("CCL_CUDA_WAIT_TIMEOUT_MS", wait_timeout_ms);
    get_bool("CCL_CUDA_COPY_ENGINE", cuda_copy_engine);
    get_size("CCL_CUDA_IPC_CACHE_ENTRIES", ipc_cache_entries);
    get_size("CCL_ATL_LARGE_MSG_SIZE", large_msg_size);
    get_str("CCL_OFI_LIBRARY_PATH", ofi_lib_path);
    get_str("CCL_MPI_LIBRARY_PATH", mpi_lib_path);
    get_int("CCL_CUDA_NVLS_STAGED_MIN_RANKS", nvls_staged_min_ranks);
    get_int("CCL_CUDA_P2P_LANES", p2p_lanes);
    get_int("CCL_CUDA_P2P_MAX_BLOCKS", p2p_max_blocks);
    get_bool("CCL_CUDA_P2P_PULL", p2p_pull);
    get_bool("CCL_CUDA_AUTO_REGISTER", auto_register);
    get_size("CCL_CUDA_AUTO_REGISTER_MIN_BYTES", auto_register_min);
    warn_about_names_without_effect();
}

void env_data::print(int rank) const {
    if ((int)logger::get().level() < (int)log_level::info || rank != 0)
        return;
    std::ostringstream ss;
    ss << "configuration:";
    ss << "\n  CCL_LOG_LEVEL=" << log_level;
    ss << "\n  CCL_BACKEND=" << (backend == backend_t::native ? "native" : "stub");
    if (!pmix_note.empty())
        ss << "\n  CCL_PROCESS_LAUNCHER=pmix: the PMIx server was not asked (" << pmix_note << "); PMIX_LOCAL_RANK / PMIX_LOCAL_SIZE used if set";
    ss << "\n  CCL_PROCESS_LAUNCHER=" << (int)process_launcher << " local_rank=" << local_rank
       << " local_size=" << local_size;
    ss << "\n  CCL_WORKER_COUNT=" << worker_count << " CCL_WORKER_OFFLOAD=" << worker_offload
       << " CCL_WORKER_WAIT=" << worker_wait << " CCL_SPIN_COUNT=" << spin_count;
    ss << "\n  CCL_ATL_TRANSPORT=" << (int)atl_transport << " CCL_ATL_SHM=" << atl_shm;
    ss << "\n  CCL_FUSION=" << fusion << " bytes<=" << fusion_bytes_threshold
       << " count<=" << fusion_count_threshold;
    ss << "\n  CCL_PRIORITY=" << (int)priority_mode << " CCL_CACHE_KEY=" << (int)cache_key
       << " CCL_CACHE_FLUSH=" << cache_flush << " CCL_STRICT_ORDER=" << strict_order
       << " CCL_OP_SYNC=" << op_sync << " CCL_UNORDERED_COLL=" << unordered_coll;
    for (auto& kv : algo_raw)
        ss << "\n  CCL_" << coll_env_suffix(kv.first) << "=" << kv.second;
    for (auto& kv : algo_gpu_raw)
        ss << "\n  CCL_CUDA_" << coll_env_suffix(kv.first) << "=" << kv.second;
    ss << "\n  CCL_ENABLE_CUDA_KERNELS=" << cuda_kernels << " CCL_CUDA_IPC_EXCHANGE=" << (int)ipc_exchange
       << " CCL_CUDA_SYMM_HEAP_SIZE=" << symm_heap_bytes << " CCL_CUDA_TMP_BUF_SIZE=" << tmp_buf_bytes
       << " CCL_CUDA_NVLS=" << nvls;
    ss << "\n  CCL_CUDA_ALLREDUCE_SMALL_THRESHOLD=" << ar_oneshot_threshold
       << " CCL_CUDA_ALLREDUCE_PIPELINE_MIN=" << ar_pipelined_min
       << " CCL_CUDA_WAIT_TIMEOUT_MS=" << wait_timeout_ms;
    LOG_INFO(ss.str());
}

static std::once_flag env_once;
static env_data* env_inst = nullptr;

env_data& env_data::get() {
    std::call_once(env_once, [] {
        env_inst = new env_data();
        env_inst->parse();
    });
    return *env_inst;
}

void env_data::reload() {
    env_data& e = get();
    e = env_data();
    e.parse();
}

} // namespace cclx
