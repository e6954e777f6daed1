#include "coll/selection.hpp"

#include <algorithm>
#include <limits>
#include <sstream>

#include "core/env.hpp"
#include "core/log.hpp"

namespace cclx {

static const size_t SZ_MAX = std::numeric_limits<size_t>::max();

const std::vector<std::string>& algorithm_selector::known_cpu_algos(coll_type c) {
    static const std::map<int, std::vector<std::string>> table = {
        { coll_allgather, { "direct", "naive", "ring", "flat", "multi_bcast", "topo" } },
        { coll_allgatherv, { "direct", "naive", "ring", "flat", "multi_bcast", "topo" } },
        { coll_allreduce,
          { "direct", "rabenseifner", "nreduce", "ring", "ring_rma", "double_tree", "recursive_doubling", "2d",
            "topo" } },
        { coll_alltoall, { "direct", "naive", "scatter", "topo" } },
        { coll_alltoallv, { "direct", "naive", "scatter", "topo" } },
        { coll_barrier, { "direct", "ring" } },
        { coll_bcast, { "direct", "ring", "double_tree", "naive", "topo" } },
        { coll_broadcast, { "direct", "ring", "double_tree", "naive", "topo" } },
        { coll_reduce, { "direct", "rabenseifner", "ring", "tree", "double_tree", "topo" } },
        { coll_reduce_scatter, { "direct", "naive", "ring", "topo" } },
        { coll_recv, { "direct", "topo", "offload" } },
        { coll_send, { "direct", "topo", "offload" } },
    };
    return table.at(c);
}

static const std::vector<std::string>& known_gpu_algos() {
    static const std::vector<std::string> v = { "auto", "oneshot", "twoshot", "symm", "nvls", "nvls_oneshot",
                                                "push", "pull",    "copy", "pipelined", "ce" };
    return v;
}

std::vector<algo_range> algorithm_selector::parse(const std::string& spec, const std::vector<std::string>& allowed) {
    std::vector<algo_range> out;
    std::stringstream ss(spec);
    std::string block;
    while (std::getline(ss, block, ';')) {
        if (block.empty())
            continue;
        algo_range r{ 0, SZ_MAX, "" };
        size_t colon = block.find(':');
        r.algo = block.substr(0, colon);
        CCL_THROW_IF_NOT(std::find(allowed.begin(), allowed.end(), r.algo) != allowed.end(), "unknown algorithm '",
                         r.algo, "' in '", spec, "'");
        if (colon != std::string::npos) {
            std::string range = block.substr(colon + 1);
            size_t dash = range.find('-');
            CCL_THROW_IF_NOT(dash != std::string::npos, "size range '", range, "' must be <min>-<max>");
            std::string lo = range.substr(0, dash), hi = range.substr(dash + 1);
            size_t v;
            CCL_THROW_IF_NOT(env_to_size(lo.c_str(), v), "bad lower bound '", lo, "' in '", spec, "'");
            r.lo = v;
            if (hi == "max")
                r.hi = SZ_MAX;
            else {
                CCL_THROW_IF_NOT(env_to_size(hi.c_str(), v), "bad upper bound '", hi, "' in '", spec, "'");
                r.hi = v;
            }
            CCL_THROW_IF_NOT(r.lo <= r.hi, "empty size range in '", spec, "'");
        }
        out.push_back(r);
    }
    CCL_THROW_IF_NOT(!out.empty(), "empty algorithm specification");
    return out;
}

algorithm_selector::algorithm_selector() {
    reload();
}

algorithm_selector& algorithm_selector::get() {
    static algorithm_selector inst;
    return inst;
}

void algorithm_selector::reload() {
    main_.clear();
    forced_.clear();
    forced_gpu_.clear();
    // default tables (message bytes -> algorithm).  The allreduce switch points are the reference's
    // (8 KiB, 1 MiB; src/coll/selection/selector.hpp:25-31) except that the ring takes over from 512 KiB:
    // measured on this transport with 2 and 4 ranks it ties with nreduce at 256-512 KiB and is 13-20 %
    // faster at 1 MiB, because its out-of-place form copies nothing and long messages go by rendezvous.
    main_[coll_allreduce] = { { 0, 8192, "recursive_doubling" }, { 8193, 512u << 10, "nreduce" }, { (512u << 10) + 1, SZ_MAX, "ring" } };
    main_[coll_allgather] = { { 0, 32768, "naive" }, { 32769, SZ_MAX, "ring" } };
    main_[coll_allgatherv] = { { 0, 32768, "naive" }, { 32769, SZ_MAX, "ring" } };
    main_[coll_alltoall] = { { 0, 1u << 20, "naive" }, { (1u << 20) + 1, SZ_MAX, "scatter" } };
    main_[coll_alltoallv] = { { 0, 1u << 20, "naive" }, { (1u << 20) + 1, SZ_MAX, "scatter" } };
    main_[coll_barrier] = { { 0, SZ_MAX, "direct" } };
    main_[coll_bcast] = { { 0, 65536, "double_tree" }, { 65537, SZ_MAX, "ring" } };
    main_[coll_broadcast] = { { 0, 65536, "double_tree" }, { 65537, SZ_MAX, "ring" } };
    main_[coll_reduce] = { { 0, 65536, "tree" }, { 65537, SZ_MAX, "rabenseifner" } };
    main_[coll_reduce_scatter] = { { 0, 65536, "naive" }, { 65537, SZ_MAX, "ring" } };
    main_[coll_send] = { { 0, SZ_MAX, "direct" } };
    main_[coll_recv] = { { 0, SZ_MAX, "direct" } };
    const env_data& env = env_data::get();
    for (auto& kv : env.algo_raw)
        forced_[kv.first] = parse(kv.second, known_cpu_algos((coll_type)kv.first));
    for (auto& kv : env.algo_scaleout_raw)
        forced_scaleout_[kv.first] = parse(kv.second, known_cpu_algos((coll_type)kv.first));
    for (auto& kv : env.algo_gpu_raw)
        forced_gpu_[kv.first] = parse(kv.second, known_gpu_algos());
}

static const std::string* lookup(const std::vector<algo_range>& t, size_t bytes) {
    for (auto& r : t)
        if (bytes >= r.lo && bytes <= r.hi)
            return &r.algo;
    return nullptr;
}

std::string algorithm_selector::select_cpu(const selector_param& p) const {
    std::string algo;
    if (p.scaleout) {
        auto so = forced_scaleout_.find(p.ctype);
        if (so != forced_scaleout_.end())
            if (const std::string* a = lookup(so->second, p.bytes))
                algo = *a;
    }
    auto f = forced_.find(p.ctype);
    if (algo.empty() && f != forced_.end())
        if (const std::string* a = lookup(f->second, p.bytes))
            algo = *a;
    const bool forced = !algo.empty();
    // CCL_ALGO_FALLBACK=0: a requested algorithm that cannot serve this call is an error instead
    // of a silent switch to the size table (reference src/coll/selection/selector_impl.hpp:311-318)
    auto fallback_allowed = [&](const char* why) {
        CCL_THROW_IF_NOT(!forced || env_data::get().algo_fallback, coll_name(p.ctype), ": requested algorithm ", algo,
                         " ", why, " and CCL_ALGO_FALLBACK=0");
    };
    if (algo.empty()) {
        auto m = main_.find(p.ctype);
        CCL_THROW_IF_NOT(m != main_.end(), "no algorithm table for ", coll_name(p.ctype));
        const std::string* a = lookup(m->second, p.bytes);
        algo = a ? *a : m->second.back().algo;
    }
    // one-sided ring: needs the transport's one-sided writes switched on, and a predefined reduction
    // is not required (the reduction runs on the receiver)
    if (algo == "ring_rma" && p.ctype == coll_allreduce && !env_data::get().atl_rma) {
        fallback_allowed("needs CCL_ATL_RMA=1");
        algo.clear();
        auto m = main_.find(p.ctype);
        const std::string* a = lookup(m->second, p.bytes);
        algo = a ? *a : m->second.back().algo;
    }
    // names that have no CPU implementation of their own
    if (algo == "topo" || (algo == "ring_rma" && p.ctype != coll_allreduce) || algo == "offload") {
        fallback_allowed("applies to device buffers only");
        LOG_DEBUG(coll_name(p.ctype), ": algorithm ", algo, " applies to device buffers only, using the size table");
        auto m = main_.find(p.ctype);
        const std::string* a = lookup(m->second, p.bytes);
        algo = a ? *a : m->second.back().algo;
    }
    if (algo == "direct") {
        // no MPI underneath: "direct" is the table's choice, except where a direct pattern exists
        switch (p.ctype) {
            case coll_allreduce: algo = p.bytes <= 8192 ? "recursive_doubling" : (p.bytes <= (512u << 10) ? "nreduce" : "ring"); break;
            case coll_allgather:
            case coll_allgatherv: algo = "naive"; break;
            case coll_alltoall:
            case coll_alltoallv: algo = "naive"; break;
            case coll_barrier: algo = "dissemination"; break;
            case coll_bcast:
            case coll_broadcast: algo = "double_tree"; break;
            case coll_reduce: algo = "tree"; break;
            case coll_reduce_scatter: algo = "naive"; break;
            default: break;
        }
    }
    if (p.vector_buf && (p.ctype == coll_allgatherv || p.ctype == coll_allgather) && algo != "naive" &&
        algo != "flat") {
        fallback_allowed("cannot address per-rank destination buffers");
        algo = "naive"; // per-rank destination buffers: only the naive pattern addresses them
    }
    return algo;
}

bool algorithm_selector::requested(coll_type c, size_t bytes, const char* algo) const {
    auto f = forced_.find(c);
    if (f == forced_.end())
        return false;
    const std::string* a = lookup(f->second, bytes);
    return a && *a == algo;
}

std::string algorithm_selector::forced_gpu(coll_type c, size_t bytes) const {
    auto f = forced_gpu_.find(c);
    if (f == forced_gpu_.end())
        return "";
    const std::string* a = lookup(f->second, bytes);
    return a ? *a : "";
}

std::string algorithm_selector::dump() const {
    std::ostringstream ss;
    for (auto& kv : main_) {
        ss << "\n  " << coll_name((coll_type)kv.first) << ":";
        auto f = forced_.find(kv.first);
        const auto& t = f != forced_.end() ? f->second : kv.second;
        for (auto& r : t)
            ss << " [" << r.lo << "-" << (r.hi == SZ_MAX ? std::string("max") : std::to_string(r.hi)) << "] " << r.algo;
    }
    return ss.str();
}

} // namespace cclx
