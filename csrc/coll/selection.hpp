// Algorithm selection: per-collective size tables, overridable from the
// environment with the reference's grammar
//     CCL_<COLL>="<algo>[:<min>-<max>][;<algo>[:<min>-<max>]...]"   (max may be the word "max")
// (reference src/coll/selection/selector_impl.hpp:26-175, tables in
// selector_allreduce.cpp:34-102, thresholds selector.hpp:25-31).  The same
// grammar drives the GPU kernels through CCL_CUDA_<COLL>.
#pragma once
#include <cstddef>
#include <map>
#include <string>
#include <vector>

#include "core/types.hpp"

namespace cclx {

struct selector_param {
    coll_type ctype;
    size_t bytes; // message size the table is keyed by
    size_t count;
    int comm_size;
    bool vector_buf = false;
    bool custom_fn = false;
    bool pof2 = false;
    bool scaleout = false; // consult the CCL_<COLL>_SCALEOUT table first
};

struct algo_range {
    size_t lo, hi; // inclusive
    std::string algo;
};

class algorithm_selector {
public:
    static algorithm_selector& get();
    void reload(); // re-read the environment (tests)
    std::string select_cpu(const selector_param& p) const;
    // "" when the environment does not force a GPU algorithm for this size
    std::string forced_gpu(coll_type c, size_t bytes) const;
    // does CCL_<COLL> name `algo` for this size?  (names such as "topo" that only device buffers honour)
    bool requested(coll_type c, size_t bytes, const char* algo) const;
    static const std::vector<std::string>& known_cpu_algos(coll_type c);
    // parses a specification; throws on syntax errors or unknown names
    static std::vector<algo_range> parse(const std::string& spec, const std::vector<std::string>& allowed);
    std::string dump() const;

private:
    algorithm_selector();
    std::map<int, std::vector<algo_range>> main_, forced_, forced_scaleout_, forced_gpu_;
};

} // namespace cclx
