#include "core/datatype.hpp"

#include "core/log.hpp"

namespace cclx {

static const char* predefined_names[] = { "int8",  "uint8",  "int16",   "uint16",  "int32",   "uint32",
                                          "int64", "uint64", "float16", "float32", "float64", "bfloat16" };

const char* coll_name(coll_type c) {
    static const char* names[] = { "allgather", "allgatherv", "allreduce", "alltoall",
                                   "alltoallv", "barrier",    "bcast",     "broadcast",
                                   "reduce",    "reduce_scatter", "recv",  "send" };
    return (c >= 0 && c < coll_last) ? names[c] : "unknown";
}

const char* reduction_name(int r) {
    switch (r) {
        case red_sum: return "sum";
        case red_prod: return "prod";
        case red_min: return "min";
        case red_max: return "max";
        case red_custom: return "custom";
        default: return "none";
    }
}

datatype_table& datatype_table::get() {
    static datatype_table inst;
    return inst;
}

int datatype_table::create(size_t size) {
    CCL_THROW_IF_NOT(size > 0, "custom datatype needs a non-zero size");
    std::lock_guard<std::mutex> lk(mu_);
    int idx = next_++;
    custom_[idx] = size;
    return idx;
}

void datatype_table::free(int idx) {
    std::lock_guard<std::mutex> lk(mu_);
    CCL_THROW_IF_NOT(idx >= dt_custom_base, "predefined datatype ", idx, " can not be freed");
    CCL_THROW_IF_NOT(custom_.erase(idx) == 1, "unknown custom datatype ", idx);
}

size_t datatype_table::size(int idx) const {
    if (idx >= 0 && idx <= dt_last_predefined)
        return predefined_dtype_size(idx);
    std::lock_guard<std::mutex> lk(mu_);
    auto it = custom_.find(idx);
    CCL_THROW_IF_NOT(it != custom_.end(), "unknown datatype ", idx);
    return it->second;
}

bool datatype_table::exists(int idx) const {
    if (idx >= 0 && idx <= dt_last_predefined)
        return true;
    std::lock_guard<std::mutex> lk(mu_);
    return custom_.count(idx) != 0;
}

std::string datatype_table::name(int idx) const {
    if (idx >= 0 && idx <= dt_last_predefined)
        return predefined_names[idx];
    return "custom" + std::to_string(idx);
}

} // namespace cclx
