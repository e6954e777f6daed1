// Datatype table: 12 predefined entries plus size-only custom datatypes.
//
// Same capability as the reference table (src/common/datatype/datatype.cpp:68-228):
// thread-safe create/free/lookup, names for logs, custom indices handed out
// after the predefined range.  Custom datatypes carry only a size; they can be
// moved (allgatherv, alltoall, bcast, send/recv) and reduced with a user
// reduction_fn, never with a built-in reduction.
#pragma once
#include <mutex>
#include <string>
#include <unordered_map>

#include "core/types.hpp"

namespace cclx {

class datatype_table {
public:
    static datatype_table& get();
    int create(size_t size);
    void free(int idx);
    size_t size(int idx) const;
    std::string name(int idx) const;
    bool is_predefined(int idx) const { return idx >= 0 && idx <= dt_last_predefined; }
    bool exists(int idx) const;

private:
    datatype_table() = default;
    mutable std::mutex mu_;
    int next_ = dt_custom_base;
    std::unordered_map<int, size_t> custom_;
};

inline size_t dtype_size(int idx) {
    return datatype_table::get().size(idx);
}

} // namespace cclx
