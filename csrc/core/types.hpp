// Internal scalar enums shared by the CPU and GPU paths.
//
// Values of `datatype` and `reduction` are the wire/ABI values of the public
// API (reference include/oneapi/ccl/types.hpp:41-69): 12 predefined datatypes,
// 5 reductions (custom last).  Custom datatypes get indices >= dt_custom_base
// from the datatype table (core/datatype.hpp).
#pragma once
#include <cstddef>
#include <cstdint>

namespace cclx {

enum datatype_t : int {
    dt_int8 = 0,
    dt_uint8,
    dt_int16,
    dt_uint16,
    dt_int32,
    dt_uint32,
    dt_int64,
    dt_uint64,
    dt_float16,
    dt_float32,
    dt_float64,
    dt_bfloat16,
    dt_last_predefined = dt_bfloat16,
    dt_custom_base = 12
};

enum reduction_t : int { red_sum = 0, red_prod, red_min, red_max, red_custom, red_none = 99 };

enum coll_type : int {
    coll_allgather = 0,
    coll_allgatherv,
    coll_allreduce,
    coll_alltoall,
    coll_alltoallv,
    coll_barrier,
    coll_bcast,
    coll_broadcast,
    coll_reduce,
    coll_reduce_scatter,
    coll_recv,
    coll_send,
    coll_last
};

const char* coll_name(coll_type c);
const char* reduction_name(int r);

// Signature of a user reduction (reference types.hpp:107-123): inout = fn(in, inout).
struct fn_context {
    const char* match_id;
    size_t offset;
};
typedef void (*reduction_fn_t)(const void* in, size_t in_count, void* inout, size_t* out_count,
                               int dtype, const fn_context* ctx);

inline size_t predefined_dtype_size(int dt) {
    switch (dt) {
        case dt_int8:
        case dt_uint8: return 1;
        case dt_int16:
        case dt_uint16:
        case dt_float16:
        case dt_bfloat16: return 2;
        case dt_int32:
        case dt_uint32:
        case dt_float32: return 4;
        case dt_int64:
        case dt_uint64:
        case dt_float64: return 8;
        default: return 0;
    }
}

} // namespace cclx
