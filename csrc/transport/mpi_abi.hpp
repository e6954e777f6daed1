// The part of the MPI binary interface that the MPI transport calls, declared here so that the
// library builds without an MPI installation and finds one at run time (dlopen), the way the reference
// reaches MPI through a table of entry points (src/common/api_wrapper/mpi_api_wrapper.hpp:26-103, loaded by
// mpi_api_wrapper.cpp:25-46).
//
// Handles and constants are those of the MPICH binary interface (MPICH, Intel MPI, MVAPICH, Cray MPICH:
// the common ABI of the MPICH ABI compatibility initiative): communicators, datatypes and requests are
// 32-bit integers with fixed values for the predefined ones, MPI_Status is five ints.  Open MPI uses
// pointers to its own structures for the same names; a library that exports Open MPI's symbols is
// refused by the loader (atl_mpi.cpp) rather than called with the wrong types.
#pragma once
#include <cstdint>

namespace cclx {
namespace mpiabi {

typedef int comm_t;
typedef int datatype_t;
typedef int request_t;

struct status_t {
    int count_lo;
    int count_hi_and_cancelled;
    int source;
    int tag;
    int error;
};

constexpr comm_t COMM_WORLD = 0x44000000;
constexpr datatype_t BYTE = 0x4c00010d;
constexpr request_t REQUEST_NULL = 0x2c000000;
constexpr int ANY_SOURCE = -2;
constexpr int ANY_TAG = -1;
constexpr int SUCCESS = 0;
constexpr int THREAD_SINGLE = 0, THREAD_FUNNELED = 1, THREAD_SERIALIZED = 2, THREAD_MULTIPLE = 3;
// the largest tag every implementation must accept (MPI_TAG_UB is at least this)
constexpr int TAG_UB_MIN = 32767;

struct library {
    void* handle = nullptr;
    int (*Init_thread)(int*, char***, int, int*) = nullptr;
    int (*Initialized)(int*) = nullptr;
    int (*Finalized)(int*) = nullptr;
    int (*Finalize)() = nullptr;
    int (*Query_thread)(int*) = nullptr;
    int (*Comm_rank)(comm_t, int*) = nullptr;
    int (*Comm_size)(comm_t, int*) = nullptr;
    int (*Comm_dup)(comm_t, comm_t*) = nullptr;
    int (*Comm_free)(comm_t*) = nullptr;
    int (*Isend)(const void*, int, datatype_t, int, int, comm_t, request_t*) = nullptr;
    int (*Irecv)(void*, int, datatype_t, int, int, comm_t, request_t*) = nullptr;
    int (*Recv)(void*, int, datatype_t, int, int, comm_t, status_t*) = nullptr;
    int (*Test)(request_t*, int*, status_t*) = nullptr;
    int (*Iprobe)(int, int, comm_t, int*, status_t*) = nullptr;
    int (*Get_count)(const status_t*, datatype_t, int*) = nullptr;
    int (*Get_library_version)(char*, int*) = nullptr;
    bool we_initialised = false;
};

} // namespace mpiabi
} // namespace cclx
