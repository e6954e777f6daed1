// Kernel argument blocks of the collective kernels (plain structs shared by host and device).
#pragma once
#include <cstddef>
#include <cstdint>

namespace cclx {
namespace dev {

constexpr int ARG_MAX_RANKS = 16;

// what one rank passes: its user buffers and, for the vector collectives,
// element counts / displacements (in elements of the datatype)
struct rank_args {
    const void* send;
    void* recv;
    size_t scount[ARG_MAX_RANKS]; // alltoallv: elements sent to peer p | allgatherv: recv_counts
    size_t sdispl[ARG_MAX_RANKS]; // alltoallv: offset in send of the block for p | allgatherv: recv offsets
    size_t rcount[ARG_MAX_RANKS]; // alltoallv: elements received from p
    size_t rdispl[ARG_MAX_RANKS]; // alltoallv: offset in recv of the block from p
};

enum : int {
    CF_SYMM_IN = 1, // send buffer lives in the symmetric heap (offset given in in_off)
    CF_SYMM_OUT = 2, // recv buffer lives in the symmetric heap (offset given in out_off)
    CF_NVLS = 4, // use multimem instructions on the multicast window
    CF_REG_IN = 16, // the send buffers are registered allocations: peers' addresses in reg_in
    CF_REG_OUT = 32, // the recv buffers are registered allocations: peers' addresses in reg_out
    CF_UNIFORM = 8 // equal 16-byte-multiple blocks at contiguous displacements, 16-byte aligned user buffers
};

struct coll_args {
    rank_args r0; // real mode: this rank's arguments
    const rank_args* emu_tab; // emulation mode: device array indexed by emulated rank
    size_t count; // elements; meaning depends on the collective
    size_t stride; // reduce_scatter: elements between consecutive rank blocks of send
    size_t in_off; // heap offsets for symmetric zero-copy paths
    size_t out_off;
    float scale;
    int do_scale;
    int root;
    int emu;
    int flags;
    int peer; // point-to-point partner
    int sig_skew; // test hook: rank + 1 whose argument signature is falsified (0 = none)
    const char* reg_in[ARG_MAX_RANKS]; // CF_REG_IN: rank p's send buffer as mapped here
    char* reg_out[ARG_MAX_RANKS]; // CF_REG_OUT: rank p's recv buffer as mapped here
};

} // namespace dev
} // namespace cclx
