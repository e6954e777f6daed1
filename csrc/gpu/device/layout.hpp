// Host-safe definitions shared by host code and kernels: limits, status
// codes, the per-rank device communicator record and the point-to-point layout.
#pragma once
#include <cstddef>
#include <stdint.h>

namespace cclx {
namespace dev {

constexpr int MAX_RANKS = 16;
constexpr int MAX_BLOCKS = 256; // flag slots per rank: MAX_BLOCKS x MAX_RANKS words

// error codes written to comm_dev::status[0]
enum : uint32_t {
    ST_OK = 0,
    ST_BARRIER_TIMEOUT = 1,
    ST_ABORTED = 2,
    ST_FLAG_TIMEOUT = 3,
    ST_MBAR_TIMEOUT = 4,
    ST_BAD_ARGS = 5,
    ST_NOT_FINITE = 6, // debug scan found NaN / Inf in a reduction result (CCL_CUDA_CHECK_NAN)
    ST_ARG_MISMATCH = 7 // a zero-copy collective was called with a different buffer kind, offset or count on a peer
};

// words of comm_dev::state
enum { STATE_EPOCH = 0, STATE_GEN = 1, STATE_DONE = 2, STATE_WORDS = 8 };

struct comm_dev {
    int rank;
    int world;
    uint32_t* flags[MAX_RANKS]; // barrier slots of every rank, peer-mapped
    char* staging[MAX_RANKS]; // two generations of staging_bytes each, peer-mapped
    char* heap[MAX_RANKS]; // symmetric heap bases, peer-mapped (zero-copy paths)
    char* mc_heap; // NVLS multicast window over the heap (nullptr when NVLS is off)
    char* mc_staging; // multicast address of staging generation 0
    uint32_t* mc_flags;
    uint32_t* p2p_flags[MAX_RANKS]; // point-to-point sequence words, peer-mapped
    uint32_t* aux[MAX_RANKS]; // auxiliary flag words (alltoallv round consensus, fused-GEMM tile flags), peer-mapped
    size_t heap_bytes;
    size_t staging_bytes; // one generation
    uint32_t* state; // local device words: epoch, generation, finished-block counter
    uint32_t* p2p_seq; // local device words: per (direction, peer, lane) count of chunks moved so far
    volatile uint32_t* status; // host-mapped: [0] code, [1] block, [2] peer, [3] detail
    volatile uint32_t* abort_flag; // host-mapped, set by communicator abort
    unsigned long long timeout_ns;
};


// point-to-point (see sendrecv_kernel): every ordered pair has P2P_LANES independent chains of chunks,
// each with a ring of P2P_STAGES chunk buffers at the receiver and a pair of counters
constexpr int P2P_LANES = 64;
constexpr int P2P_STAGES = 4; // chunks of one lane that may be in flight between a sender and its receiver
constexpr size_t P2P_CHUNK_BYTES = 128u << 10;
constexpr size_t P2P_SLOT_BYTES = (size_t)P2P_LANES * P2P_STAGES * P2P_CHUNK_BYTES; // per ordered pair, at the receiver
constexpr int P2P_ACK_BASE = MAX_RANKS * P2P_LANES;
constexpr int P2P_SPARE_WORD = 2 * MAX_RANKS * P2P_LANES; // never written: timeout test
constexpr int P2P_FLAG_WORDS = 2 * MAX_RANKS * P2P_LANES + 16;
constexpr int P2P_SEQ_WORDS = 2 * MAX_RANKS * P2P_LANES;
// Argument signatures of the zero-copy collectives live behind the point-to-point flags in the same
// peer-mapped page: SIG_SLOTS generations x MAX_RANKS writers x one word (see peer_barrier).
constexpr int SIG_SLOTS = 4;
constexpr int SIG_BASE_WORD = 4160;
constexpr int P2P_PAGE_WORDS = 5120; // the peer-mapped area that holds both
static_assert(P2P_FLAG_WORDS <= SIG_BASE_WORD && SIG_BASE_WORD + SIG_SLOTS * MAX_RANKS <= P2P_PAGE_WORDS,
              "signature words must fit the area of the point-to-point flags");

// auxiliary flag region (words): [0, A2A_HDR_WORDS) alltoallv consensus, the rest is
// handed out to the fused kernels by the host
constexpr int A2A_HDR_WORDS = 2 * MAX_BLOCKS * MAX_RANKS;

// operations of one point-to-point launch (one entry per rank in emulation mode)
struct p2p_op {
    const void* send;
    void* recv;
    size_t bytes;
    int peer; // -1: no operation
    int is_send;
};
constexpr int P2P_MAX_OPS = 8;
struct p2p_ops {
    int n;
    p2p_op op[P2P_MAX_OPS];
};

struct p2p_layout {
    char* data[MAX_RANKS]; // p2p data areas, peer-mapped; slot s of rank x holds data from sender s (push) or for receiver s (pull)
    size_t slot_bytes;
    int lanes; // lanes in use, at most P2P_LANES; the same on every rank
    int pull; // 1: the ring of a pair lives at the sender and the receiver loads from it; 0: at the receiver, the sender stores into it
};

} // namespace dev
} // namespace cclx
