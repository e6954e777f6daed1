// Schedule builders of the CPU collectives.  Every function appends entries to a
// schedule; the caller (coll/coll.cpp) picked the algorithm.
//
// Algorithm set and names follow the reference (src/coll/algorithms/algorithm_utils.hpp:26-168,
// builders in src/coll/algorithms/*.cpp): allreduce {direct, rabenseifner, nreduce,
// ring, double_tree, recursive_doubling, 2d}; allgatherv {direct, naive, ring,
// flat, multi_bcast}; alltoall(v) {direct, naive, scatter}; barrier {direct, ring};
// bcast / broadcast {direct, ring, double_tree, naive}; reduce {direct,
// rabenseifner, ring, tree, double_tree}; reduce_scatter {direct, naive, ring}.
// "direct" means "hand the whole collective to MPI" in the reference; with no MPI
// underneath it is an alias of the algorithm the size table would pick.
#pragma once
#include <cstddef>
#include <vector>

#include "core/types.hpp"
#include "sched/sched.hpp"

namespace cclx {
namespace algo {

struct buf_desc {
    const void* send;
    void* recv;
    size_t count;
    int dtype;
    int op;
    reduction_fn_t fn;
};

// allreduce
void allreduce_ring(sched& s, const buf_desc& b);
void allreduce_recursive_doubling(sched& s, const buf_desc& b);
void allreduce_rabenseifner(sched& s, const buf_desc& b);
void allreduce_nreduce(sched& s, const buf_desc& b);
void allreduce_2d(sched& s, const buf_desc& b);
void allreduce_ring_rma(sched& s, const buf_desc& b);
void allreduce_double_tree(sched& s, const buf_desc& b);

// one rank's neighbours in one of the two complementary binary trees (which = 0 / 1) over `size` ranks;
// root >= 0 puts that rank at the top (it swaps places with the tree's own root), -1 keeps the tree's root
struct bin_tree {
    bin_tree(int size, int rank, int which, int root);
    int parent = -1, left = -1, right = -1;
    int root_rank = -1;
};
// halves of the message travel through the two trees at the same time
void bcast_double_tree(sched& s, void* buf, size_t count, int dtype, int root);
void reduce_double_tree(sched& s, const buf_desc& b, int root);

// reduce_scatter: send has recv_count * size elements; recv gets block `rank`
void reduce_scatter_ring(sched& s, const buf_desc& b); // b.count = recv_count
void reduce_scatter_naive(sched& s, const buf_desc& b);
// variable block sizes (used by allreduce ring / rabenseifner internals)
// `local` (optional): this rank's contribution lives there and `inout` starts out undefined; blocks are
// received straight into `inout` and combined with `local`, so an out-of-place caller copies nothing
void reduce_scatter_ring_v(sched& s, void* inout, const std::vector<size_t>& counts, const std::vector<size_t>& offs,
                           int dtype, int op, reduction_fn_t fn, uint64_t step_base, const void* local = nullptr);

// allgatherv: counts/offsets in elements of dtype, recv holds all blocks
void allgatherv_naive(sched& s, const void* send, void* recv, const std::vector<size_t>& counts,
                      const std::vector<size_t>& offs, int dtype, uint64_t step_base = 0);
void allgatherv_ring(sched& s, const void* send, void* recv, const std::vector<size_t>& counts,
                     const std::vector<size_t>& offs, int dtype, uint64_t step_base = 0);
void allgatherv_flat(sched& s, const void* send, void* recv, const std::vector<size_t>& counts,
                     const std::vector<size_t>& offs, int dtype);
void allgatherv_multi_bcast(sched& s, const void* send, void* recv, const std::vector<size_t>& counts,
                            const std::vector<size_t>& offs, int dtype);
// vector-of-buffers form: one destination buffer per rank
void allgatherv_naive_vec(sched& s, const void* send, const std::vector<void*>& recv_bufs,
                          const std::vector<size_t>& counts, int dtype);

// alltoallv: counts/offsets in elements
void alltoallv_naive(sched& s, const void* send, const std::vector<size_t>& scounts, const std::vector<size_t>& soffs,
                     void* recv, const std::vector<size_t>& rcounts, const std::vector<size_t>& roffs, int dtype);
void alltoallv_scatter(sched& s, const void* send, const std::vector<size_t>& scounts,
                       const std::vector<size_t>& soffs, void* recv, const std::vector<size_t>& rcounts,
                       const std::vector<size_t>& roffs, int dtype, size_t max_ops);

void barrier_dissemination(sched& s);
void barrier_ring(sched& s);

void bcast_naive(sched& s, void* buf, size_t bytes, int root, uint64_t step_base = 0);
void bcast_tree(sched& s, void* buf, size_t bytes, int root, uint64_t step_base = 0, int shift = 0);
void bcast_ring(sched& s, void* buf, size_t count, int dtype, int root);

void reduce_tree(sched& s, const buf_desc& b, int root, uint64_t step_base = 0, int shift = 0);
void reduce_rabenseifner(sched& s, const buf_desc& b, int root);
void reduce_ring(sched& s, const buf_desc& b, int root);

void send_direct(sched& s, const void* buf, size_t bytes, int peer, uint64_t seq);
void recv_direct(sched& s, void* buf, size_t bytes, int peer, uint64_t seq);

// [0,count) cut into `parts` blocks: counts and offsets
void block_partition(size_t count, int parts, std::vector<size_t>& counts, std::vector<size_t>& offs);

} // namespace algo
} // namespace cclx
