#include "coll/algorithms.hpp"

#include <algorithm>
#include <functional>

#include "comm/host_comm.hpp"
#include "core/datatype.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "sched/entries.hpp"

namespace cclx {
namespace algo {

namespace {

inline char* at(void* base, size_t elems, size_t esz) {
    return (char*)base + elems * esz;
}
inline const char* at(const void* base, size_t elems, size_t esz) {
    return (const char*)base + elems * esz;
}

int pof2_floor(int n) {
    int p = 1;
    while (p * 2 <= n)
        p *= 2;
    return p;
}

// out-of-place collectives work in place on recv after this copy
void copy_in(sched& s, const void* send, void* recv, size_t bytes) {
    if (send && send != recv && bytes) {
        s.add<copy_entry>(send, recv, bytes);
        s.add_barrier();
    }
}

// A message may travel as several chunks so that the receiver starts working on
// the first while the rest is still on the wire.  Chunk k of step s uses tag
// s + k * CHUNK_TAG_STRIDE; steps stay below the stride, chunks below MAX_CHUNKS,
// and the product fits the 16 bits of step space that one partial schedule owns.
constexpr uint64_t CHUNK_TAG_STRIDE = 2048;
constexpr size_t MAX_CHUNKS = 16;

// number of chunks for `bytes` (`count` elements): `want`, lowered until every
// chunk has `min_bytes` and at least one element.  Both sides of a message call
// this with the same arguments (reference
// src/sched/entry/factory/chunked_entry_factory.hpp:24-41,
// src/coll/algorithms/reduce_scatter/reduce_scatter.cpp:226-240).
size_t chunks_for(size_t bytes, size_t count, size_t want, size_t min_bytes) {
    size_t c = std::min(std::max<size_t>(want, 1), MAX_CHUNKS);
    while (c > 1 && (bytes / c < min_bytes || count < c))
        c--;
    return c;
}

// element range of chunk k: equal shares, the last takes the remainder
inline void chunk_range(size_t count, size_t chunks, size_t k, size_t& off, size_t& n) {
    const size_t main = count / chunks;
    off = k * main;
    n = (k == chunks - 1) ? count - off : main;
}

// CCL_CHUNK_COUNT / CCL_MIN_CHUNK_SIZE: point-to-point transfers of the alltoall family
void chunked_send(sched& s, const void* buf, size_t count, size_t esz, int dst, uint64_t step) {
    const auto& e = env_data::get();
    const size_t chunks = chunks_for(count * esz, count, e.chunk_count, e.min_chunk_size);
    for (size_t k = 0; k < chunks; k++) {
        size_t off, n;
        chunk_range(count, chunks, k, off, n);
        s.add<send_entry>(at(buf, off, esz), n * esz, dst, step + k * CHUNK_TAG_STRIDE);
    }
}
void chunked_recv(sched& s, void* buf, size_t count, size_t esz, int src, uint64_t step) {
    const auto& e = env_data::get();
    const size_t chunks = chunks_for(count * esz, count, e.chunk_count, e.min_chunk_size);
    for (size_t k = 0; k < chunks; k++) {
        size_t off, n;
        chunk_range(count, chunks, k, off, n);
        s.add<recv_entry>(at(buf, off, esz), n * esz, src, step + k * CHUNK_TAG_STRIDE);
    }
}

// Non-power-of-two fold used by recursive doubling / halving: the first 2*rem
// ranks pair up, even ones hand their data to the odd neighbour and sit out.
struct fold {
    int pof2, rem, newrank; // newrank == -1: this rank sits out
    int real(int nr) const { return nr < rem ? nr * 2 + 1 : nr + rem; }
};

fold make_fold(int N, int r) {
    fold f;
    f.pof2 = pof2_floor(N);
    f.rem = N - f.pof2;
    if (r < 2 * f.rem)
        f.newrank = (r % 2 == 0) ? -1 : r / 2;
    else
        f.newrank = r - f.rem;
    return f;
}

// Recursive-halving reduce-scatter over the pof2 participants, in place on buf.
// Blocks = block_partition(count, pof2).  On return newrank holds block newrank.
void rs_recursive_halving(sched& s, void* buf, const fold& f, const std::vector<size_t>& cnt,
                          const std::vector<size_t>& off, int dtype, int op, reduction_fn_t fn, uint64_t step_base) {
    const size_t esz = dtype_size(dtype);
    int lo = 0, hi = f.pof2;
    uint64_t step = step_base;
    size_t max_half = 0;
    for (int i = 0; i < f.pof2; i++)
        max_half += cnt[i];
    void* tmp = s.alloc_tmp((max_half / 2 + cnt[0] + 1) * esz + 64);
    for (int mask = f.pof2 / 2; mask >= 1; mask /= 2, step++) {
        const int mid = (lo + hi) / 2;
        const int partner = f.real(f.newrank ^ mask);
        int klo, khi, slo, shi; // keep / send ranges in blocks
        if ((f.newrank & mask) == 0) {
            klo = lo, khi = mid, slo = mid, shi = hi;
        }
        else {
            klo = mid, khi = hi, slo = lo, shi = mid;
        }
        auto span = [&](int a, int b) { return (b > a) ? (off[b - 1] + cnt[b - 1] - off[a]) : (size_t)0; };
        s.add<send_entry>(at(buf, off[slo], esz), span(slo, shi) * esz, partner, step);
        s.add<recv_reduce_entry>(at(buf, off[klo], esz), span(klo, khi), dtype, op, partner, step, fn, tmp);
        s.add_barrier();
        lo = klo;
        hi = khi;
    }
}

// Recursive-doubling allgather, the mirror image of the function above.
void ag_recursive_doubling(sched& s, void* buf, const fold& f, const std::vector<size_t>& cnt,
                           const std::vector<size_t>& off, int dtype, uint64_t step_base) {
    const size_t esz = dtype_size(dtype);
    int lo = f.newrank, hi = f.newrank + 1;
    uint64_t step = step_base;
    auto span = [&](int a, int b) { return (b > a) ? (off[b - 1] + cnt[b - 1] - off[a]) : (size_t)0; };
    for (int mask = 1; mask < f.pof2; mask *= 2, step++) {
        const int partner = f.real(f.newrank ^ mask);
        const int size = hi - lo;
        int plo, phi;
        if ((f.newrank & mask) == 0) {
            plo = hi, phi = hi + size;
        }
        else {
            plo = lo - size, phi = lo;
        }
        s.add<send_entry>(at(buf, off[lo], esz), span(lo, hi) * esz, partner, step);
        s.add<recv_entry>(at(buf, off[plo], esz), span(plo, phi) * esz, partner, step);
        s.add_barrier();
        lo = std::min(lo, plo);
        hi = std::max(hi, phi);
    }
}

} // namespace

void block_partition(size_t count, int parts, std::vector<size_t>& counts, std::vector<size_t>& offs) {
    counts.assign(parts, 0);
    offs.assign(parts, 0);
    const size_t base = count / parts, rem = count % parts;
    size_t o = 0;
    for (int i = 0; i < parts; i++) {
        counts[i] = base + ((size_t)i < rem ? 1 : 0);
        offs[i] = o;
        o += counts[i];
    }
}

// ---------------------------------------------------------------------------- reduce_scatter
void reduce_scatter_ring_v(sched& s, void* inout, const std::vector<size_t>& counts, const std::vector<size_t>& offs,
                           int dtype, int op, reduction_fn_t fn, uint64_t step_base, const void* local) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    if (N == 1)
        return;
    const size_t esz = dtype_size(dtype);
    size_t maxc = *std::max_element(counts.begin(), counts.end());
    void* tmp = local ? nullptr : s.alloc_tmp(maxc * esz + 64);
    const int next = (r + 1) % N, prev = (r - 1 + N) % N;
    const auto& e = env_data::get();
    for (int st = 0; st < N - 1; st++) {
        const int sb = (r - st - 1 + 2 * N) % N, rb = (r - st - 2 + 2 * N) % N;
        // CCL_RS_CHUNK_COUNT > 1: the block travels in chunks, each reduced on arrival while
        // the next is still in flight (reference reduce_scatter.cpp:289-390 delays the
        // reduction by one chunk for the same overlap)
        const size_t want = N < 1000 ? e.rs_chunk_count : 1; // steps must stay below the chunk tag stride
        const size_t sc = chunks_for(counts[sb] * esz, counts[sb], want, e.rs_min_chunk_size);
        const size_t rc = chunks_for(counts[rb] * esz, counts[rb], want, e.rs_min_chunk_size);
        for (size_t k = 0; k < sc; k++) {
            size_t off, n;
            chunk_range(counts[sb], sc, k, off, n);
            // the first block that leaves holds only this rank's data; later ones are partial sums
            const void* src = (local && st == 0) ? (const void*)at(local, offs[sb] + off, esz)
                                                 : (const void*)at(inout, offs[sb] + off, esz);
            s.add<send_entry>(src, n * esz, next, step_base + st + k * CHUNK_TAG_STRIDE);
        }
        for (size_t k = 0; k < rc; k++) {
            size_t off, n;
            chunk_range(counts[rb], rc, k, off, n);
            if (local)
                s.add<recv_reduce_entry>(at(inout, offs[rb] + off, esz), n, dtype, op, prev,
                                         step_base + st + k * CHUNK_TAG_STRIDE, fn, nullptr,
                                         at(local, offs[rb] + off, esz));
            else
                s.add<recv_reduce_entry>(at(inout, offs[rb] + off, esz), n, dtype, op, prev,
                                         step_base + st + k * CHUNK_TAG_STRIDE, fn, at(tmp, off, esz));
        }
        s.add_barrier();
    }
}

void reduce_scatter_ring(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    const size_t rc = b.count;
    if (N == 1) {
        copy_in(s, b.send, b.recv, rc * esz);
        return;
    }
    // partial sums live in scratch memory so that send stays intact; this rank's own contribution is
    // read from send where it is needed
    void* work = s.alloc_tmp(rc * N * esz + 64);
    std::vector<size_t> cnt(N, rc), off(N);
    for (int i = 0; i < N; i++)
        off[i] = (size_t)i * rc;
    reduce_scatter_ring_v(s, work, cnt, off, b.dtype, b.op, b.fn, 0, b.send);
    s.add<copy_entry>(at(work, off[r], esz), b.recv, rc * esz);
}

void reduce_scatter_naive(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    const size_t rc = b.count;
    const bool inplace = b.recv == at(b.send, (size_t)r * rc, esz);
    std::vector<void*> tmps(N, nullptr);
    for (int k = 1; k < N; k++) {
        const int p = (r + k) % N;
        tmps[p] = s.alloc_tmp(rc * esz + 64);
        s.add<recv_entry>(tmps[p], rc * esz, p, 0);
        s.add<send_entry>(at(b.send, (size_t)p * rc, esz), rc * esz, p, 0);
    }
    s.add_barrier();
    if (!inplace)
        s.add<copy_entry>(at(b.send, (size_t)r * rc, esz), b.recv, rc * esz);
    s.add_barrier();
    for (int p = 0; p < N; p++) // fixed order: reproducible rounding
        if (p != r) {
            s.add<reduce_local_entry>(tmps[p], b.recv, rc, b.dtype, b.op, b.fn);
            s.add_barrier();
        }
}

// ---------------------------------------------------------------------------- allgatherv
void allgatherv_naive(sched& s, const void* send, void* recv, const std::vector<size_t>& counts,
                      const std::vector<size_t>& offs, int dtype, uint64_t step_base) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(dtype);
    char* mine = at(recv, offs[r], esz);
    if (send && send != mine) {
        s.add<copy_entry>(send, mine, counts[r] * esz);
        s.add_barrier();
    }
    for (int k = 1; k < N; k++) {
        const int p = (r + k) % N;
        s.add<recv_entry>(at(recv, offs[p], esz), counts[p] * esz, p, step_base);
        s.add<send_entry>(mine, counts[r] * esz, p, step_base);
    }
    s.add_barrier();
}

// flat: every peer gets a sub-schedule of its own (reference allgatherv.cpp:327-395 spreads the peers over
// the partial schedules of the workers), so the exchanges with different peers progress independently, and
// the blocks are sent straight from the user's send buffer, without waiting for the local copy.
void allgatherv_flat(sched& s, const void* send, void* recv, const std::vector<size_t>& counts,
                     const std::vector<size_t>& offs, int dtype) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(dtype);
    char* mine = at(recv, offs[r], esz);
    const void* src = send ? send : mine;
    const size_t my_bytes = counts[r] * esz;
    if (send && send != mine)
        s.add<copy_entry>(send, mine, my_bytes); // no barrier: nobody below depends on it
    for (int k = 1; k < N; k++) {
        const int p = (r + k) % N;
        void* dst = at(recv, offs[p], esz);
        const size_t pb = counts[p] * esz;
        s.add<subsched_entry>(
            [=](sched& sub) {
                sub.add<recv_entry>(dst, pb, p, 0);
                sub.add<send_entry>(src, my_bytes, p, 0);
            },
            "AG_FLAT_PEER");
    }
    s.add_barrier();
}

void allgatherv_ring(sched& s, const void* send, void* recv, const std::vector<size_t>& counts,
                     const std::vector<size_t>& offs, int dtype, uint64_t step_base) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(dtype);
    char* mine = at(recv, offs[r], esz);
    if (send && send != mine) {
        s.add<copy_entry>(send, mine, counts[r] * esz);
        s.add_barrier();
    }
    const int next = (r + 1) % N, prev = (r - 1 + N) % N;
    for (int st = 0; st < N - 1; st++) {
        const int sb = (r - st + N) % N, rb = (r - st - 1 + N) % N;
        s.add<send_entry>(at(recv, offs[sb], esz), counts[sb] * esz, next, step_base + st);
        s.add<recv_entry>(at(recv, offs[rb], esz), counts[rb] * esz, prev, step_base + st);
        s.add_barrier();
    }
}

void allgatherv_multi_bcast(sched& s, const void* send, void* recv, const std::vector<size_t>& counts,
                            const std::vector<size_t>& offs, int dtype) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(dtype);
    char* mine = at(recv, offs[r], esz);
    if (send && send != mine) {
        s.add<copy_entry>(send, mine, counts[r] * esz);
        s.add_barrier();
    }
    // one tree broadcast per root, all running concurrently on disjoint step ranges
    for (int root = 0; root < N; root++) {
        void* blk = at(recv, offs[root], esz);
        const size_t bytes = counts[root] * esz;
        const uint64_t base = (uint64_t)(root + 1) * 64;
        s.add<subsched_entry>([=](sched& sub) { bcast_tree(sub, blk, bytes, root, base); }, "AGV_BCAST");
    }
    s.add_barrier();
}

void allgatherv_naive_vec(sched& s, const void* send, const std::vector<void*>& recv_bufs,
                          const std::vector<size_t>& counts, int dtype) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(dtype);
    if (send && send != recv_bufs[r]) {
        s.add<copy_entry>(send, recv_bufs[r], counts[r] * esz);
        s.add_barrier();
    }
    for (int k = 1; k < N; k++) {
        const int p = (r + k) % N;
        s.add<recv_entry>(recv_bufs[p], counts[p] * esz, p, 0);
        s.add<send_entry>(send ? send : recv_bufs[r], counts[r] * esz, p, 0);
    }
    s.add_barrier();
}

// ---------------------------------------------------------------------------- allreduce
void allreduce_ring(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const int N = c->size();
    const size_t esz = dtype_size(b.dtype);
    if (N == 1) {
        copy_in(s, b.send, b.recv, b.count * esz);
        return;
    }
    std::vector<size_t> cnt, off;
    block_partition(b.count, N, cnt, off);
    // out of place: no copy of send into recv first, every block of recv is written by the ring itself
    // (N - 1 blocks as reduction targets, the remaining one by the allgather)
    const void* local = (b.send && b.send != b.recv) ? b.send : nullptr;
    reduce_scatter_ring_v(s, b.recv, cnt, off, b.dtype, b.op, b.fn, 0, local);
    allgatherv_ring(s, nullptr, b.recv, cnt, off, b.dtype, 1000);
}

// Ring allreduce by one-sided writes (reference src/coll/algorithms/allreduce/allreduce_rma.cpp:121-330):
// every rank registers its result buffer, a scratch area with one slot per reduce-scatter step and a flag
// per step, tells them to its left neighbour (its only writer) and learns those of its right neighbour.
// A step writes the block, then the flag; the receiver waits on the flag in its own memory, so no
// receive is ever posted.  Regions and flags are set up again on every run of a cached schedule, and a
// writer cannot start before it has the description of this run, which orders runs against one another.
void allreduce_ring_rma(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    copy_in(s, b.send, b.recv, b.count * esz);
    if (N == 1)
        return;
    std::vector<size_t> cnt, off;
    block_partition(b.count, N, cnt, off);
    const size_t slot = (cnt[0] * esz + 63) & ~(size_t)63; // the first block is never smaller than another
    const int steps = 2 * (N - 1);
    struct regions {
        atl_mr mine[3], next[3]; // result buffer, scratch slots, flags
    };
    auto reg = std::make_shared<regions>();
    char* scratch = (char*)s.alloc_tmp(slot * (size_t)(N - 1) + 64);
    uint64_t* flags = (uint64_t*)s.alloc_tmp(sizeof(uint64_t) * (size_t)steps);
    const int next = (r + 1) % N, prev = (r - 1 + N) % N;
    s.add<function_entry>([reg, flags, steps] {
        for (int i = 0; i < steps; i++)
            __atomic_store_n(&flags[i], 0, __ATOMIC_RELEASE);
    });
    s.add<register_entry>(b.recv, b.count * esz, &reg->mine[0]);
    s.add<register_entry>(scratch, slot * (size_t)(N - 1), &reg->mine[1]);
    s.add<register_entry>(flags, sizeof(uint64_t) * (size_t)steps, &reg->mine[2]);
    s.add_barrier();
    s.add<send_entry>(reg->mine, sizeof(reg->mine), prev, 0);
    s.add<recv_entry>(reg->next, sizeof(reg->next), next, 0);
    s.add_barrier();
    for (int st = 0; st < steps; st++) {
        const bool scatter = st < N - 1;
        const int k = scatter ? st : st - (N - 1);
        // reduce-scatter: block r-k-1 goes into the neighbour's slot k and is added to its block;
        // allgather: the finished block r-k goes straight into the neighbour's result buffer
        const int sb = scatter ? (r - k - 1 + 2 * N) % N : (r - k + 2 * N) % N;
        const int rb = (r - k - 2 + 2 * N) % N; // reduce-scatter only
        if (scatter)
            s.add<write_entry>(at(b.recv, off[sb], esz), cnt[sb] * esz, &reg->next[1], (uint64_t)k * slot);
        else
            s.add<write_entry>(at(b.recv, off[sb], esz), cnt[sb] * esz, &reg->next[0], (uint64_t)(off[sb] * esz));
        s.add_barrier();
        s.add<write_entry>((uint64_t)1, &reg->next[2], (uint64_t)st * sizeof(uint64_t));
        s.add<wait_value_entry>((const volatile uint64_t*)&flags[st], 1);
        s.add_barrier();
        if (scatter) {
            s.add<reduce_local_entry>(scratch + (size_t)k * slot, at(b.recv, off[rb], esz), cnt[rb], b.dtype, b.op, b.fn);
            s.add_barrier();
        }
    }
    for (int i = 0; i < 3; i++)
        s.add<deregister_entry>(&reg->mine[i]);
}

void allreduce_recursive_doubling(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    const size_t bytes = b.count * esz;
    copy_in(s, b.send, b.recv, bytes);
    if (N == 1)
        return;
    const fold f = make_fold(N, r);
    void* tmp = s.alloc_tmp(bytes + 64);
    if (r < 2 * f.rem) {
        if (f.newrank < 0) {
            s.add<send_entry>(b.recv, bytes, r + 1, 0);
        }
        else {
            s.add<recv_reduce_entry>(b.recv, b.count, b.dtype, b.op, r - 1, 0, b.fn, tmp);
        }
        s.add_barrier();
    }
    if (f.newrank >= 0) {
        uint64_t step = 1;
        for (int mask = 1; mask < f.pof2; mask *= 2, step++) {
            const int partner = f.real(f.newrank ^ mask);
            // exchange whole buffers; reduce only after my send has left the buffer
            s.add<send_entry>(b.recv, bytes, partner, step);
            s.add<recv_entry>(tmp, bytes, partner, step);
            s.add_barrier();
            s.add<reduce_local_entry>(tmp, b.recv, b.count, b.dtype, b.op, b.fn);
            s.add_barrier();
        }
    }
    if (r < 2 * f.rem) {
        if (f.newrank < 0)
            s.add<recv_entry>(b.recv, bytes, r + 1, 999);
        else
            s.add<send_entry>(b.recv, bytes, r - 1, 999);
        s.add_barrier();
    }
}

void allreduce_rabenseifner(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    const size_t bytes = b.count * esz;
    copy_in(s, b.send, b.recv, bytes);
    if (N == 1)
        return;
    const fold f = make_fold(N, r);
    if ((size_t)f.pof2 > b.count) { // fewer elements than participants: blocks would be empty
        allreduce_recursive_doubling(s, buf_desc{ nullptr, b.recv, b.count, b.dtype, b.op, b.fn });
        return;
    }
    if (r < 2 * f.rem) {
        if (f.newrank < 0)
            s.add<send_entry>(b.recv, bytes, r + 1, 0);
        else
            s.add<recv_reduce_entry>(b.recv, b.count, b.dtype, b.op, r - 1, 0, b.fn);
        s.add_barrier();
    }
    if (f.newrank >= 0) {
        std::vector<size_t> cnt, off;
        block_partition(b.count, f.pof2, cnt, off);
        rs_recursive_halving(s, b.recv, f, cnt, off, b.dtype, b.op, b.fn, 1);
        ag_recursive_doubling(s, b.recv, f, cnt, off, b.dtype, 100);
    }
    if (r < 2 * f.rem) {
        if (f.newrank < 0)
            s.add<recv_entry>(b.recv, bytes, r + 1, 999);
        else
            s.add<send_entry>(b.recv, bytes, r - 1, 999);
        s.add_barrier();
    }
}

void allreduce_nreduce(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    if (N == 1) {
        copy_in(s, b.send, b.recv, b.count * esz);
        return;
    }
    const auto& e = env_data::get();
    const void* src = b.send ? b.send : b.recv;
    // The vector is processed in segments of CCL_ALLREDUCE_NREDUCE_SEGMENT_SIZE bytes, so the
    // scratch memory is bounded by one segment whatever the message size (reference
    // src/coll/algorithms/allreduce/allreduce.cpp:324-345).  With CCL_ALLREDUCE_NREDUCE_BUFFERING
    // the owned block is reduced in scratch and copied to recv afterwards, which keeps recv
    // untouched until the segment's result is final.
    size_t seg_elems = std::max<size_t>(e.nreduce_segment_size / esz, (size_t)N);
    seg_elems = std::min(seg_elems, b.count);
    const size_t max_block = seg_elems / N + 1;
    std::vector<void*> tmps(N, nullptr);
    for (int p = 0; p < N; p++)
        if (p != r || e.nreduce_buffering)
            tmps[p] = s.alloc_tmp(max_block * esz + 64);
    for (size_t seg = 0; seg < b.count; seg += seg_elems) {
        const size_t n = std::min(seg_elems, b.count - seg);
        const char* sseg = at(src, seg, esz);
        char* rseg = at(b.recv, seg, esz);
        std::vector<size_t> cnt, off;
        block_partition(n, N, cnt, off);
        // every rank owns one block: gather the N-1 foreign contributions, reduce in rank order
        for (int k = 1; k < N; k++) {
            const int p = (r + k) % N;
            s.add<recv_entry>(tmps[p], cnt[r] * esz, p, 0);
            s.add<send_entry>(sseg + off[p] * esz, cnt[p] * esz, p, 0);
        }
        char* acc = e.nreduce_buffering ? (char*)tmps[r] : rseg + off[r] * esz;
        if ((const char*)acc != sseg + off[r] * esz)
            s.add<copy_entry>(sseg + off[r] * esz, acc, cnt[r] * esz);
        s.add_barrier();
        for (int p = 0; p < N; p++)
            if (p != r) {
                s.add<reduce_local_entry>(tmps[p], acc, cnt[r], b.dtype, b.op, b.fn);
                s.add_barrier();
            }
        if (e.nreduce_buffering) {
            s.add<copy_entry>(acc, rseg + off[r] * esz, cnt[r] * esz);
            s.add_barrier();
        }
        allgatherv_naive(s, nullptr, rseg, cnt, off, b.dtype, 1);
    }
}

void allreduce_2d(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const size_t esz = dtype_size(b.dtype);
    const auto& e = env_data::get();
    auto node = c->node_comm();
    auto r2r = c->r2r_comm();
    if (!node || !r2r || r2r->size() == 1 || node->size() == 1 || node->size() * r2r->size() != c->size()) {
        allreduce_ring(s, b);
        return;
    }
    copy_in(s, b.send, b.recv, b.count * esz);
    // reduce-scatter in the first dimension, allreduce of my block in the second, allgather in
    // the first.  CCL_ALLREDUCE_2D_SWITCH_DIMS makes the cross-node communicator the first one
    // (reference src/coll/algorithms/allreduce/allreduce.cpp:811-817).
    host_comm* first = e.ar2d_switch_dims ? r2r.get() : node.get();
    host_comm* second = e.ar2d_switch_dims ? node.get() : r2r.get();
    const int F = first->size(), fr = first->rank();
    const int dtype = b.dtype, op = b.op;
    reduction_fn_t fn = b.fn;
    // CCL_ALLREDUCE_2D_CHUNK_COUNT > 1: the vector is cut into chunks that move through the
    // three phases as a pipeline, so chunk t is scattered inside the first dimension while
    // chunk t-1 crosses the second and chunk t-2 is gathered.  The two phases that share a
    // communicator use disjoint steps (0.. and 1000..).
    size_t chunks = std::min(std::max<size_t>(e.ar2d_chunk_count, 1), MAX_CHUNKS);
    while (chunks > 1 && (b.count * esz / chunks < e.ar2d_min_chunk_size || b.count / chunks < (size_t)F))
        chunks--;
    struct piece {
        void* base;
        std::vector<size_t> cnt, off;
    };
    std::vector<piece> pieces(chunks);
    for (size_t k = 0; k < chunks; k++) {
        size_t o, n;
        chunk_range(b.count, chunks, k, o, n);
        pieces[k].base = at(b.recv, o, esz);
        block_partition(n, F, pieces[k].cnt, pieces[k].off);
    }
    for (size_t t = 0; t < chunks + 2; t++) {
        if (t < chunks) {
            const piece pc = pieces[t];
            s.add<subsched_entry>(
                [=](sched& sub) { reduce_scatter_ring_v(sub, pc.base, pc.cnt, pc.off, dtype, op, fn, 0); }, "2D_RS",
                first);
        }
        if (t >= 1 && t - 1 < chunks) {
            const piece pc = pieces[t - 1];
            s.add<subsched_entry>(
                [=](sched& sub) {
                    allreduce_ring(sub,
                                   buf_desc{ nullptr, at(pc.base, pc.off[fr], dtype_size(dtype)), pc.cnt[fr], dtype, op, fn });
                },
                "2D_AR", second);
        }
        if (t >= 2) {
            const piece pc = pieces[t - 2];
            s.add<subsched_entry>(
                [=](sched& sub) { allgatherv_ring(sub, nullptr, pc.base, pc.cnt, pc.off, dtype, 1000); }, "2D_AG", first);
        }
        s.add_barrier();
    }
}

// ---------------------------------------------------------------------------- double binary tree
// Two complementary binary trees over the ranks (the topology of the reference's double-tree operations,
// src/common/utils/tree.hpp:22-216 and src/coll/algorithms/double_tree_ops.cpp:118-331, built here from the
// in-order numbering instead of being taken over).  Positions 1..N in in-order: a position's height is the
// number of trailing zero bits, odd positions are leaves, a node of height h has the children i - 2^(h-1) and
// i + 2^(h-1) (a right child beyond N is replaced by the highest node of its subtree that exists), the root
// is the largest power of two <= N.  Tree A puts rank i-1 on position i; tree B puts rank i mod N there, a
// shift by one, so that the inner nodes of A (odd ranks) are leaves of B and the other way round: every
// rank forwards data in one tree only, which is what lets the two halves of a message travel at full rate.
// A root other than the tree's own swaps places with it.
bin_tree::bin_tree(int size, int rank, int which, int root) {
    const int N = size;
    auto height = [](int i) {
        int h = 0;
        while (!(i & 1)) {
            i >>= 1;
            h++;
        }
        return h;
    };
    int top = 1;
    while (top * 2 <= N)
        top *= 2;
    std::vector<int> par(N + 1, 0), lc(N + 1, 0), rc(N + 1, 0);
    for (int i = 1; i <= N; i++) {
        const int h = height(i);
        if (h == 0)
            continue;
        lc[i] = i - (1 << (h - 1));
        int r = 0;
        for (int k = h; k >= 1 && !r; k--) // highest existing node of the right subtree
            if (i + (1 << (k - 1)) <= N)
                r = i + (1 << (k - 1));
        rc[i] = r;
        par[lc[i]] = i;
        if (r)
            par[r] = i;
    }
    // position -> rank
    std::vector<int> at(N + 1, 0);
    for (int i = 1; i <= N; i++)
        at[i] = which == 0 ? i - 1 : i % N;
    if (root >= 0 && at[top] != root) {
        for (int i = 1; i <= N; i++)
            if (at[i] == root) {
                std::swap(at[i], at[top]);
                break;
            }
    }
    int me = 0;
    for (int i = 1; i <= N; i++)
        if (at[i] == rank)
            me = i;
    parent = par[me] ? at[par[me]] : -1;
    left = lc[me] ? at[lc[me]] : -1;
    right = rc[me] ? at[rc[me]] : -1;
    root_rank = at[top];
}

// reduce towards the root of `t`: accumulate the children's contributions into acc, hand the result up
static void reduce_bin_tree(sched& s, void* acc, size_t count, int dtype, int op, reduction_fn_t fn, const bin_tree& t,
                            uint64_t tag) {
    const size_t bytes = count * dtype_size(dtype);
    void* tmp = (t.left >= 0 || t.right >= 0) ? s.alloc_tmp(bytes + 64) : nullptr;
    for (int child : { t.left, t.right })
        if (child >= 0) {
            s.add<recv_reduce_entry>(acc, count, dtype, op, child, tag, fn, tmp);
            s.add_barrier();
        }
    if (t.parent >= 0) {
        s.add<send_entry>(acc, bytes, t.parent, tag);
        s.add_barrier();
    }
}

static void bcast_bin_tree(sched& s, void* buf, size_t bytes, const bin_tree& t, uint64_t tag) {
    if (t.parent >= 0) {
        s.add<recv_entry>(buf, bytes, t.parent, tag);
        s.add_barrier();
    }
    for (int child : { t.left, t.right })
        if (child >= 0)
            s.add<send_entry>(buf, bytes, child, tag);
    s.add_barrier();
}

// number of pipeline parts a half is cut into (CCL_DTREE_PARTITION_COUNT; reference
// src/coll/algorithms/double_tree_ops.cpp:146-151)
static size_t dtree_parts(size_t count) {
    const size_t want = std::min(std::max<size_t>(env_data::get().dtree_partition_count, 1), MAX_CHUNKS);
    return std::min(want, std::max<size_t>(count, 1));
}

void bcast_double_tree(sched& s, void* buf, size_t count, int dtype, int root) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    if (N == 1 || count == 0)
        return;
    const size_t esz = dtype_size(dtype);
    const size_t h0 = count / 2, h1 = count - h0;
    for (int which = 0; which < 2; which++) {
        const size_t n = which == 0 ? h0 : h1;
        if (n == 0)
            continue;
        void* base = which == 0 ? buf : at(buf, h0, esz);
        const bin_tree t(N, r, which, root);
        const size_t parts = dtree_parts(n);
        // the halves (and the parts of a half) are independent streams: sub-schedules progress side by side
        for (size_t k = 0; k < parts; k++) {
            size_t o, m;
            chunk_range(n, parts, k, o, m);
            void* p = at(base, o, esz);
            const uint64_t tag = 2000 * (uint64_t)which + k;
            s.add<subsched_entry>([=](sched& sub) { bcast_bin_tree(sub, p, m * esz, t, tag); },
                                  which == 0 ? "DTREE_BCAST_A" : "DTREE_BCAST_B");
        }
    }
    s.add_barrier();
}

void reduce_double_tree(sched& s, const buf_desc& b, int root) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    const size_t bytes = b.count * esz;
    // every rank accumulates in a work buffer; the root's is its recv buffer
    void* acc = b.recv;
    if (b.send) {
        if (r != root || !b.recv)
            acc = s.alloc_tmp(bytes + 64);
        if (acc != b.send) {
            s.add<copy_entry>(b.send, acc, bytes);
            s.add_barrier();
        }
    }
    if (N == 1 || b.count == 0)
        return;
    const size_t h0 = b.count / 2, h1 = b.count - h0;
    const int dtype = b.dtype, op = b.op;
    reduction_fn_t fn = b.fn;
    for (int which = 0; which < 2; which++) {
        const size_t n = which == 0 ? h0 : h1;
        if (n == 0)
            continue;
        void* base = which == 0 ? acc : at(acc, h0, esz);
        const bin_tree t(N, r, which, root);
        const size_t parts = dtree_parts(n);
        for (size_t k = 0; k < parts; k++) {
            size_t o, m;
            chunk_range(n, parts, k, o, m);
            void* p = at(base, o, esz);
            const uint64_t tag = 2000 * (uint64_t)which + k;
            s.add<subsched_entry>([=](sched& sub) { reduce_bin_tree(sub, p, m, dtype, op, fn, t, tag); },
                                  which == 0 ? "DTREE_REDUCE_A" : "DTREE_REDUCE_B");
        }
    }
    s.add_barrier();
}

void allreduce_double_tree(sched& s, const buf_desc& b) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    copy_in(s, b.send, b.recv, b.count * esz);
    if (N == 1 || b.count == 0)
        return;
    // Half 0 is reduced up tree A and broadcast down it, half 1 uses tree B; each tree keeps its own root, so
    // nothing is swapped and the trees stay exactly complementary.  Parts of a half follow one another: the
    // broadcast of part k runs beside the reduction of part k+1.
    const size_t h0 = b.count / 2, h1 = b.count - h0;
    const int dtype = b.dtype, op = b.op;
    reduction_fn_t fn = b.fn;
    void* recv = b.recv;
    for (int which = 0; which < 2; which++) {
        const size_t n = which == 0 ? h0 : h1;
        if (n == 0)
            continue;
        void* base = which == 0 ? recv : at(recv, h0, esz);
        const bin_tree t(N, r, which, -1);
        const size_t parts = dtree_parts(n);
        const uint64_t tag0 = 4000 * (uint64_t)which;
        s.add<subsched_entry>(
            [=](sched& half) {
                for (size_t k = 0; k <= parts; k++) {
                    if (k < parts) {
                        size_t o, m;
                        chunk_range(n, parts, k, o, m);
                        void* p = at(base, o, esz);
                        half.add<subsched_entry>(
                            [=](sched& ss) { reduce_bin_tree(ss, p, m, dtype, op, fn, t, tag0 + k); }, "DTREE_R");
                    }
                    if (k >= 1) {
                        size_t o, m;
                        chunk_range(n, parts, k - 1, o, m);
                        void* p = at(base, o, esz);
                        half.add<subsched_entry>(
                            [=](sched& ss) { bcast_bin_tree(ss, p, m * esz, t, tag0 + 2000 + (k - 1)); }, "DTREE_B");
                    }
                    half.add_barrier();
                }
            },
            which == 0 ? "DTREE_A" : "DTREE_B");
    }
    s.add_barrier();
}

// ---------------------------------------------------------------------------- alltoallv
namespace {
// In place (send == recv; every pair exchanges equal amounts, so the block layout is the same on both
// sides): blocks are received into scratch memory and copied over the send data once every send has left
// (reference src/coll/algorithms/alltoallv.cpp:129-200).
struct a2a_landing {
    char* base; // where block p lands: base + roffs[p] * esz
    bool staged;
};
a2a_landing a2a_prepare(sched& s, const void* send, void* recv, const std::vector<size_t>& scounts,
                        const std::vector<size_t>& soffs, const std::vector<size_t>& rcounts,
                        const std::vector<size_t>& roffs, size_t esz) {
    const int r = s.comm()->rank();
    if (send == recv) {
        size_t total = 0;
        for (size_t i = 0; i < rcounts.size(); i++)
            total = std::max(total, roffs[i] + rcounts[i]);
        return a2a_landing{ (char*)s.alloc_tmp(total * esz + 64), true };
    }
    s.add<copy_entry>(at(send, soffs[r], esz), at(recv, roffs[r], esz), std::min(scounts[r], rcounts[r]) * esz);
    return a2a_landing{ (char*)recv, false };
}
void a2a_finish(sched& s, const a2a_landing& l, void* recv, const std::vector<size_t>& rcounts,
                const std::vector<size_t>& roffs, size_t esz) {
    if (!l.staged)
        return;
    const int N = s.comm()->size(), r = s.comm()->rank();
    for (int p = 0; p < N; p++)
        if (p != r && rcounts[p])
            s.add<copy_entry>(l.base + roffs[p] * esz, at(recv, roffs[p], esz), rcounts[p] * esz);
    s.add_barrier();
}
} // namespace

void alltoallv_naive(sched& s, const void* send, const std::vector<size_t>& scounts, const std::vector<size_t>& soffs,
                     void* recv, const std::vector<size_t>& rcounts, const std::vector<size_t>& roffs, int dtype) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(dtype);
    const a2a_landing land = a2a_prepare(s, send, recv, scounts, soffs, rcounts, roffs, esz);
    for (int k = 1; k < N; k++) {
        const int src = (r - k + N) % N, dst = (r + k) % N;
        // The step is the distance between the ranks, as in alltoallv_scatter: the size table sees this
        // rank's own send total, so two ranks of one alltoallv may pick different patterns, and the
        // messages of the two must still match.
        chunked_recv(s, land.base + roffs[src] * esz, rcounts[src], esz, src, (uint64_t)k);
        chunked_send(s, at(send, soffs[dst], esz), scounts[dst], esz, dst, (uint64_t)k);
    }
    s.add_barrier();
    a2a_finish(s, land, recv, rcounts, roffs, esz);
}

void alltoallv_scatter(sched& s, const void* send, const std::vector<size_t>& scounts,
                       const std::vector<size_t>& soffs, void* recv, const std::vector<size_t>& rcounts,
                       const std::vector<size_t>& roffs, int dtype, size_t max_ops) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(dtype);
    if (max_ops == 0)
        max_ops = 1;
    const a2a_landing land = a2a_prepare(s, send, recv, scounts, soffs, rcounts, roffs, esz);
    // flow control: at most max_ops exchanges in flight, then a barrier point
    size_t in_batch = 0;
    for (int k = 1; k < N; k++) {
        const int src = (r - k + N) % N, dst = (r + k) % N;
        chunked_recv(s, land.base + roffs[src] * esz, rcounts[src], esz, src, (uint64_t)k);
        chunked_send(s, at(send, soffs[dst], esz), scounts[dst], esz, dst, (uint64_t)k);
        if (++in_batch == max_ops) {
            s.add_barrier();
            in_batch = 0;
        }
    }
    s.add_barrier();
    a2a_finish(s, land, recv, rcounts, roffs, esz);
}

// ---------------------------------------------------------------------------- barrier
void barrier_dissemination(sched& s) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    uint64_t step = 0;
    for (int d = 1; d < N; d *= 2, step++) {
        s.add<send_entry>(nullptr, 0, (r + d) % N, step);
        s.add<recv_entry>(nullptr, 0, (r - d + N) % N, step);
        s.add_barrier();
    }
}

void barrier_ring(sched& s) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    if (N == 1)
        return;
    // two trips of a token around the ring
    for (uint64_t trip = 0; trip < 2; trip++) {
        if (r == 0) {
            s.add<send_entry>(nullptr, 0, 1 % N, trip);
            s.add<recv_entry>(nullptr, 0, N - 1, trip);
        }
        else {
            s.add<recv_entry>(nullptr, 0, r - 1, trip);
            s.add_barrier();
            s.add<send_entry>(nullptr, 0, (r + 1) % N, trip);
        }
        s.add_barrier();
    }
}

// ---------------------------------------------------------------------------- bcast
void bcast_naive(sched& s, void* buf, size_t bytes, int root, uint64_t step_base) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    if (r == root) {
        for (int p = 0; p < N; p++)
            if (p != root)
                s.add<send_entry>(buf, bytes, p, step_base);
    }
    else
        s.add<recv_entry>(buf, bytes, root, step_base);
    s.add_barrier();
}

void bcast_tree(sched& s, void* buf, size_t bytes, int root, uint64_t step_base, int shift) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    (void)shift;
    if (N == 1)
        return;
    const int v = (r - root + N) % N;
    int mask = 1;
    while (mask < N) {
        if (v & mask) {
            s.add<recv_entry>(buf, bytes, ((v - mask) + root) % N, step_base);
            s.add_barrier();
            break;
        }
        mask <<= 1;
    }
    mask >>= 1;
    while (mask > 0) {
        if (v + mask < N)
            s.add<send_entry>(buf, bytes, ((v + mask) + root) % N, step_base);
        mask >>= 1;
    }
    s.add_barrier();
}

void bcast_ring(sched& s, void* buf, size_t count, int dtype, int root) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(dtype);
    if (N == 1)
        return;
    std::vector<size_t> cnt, off;
    block_partition(count, N, cnt, off);
    // scatter from the root, then a ring allgather
    if (r == root) {
        for (int p = 0; p < N; p++)
            if (p != root)
                s.add<send_entry>(at(buf, off[p], esz), cnt[p] * esz, p, 0);
    }
    else
        s.add<recv_entry>(at(buf, off[r], esz), cnt[r] * esz, root, 0);
    s.add_barrier();
    allgatherv_ring(s, nullptr, buf, cnt, off, dtype, 10);
}

// ---------------------------------------------------------------------------- reduce
void reduce_tree(sched& s, const buf_desc& b, int root, uint64_t step_base, int shift) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    (void)shift;
    const size_t esz = dtype_size(b.dtype);
    const size_t bytes = b.count * esz;
    // non-root ranks accumulate in scratch unless the caller reduces in place (send == nullptr)
    void* acc = b.recv;
    if (b.send) {
        if (r != root || !b.recv)
            acc = s.alloc_tmp(bytes + 64);
        if (acc != b.send) {
            s.add<copy_entry>(b.send, acc, bytes);
            s.add_barrier();
        }
    }
    if (N == 1)
        return;
    const int v = (r - root + N) % N;
    void* tmp = s.alloc_tmp(bytes + 64);
    int mask = 1;
    while (mask < N) {
        if (v & mask) {
            s.add<send_entry>(acc, bytes, ((v & ~mask) + root) % N, step_base);
            s.add_barrier();
            break;
        }
        const int child = v | mask;
        if (child < N) {
            s.add<recv_reduce_entry>(acc, b.count, b.dtype, b.op, (child + root) % N, step_base, b.fn, tmp);
            s.add_barrier();
        }
        mask <<= 1;
    }
}

void reduce_ring(sched& s, const buf_desc& b, int root) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    const size_t bytes = b.count * esz;
    if (N == 1) {
        copy_in(s, b.send, b.recv, bytes);
        return;
    }
    void* work = (r == root) ? b.recv : s.alloc_tmp(bytes + 64);
    if (b.send && b.send != work) {
        s.add<copy_entry>(b.send, work, bytes);
        s.add_barrier();
    }
    std::vector<size_t> cnt, off;
    block_partition(b.count, N, cnt, off);
    reduce_scatter_ring_v(s, work, cnt, off, b.dtype, b.op, b.fn, 0);
    // gather the reduced blocks at the root
    if (r == root) {
        for (int p = 0; p < N; p++)
            if (p != root)
                s.add<recv_entry>(at(work, off[p], esz), cnt[p] * esz, p, 2000);
    }
    else
        s.add<send_entry>(at(work, off[r], esz), cnt[r] * esz, root, 2000);
    s.add_barrier();
}

void reduce_rabenseifner(sched& s, const buf_desc& b, int root) {
    host_comm* c = s.comm();
    const int N = c->size(), r = c->rank();
    const size_t esz = dtype_size(b.dtype);
    const size_t bytes = b.count * esz;
    const fold f = make_fold(N, r);
    if (N == 1 || (size_t)f.pof2 > b.count) {
        reduce_tree(s, b, root);
        return;
    }
    void* work = (r == root) ? b.recv : s.alloc_tmp(bytes + 64);
    if (b.send && b.send != work) {
        s.add<copy_entry>(b.send, work, bytes);
        s.add_barrier();
    }
    if (r < 2 * f.rem) {
        if (f.newrank < 0)
            s.add<send_entry>(work, bytes, r + 1, 0);
        else
            s.add<recv_reduce_entry>(work, b.count, b.dtype, b.op, r - 1, 0, b.fn);
        s.add_barrier();
    }
    std::vector<size_t> cnt, off;
    block_partition(b.count, f.pof2, cnt, off);
    if (f.newrank >= 0)
        rs_recursive_halving(s, work, f, cnt, off, b.dtype, b.op, b.fn, 1);
    // every participant sends its block to the root
    if (r == root) {
        for (int nr = 0; nr < f.pof2; nr++) {
            const int p = f.real(nr);
            if (p != root)
                s.add<recv_entry>(at(work, off[nr], esz), cnt[nr] * esz, p, 3000);
        }
    }
    else if (f.newrank >= 0)
        s.add<send_entry>(at(work, off[f.newrank], esz), cnt[f.newrank] * esz, root, 3000);
    s.add_barrier();
}

// ---------------------------------------------------------------------------- point to point
void send_direct(sched& s, const void* buf, size_t bytes, int peer, uint64_t seq) {
    s.add<send_entry>(buf, bytes, peer, seq & 0xffff, /*one_way=*/true);
}
void recv_direct(sched& s, void* buf, size_t bytes, int peer, uint64_t seq) {
    s.add<recv_entry>(buf, bytes, peer, seq & 0xffff);
}

} // namespace algo
} // namespace cclx
