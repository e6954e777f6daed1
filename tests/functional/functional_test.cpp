// Functional matrix of the public C++ API on host buffers:
//   functional_test <rank> <size> <address-file> [keep-one-in]
//
// Same axes as the reference's functional suite (tests/functional/conf.hpp:44-140, oracle
// test_impl.hpp:241-324): datatype (12), element count (3), buffers in flight (1 or 4), in / out of
// place, start order and completion order (direct, reverse, shuffled), completion by wait or by test,
// cached or not (match_id per buffer, second iteration reuses the schedule), synchronous or not,
// reduction (sum, prod, min, max, custom).  The full cross product is large, so a deterministic hash of
// the configuration keeps one in `keep-one-in` (default 97); every rank evaluates the same hash, and
// every datatype x reduction pair is always kept once per operation.  Values are small integers, exact
// in every datatype including float16 / bfloat16, and every element is checked against a closed form.
// FUNCTIONAL_TEST_DYNAMIC_POINTER=1 re-allocates the buffers before the second iteration of a cached
// configuration; FUNCTIONAL_TEST_VERBOSE=1 names every configuration before it runs.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <numeric>
#include <string>
#include <vector>

#include "oneapi/ccl.hpp"
#include "store.hpp"

namespace {

int g_rank = 0, g_size = 1;
long g_configs = 0, g_failures = 0;
bool g_dynamic_pointers = false; // FUNCTIONAL_TEST_DYNAMIC_POINTER=1

// ---- datatypes ------------------------------------------------------------------------------
struct dtype_desc {
    ccl::datatype dt;
    const char* name;
    size_t size;
};
const dtype_desc DTYPES[] = {
    { ccl::datatype::int8, "int8", 1 },       { ccl::datatype::uint8, "uint8", 1 },
    { ccl::datatype::int16, "int16", 2 },     { ccl::datatype::uint16, "uint16", 2 },
    { ccl::datatype::int32, "int32", 4 },     { ccl::datatype::uint32, "uint32", 4 },
    { ccl::datatype::int64, "int64", 8 },     { ccl::datatype::uint64, "uint64", 8 },
    { ccl::datatype::float16, "float16", 2 }, { ccl::datatype::float32, "float32", 4 },
    { ccl::datatype::float64, "float64", 8 }, { ccl::datatype::bfloat16, "bfloat16", 2 },
};
constexpr int N_DTYPES = 12;

uint16_t to_half(float f) { // exact for the small integers used here; round to nearest even otherwise
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000;
    int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    uint32_t man = x & 0x7fffff;
    if (exp <= 0)
        return (uint16_t)sign;
    if (exp >= 31)
        return (uint16_t)(sign | 0x7c00);
    uint32_t h = sign | ((uint32_t)exp << 10) | (man >> 13);
    if ((man & 0x1fff) > 0x1000 || ((man & 0x1fff) == 0x1000 && (h & 1)))
        h++;
    return (uint16_t)h;
}
float from_half(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    const uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff;
    uint32_t x;
    if (exp == 0)
        x = sign; // subnormals do not occur here
    else if (exp == 31)
        x = sign | 0x7f800000 | (man << 13);
    else
        x = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}
uint16_t to_bf16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    x += 0x7fff + ((x >> 16) & 1);
    return (uint16_t)(x >> 16);
}
float from_bf16(uint16_t b) {
    const uint32_t x = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

void put(void* base, size_t i, int d, long v) {
    char* p = (char*)base + i * DTYPES[d].size;
    switch (d) {
        case 0: *(int8_t*)p = (int8_t)v; break;
        case 1: *(uint8_t*)p = (uint8_t)v; break;
        case 2: *(int16_t*)p = (int16_t)v; break;
        case 3: *(uint16_t*)p = (uint16_t)v; break;
        case 4: *(int32_t*)p = (int32_t)v; break;
        case 5: *(uint32_t*)p = (uint32_t)v; break;
        case 6: *(int64_t*)p = (int64_t)v; break;
        case 7: *(uint64_t*)p = (uint64_t)v; break;
        case 8: *(uint16_t*)p = to_half((float)v); break;
        case 9: *(float*)p = (float)v; break;
        case 10: *(double*)p = (double)v; break;
        case 11: *(uint16_t*)p = to_bf16((float)v); break;
    }
}
long get(const void* base, size_t i, int d) {
    const char* p = (const char*)base + i * DTYPES[d].size;
    switch (d) {
        case 0: return *(const int8_t*)p;
        case 1: return *(const uint8_t*)p;
        case 2: return *(const int16_t*)p;
        case 3: return *(const uint16_t*)p;
        case 4: return *(const int32_t*)p;
        case 5: return (long)*(const uint32_t*)p;
        case 6: return (long)*(const int64_t*)p;
        case 7: return (long)*(const uint64_t*)p;
        case 8: return std::lround(from_half(*(const uint16_t*)p));
        case 9: return std::lround(*(const float*)p);
        case 10: return std::lround(*(const double*)p);
        case 11: return std::lround(from_bf16(*(const uint16_t*)p));
    }
    return 0;
}

// ---- the axes -------------------------------------------------------------------------------
enum op_kind { OP_ALLGATHER, OP_ALLGATHERV, OP_ALLREDUCE, OP_ALLTOALL, OP_ALLTOALLV, OP_BROADCAST, OP_REDUCE,
               OP_REDUCE_SCATTER, OP_LAST };
const char* OP_NAMES[] = { "allgather", "allgatherv", "allreduce", "alltoall", "alltoallv", "broadcast", "reduce",
                           "reduce_scatter" };
enum red_kind { RED_SUM, RED_PROD, RED_MIN, RED_MAX, RED_CUSTOM, RED_LAST };
const char* RED_NAMES[] = { "sum", "prod", "min", "max", "custom" };
const size_t COUNTS[] = { 7, 1027, 65539 };
const int BUFFERS[] = { 1, 4 };
enum order_kind { ORDER_DIRECT, ORDER_REVERSE, ORDER_SHUFFLED, ORDER_LAST };

struct config {
    int op, dtype, count_idx, buffers_idx, in_place, start_order, complete_order, use_test, cached, synchronous, red;
    std::string str() const {
        return std::string(OP_NAMES[op]) + " " + DTYPES[dtype].name + " count=" + std::to_string(COUNTS[count_idx]) +
               " buffers=" + std::to_string(BUFFERS[buffers_idx]) + (in_place ? " in-place" : " out-of-place") +
               " start=" + std::to_string(start_order) + " complete=" + std::to_string(complete_order) +
               (use_test ? " test" : " wait") + (cached ? " cached" : "") + (synchronous ? " sync" : "") + " " +
               RED_NAMES[red];
    }
    uint64_t hash() const {
        uint64_t h = 1469598103934665603ull;
        for (int v : { op, dtype, count_idx, buffers_idx, in_place, start_order, complete_order, use_test, cached,
                       synchronous, red }) {
            h ^= (uint64_t)(v + 1);
            h *= 1099511628211ull;
        }
        return h ^ (h >> 29);
    }
};

bool has_reduction(int op) {
    return op == OP_ALLREDUCE || op == OP_REDUCE || op == OP_REDUCE_SCATTER;
}

// value of element i of send buffer b on rank p; small enough that sums and products over the ranks
// stay exact in every datatype (int8 and bfloat16 bound them: |x| <= 127, integers up to 256)
long fill_value(int p, int b, size_t i, int red) {
    if (red == RED_PROD)
        return 1 + (long)((p + b + i) % 2);
    return 1 + (long)((p * 2 + b + i) % 5);
}
long reduce_values(int red, int b, size_t i) {
    long acc = fill_value(0, b, i, red);
    for (int p = 1; p < g_size; p++) {
        const long v = fill_value(p, b, i, red);
        switch (red) {
            case RED_SUM:
            case RED_CUSTOM: acc += v; break; // the custom function below is a sum
            case RED_PROD: acc *= v; break;
            case RED_MIN: acc = std::min(acc, v); break;
            case RED_MAX: acc = std::max(acc, v); break;
        }
    }
    return acc;
}

// custom reduction: element-wise sum written against the public callback signature
void custom_sum(const void* in, size_t n, void* inout, size_t* out_n, ccl::datatype dt, const ccl::fn_context*) {
    int d = 0;
    for (int k = 0; k < N_DTYPES; k++)
        if (DTYPES[k].dt == dt)
            d = k;
    for (size_t i = 0; i < n; i++)
        put(inout, i, d, get(in, i, d) + get(inout, i, d));
    if (out_n)
        *out_n = n;
}

ccl::reduction to_reduction(int red) {
    switch (red) {
        case RED_SUM: return ccl::reduction::sum;
        case RED_PROD: return ccl::reduction::prod;
        case RED_MIN: return ccl::reduction::min;
        case RED_MAX: return ccl::reduction::max;
        default: return ccl::reduction::custom;
    }
}

std::vector<int> make_order(int kind, int n, uint64_t seed) {
    std::vector<int> o(n);
    std::iota(o.begin(), o.end(), 0);
    if (kind == ORDER_REVERSE)
        std::reverse(o.begin(), o.end());
    else if (kind == ORDER_SHUFFLED)
        for (int i = n - 1; i > 0; i--) {
            seed = seed * 6364136223846793005ull + 1442695040888963407ull;
            std::swap(o[i], o[(int)((seed >> 33) % (uint64_t)(i + 1))]);
        }
    return o;
}

template <class Attr>
Attr make_attr(const config& c, int b) {
    auto attr = ccl::create_operation_attr<Attr>();
    if (c.cached) {
        attr.template set<ccl::operation_attr_id::to_cache>(true);
        attr.template set<ccl::operation_attr_id::match_id>(ccl::string_class(c.str() + "#" + std::to_string(b)));
    }
    if (c.synchronous)
        attr.template set<ccl::operation_attr_id::synchronous>(true);
    return attr;
}

// ---- one configuration ------------------------------------------------------------------------
struct buffers {
    std::vector<std::vector<char>> send, recv; // per buffer in flight
};

size_t agv_count(size_t count, int p) { // allgatherv: rank p contributes count + p elements
    return count + (size_t)p;
}
// alltoallv: what rank `from` sends to rank `to`; symmetric, as the in-place form requires
size_t a2av_count(size_t count, int from, int to) {
    return 1 + (count / 4) * (size_t)(1 + (from + to) % 3);
}

bool run_config(const config& c, const ccl::communicator& comm) {
    const int N = g_size, R = g_rank, d = c.dtype, B = BUFFERS[c.buffers_idx];
    const size_t count = COUNTS[c.count_idx], esz = DTYPES[d].size;
    const ccl::datatype dt = DTYPES[d].dt;
    // element counts of the send and recv sides
    size_t send_elems = count, recv_elems = count;
    std::vector<size_t> agv(N), sc(N), rc(N);
    switch (c.op) {
        case OP_ALLGATHER: recv_elems = count * N; break;
        case OP_ALLGATHERV:
            recv_elems = 0;
            for (int p = 0; p < N; p++) {
                agv[p] = agv_count(count, p);
                recv_elems += agv[p];
            }
            send_elems = agv[R];
            break;
        case OP_ALLTOALL: send_elems = recv_elems = count * N; break;
        case OP_ALLTOALLV:
            send_elems = recv_elems = 0;
            for (int p = 0; p < N; p++) {
                sc[p] = a2av_count(count, R, p);
                rc[p] = a2av_count(count, p, R);
                send_elems += sc[p];
                recv_elems += rc[p];
            }
            break;
        case OP_REDUCE_SCATTER: send_elems = count * N; break;
        default: break;
    }
    buffers bufs;
    bufs.send.assign(B, std::vector<char>());
    bufs.recv.assign(B, std::vector<char>());
    for (int b = 0; b < B; b++) {
        bufs.send[b].resize(std::max(send_elems, recv_elems) * esz);
        bufs.recv[b].resize(std::max(send_elems, recv_elems) * esz);
    }
    const int iterations = c.cached ? 2 : 1; // the second run takes the schedule from the cache
    bool ok = true;
    for (int it = 0; it < iterations && ok; it++) {
        if (it > 0 && g_dynamic_pointers) {
            // the reference's "dynamic pointer" mode (test_impl.hpp:326-372): new allocations under the
            // same match_id; the old ones stay alive so that the addresses really differ
            for (int b = 0; b < B; b++) {
                bufs.send.emplace_back(bufs.send[b].size());
                bufs.recv.emplace_back(bufs.recv[b].size());
                std::swap(bufs.send[b], bufs.send.back());
                std::swap(bufs.recv[b], bufs.recv.back());
            }
        }
        // ---- fill: the in-place forms keep their input where the operation defines it
        std::vector<void*> sptr(B), rptr(B);
        for (int b = 0; b < B; b++) {
            char* s = bufs.send[b].data();
            char* r = bufs.recv[b].data();
            for (size_t i = 0; i < bufs.recv[b].size() / esz; i++)
                put(r, i, d, 99);
            const int root = b % N;
            if (c.in_place) {
                switch (c.op) {
                    case OP_ALLGATHER: s = r + (size_t)R * count * esz; break;
                    case OP_ALLGATHERV: {
                        size_t off = 0;
                        for (int p = 0; p < R; p++)
                            off += agv[p];
                        s = r + off * esz;
                        break;
                    }
                    case OP_REDUCE_SCATTER: r = s + (size_t)R * count * esz; break; // recv inside send
                    default: s = r; break;
                }
            }
            for (size_t i = 0; i < send_elems; i++) {
                long v = fill_value(R, b, i, c.red);
                if (c.op == OP_BROADCAST && R != root)
                    v = 77; // only the root's data may survive
                put(s, i, d, v);
            }
            sptr[b] = s;
            rptr[b] = r;
        }
        // ---- start in the configured order (the same on every rank)
        const std::vector<int> start = make_order(c.start_order, B, c.hash());
        std::vector<ccl::event> events(B);
        for (int b : start) {
            const int root = b % N;
            switch (c.op) {
                case OP_ALLGATHER:
                    events[b] = ccl::allgather(sptr[b], rptr[b], count, dt, comm, make_attr<ccl::allgather_attr>(c, b));
                    break;
                case OP_ALLGATHERV:
                    events[b] = ccl::allgatherv(sptr[b], agv[R], rptr[b], agv, dt, comm,
                                                make_attr<ccl::allgatherv_attr>(c, b));
                    break;
                case OP_ALLREDUCE: {
                    auto attr = make_attr<ccl::allreduce_attr>(c, b);
                    if (c.red == RED_CUSTOM)
                        attr.set<ccl::allreduce_attr_id::reduction_fn>((ccl::reduction_fn)custom_sum);
                    events[b] = ccl::allreduce(sptr[b], rptr[b], count, dt, to_reduction(c.red), comm, attr);
                    break;
                }
                case OP_ALLTOALL:
                    events[b] = ccl::alltoall(sptr[b], rptr[b], count, dt, comm, make_attr<ccl::alltoall_attr>(c, b));
                    break;
                case OP_ALLTOALLV:
                    events[b] = ccl::alltoallv(sptr[b], sc, rptr[b], rc, dt, comm, make_attr<ccl::alltoallv_attr>(c, b));
                    break;
                case OP_BROADCAST:
                    if (c.in_place)
                        events[b] = ccl::broadcast(rptr[b], count, dt, root, comm, make_attr<ccl::broadcast_attr>(c, b));
                    else
                        events[b] = ccl::broadcast(sptr[b], rptr[b], count, dt, root, comm,
                                                   make_attr<ccl::broadcast_attr>(c, b));
                    break;
                case OP_REDUCE: {
                    auto attr = make_attr<ccl::reduce_attr>(c, b);
                    if (c.red == RED_CUSTOM)
                        attr.set<ccl::reduce_attr_id::reduction_fn>((ccl::reduction_fn)custom_sum);
                    events[b] = ccl::reduce(sptr[b], rptr[b], count, dt, to_reduction(c.red), root, comm, attr);
                    break;
                }
                case OP_REDUCE_SCATTER: {
                    auto attr = make_attr<ccl::reduce_scatter_attr>(c, b);
                    if (c.red == RED_CUSTOM)
                        attr.set<ccl::reduce_scatter_attr_id::reduction_fn>((ccl::reduction_fn)custom_sum);
                    events[b] = ccl::reduce_scatter(sptr[b], rptr[b], count, dt, to_reduction(c.red), comm, attr);
                    break;
                }
            }
        }
        // ---- complete in an order of this rank's own
        const std::vector<int> finish = make_order(c.complete_order, B, c.hash() * 31 + (uint64_t)R);
        if (c.use_test) {
            std::vector<char> done(B, 0);
            int left = B;
            while (left > 0)
                for (int b : finish)
                    if (!done[b] && events[b].test()) {
                        done[b] = 1;
                        left--;
                    }
        }
        else
            for (int b : finish)
                events[b].wait();
        // ---- check every element
        for (int b = 0; b < B && ok; b++) {
            const char* r = (const char*)rptr[b];
            const int root = b % N;
            auto expect = [&](size_t i, long want, const char* what) {
                const long got = get(r, i, d);
                if (got != want && ok) {
                    ok = false;
                    std::cout << "FAILED rank " << R << ": " << c.str() << " iteration " << it << " buffer " << b << " "
                              << what << "[" << i << "] = " << got << ", expected " << want << std::endl;
                }
            };
            switch (c.op) {
                case OP_ALLGATHER:
                    for (int p = 0; p < N; p++)
                        for (size_t i = 0; i < count; i++)
                            expect((size_t)p * count + i, fill_value(p, b, i, c.red), "recv");
                    break;
                case OP_ALLGATHERV: {
                    size_t off = 0;
                    for (int p = 0; p < N; p++) {
                        for (size_t i = 0; i < agv[p]; i++)
                            expect(off + i, fill_value(p, b, i, c.red), "recv");
                        off += agv[p];
                    }
                    break;
                }
                case OP_ALLREDUCE:
                    for (size_t i = 0; i < count; i++)
                        expect(i, reduce_values(c.red, b, i), "recv");
                    break;
                case OP_ALLTOALL:
                    for (int p = 0; p < N; p++)
                        for (size_t i = 0; i < count; i++)
                            expect((size_t)p * count + i, fill_value(p, b, (size_t)R * count + i, c.red), "recv");
                    break;
                case OP_ALLTOALLV: {
                    size_t off = 0;
                    for (int p = 0; p < N; p++) {
                        // rank p keeps the block for rank R after the blocks for ranks 0..R-1
                        size_t soff = 0;
                        for (int q = 0; q < R; q++)
                            soff += a2av_count(count, p, q);
                        for (size_t i = 0; i < rc[p]; i++)
                            expect(off + i, fill_value(p, b, soff + i, c.red), "recv");
                        off += rc[p];
                    }
                    break;
                }
                case OP_BROADCAST:
                    for (size_t i = 0; i < count; i++)
                        expect(i, fill_value(root, b, i, c.red), "recv");
                    break;
                case OP_REDUCE:
                    if (R == root)
                        for (size_t i = 0; i < count; i++)
                            expect(i, reduce_values(c.red, b, i), "recv");
                    break;
                case OP_REDUCE_SCATTER:
                    for (size_t i = 0; i < count; i++)
                        expect(i, reduce_values(c.red, b, (size_t)R * count + i), "recv");
                    break;
            }
            // out of place: the send buffer is untouched
            if (!c.in_place && ok && c.op != OP_BROADCAST) {
                const char* s = (const char*)sptr[b];
                for (size_t i = 0; i < send_elems; i++)
                    if (get(s, i, d) != fill_value(R, b, i, c.red)) {
                        ok = false;
                        std::cout << "FAILED rank " << R << ": " << c.str() << " send buffer changed at " << i
                                  << std::endl;
                        break;
                    }
            }
        }
    }
    return ok;
}

} // namespace

int main(int argc, char** argv) {
    if (argc < 4) {
        std::cerr << "usage: " << argv[0] << " <rank> <size> <address-file> [keep-one-in]\n";
        return 2;
    }
    g_rank = std::atoi(argv[1]);
    g_size = std::atoi(argv[2]);
    const uint64_t keep = argc > 4 ? (uint64_t)std::atoll(argv[4]) : 97;
    g_dynamic_pointers = std::getenv("FUNCTIONAL_TEST_DYNAMIC_POINTER") != nullptr;
    const bool verbose = std::getenv("FUNCTIONAL_TEST_VERBOSE") != nullptr; // names every configuration first
    ccl::init();
    auto kvs = bootstrap_kvs(g_rank, argv[3]);
    auto comm = ccl::create_communicator(g_size, g_rank, kvs);
    std::vector<long> per_op(OP_LAST, 0);
    config c{};
    for (c.op = 0; c.op < OP_LAST; c.op++)
        for (c.dtype = 0; c.dtype < N_DTYPES; c.dtype++)
            for (c.red = 0; c.red < RED_LAST; c.red++) {
                if (!has_reduction(c.op) && c.red != RED_SUM)
                    continue;
                // products overflow nothing here, but the custom function sums: keep it to reductions
                bool first_of_pair = true;
                for (c.count_idx = 0; c.count_idx < 3; c.count_idx++)
                    for (c.buffers_idx = 0; c.buffers_idx < 2; c.buffers_idx++)
                        for (c.in_place = 0; c.in_place < 2; c.in_place++)
                            for (c.start_order = 0; c.start_order < ORDER_LAST; c.start_order++)
                                for (c.complete_order = 0; c.complete_order < ORDER_LAST; c.complete_order++)
                                    for (c.use_test = 0; c.use_test < 2; c.use_test++)
                                        for (c.cached = 0; c.cached < 2; c.cached++)
                                            for (c.synchronous = 0; c.synchronous < 2; c.synchronous++) {
                                                const bool keep_it = first_of_pair || keep <= 1 || c.hash() % keep == 0;
                                                first_of_pair = false;
                                                if (!keep_it)
                                                    continue;
                                                g_configs++;
                                                per_op[c.op]++;
                                                if (verbose)
                                                    std::cout << "rank " << g_rank << " #" << g_configs << " " << c.str()
                                                              << std::endl;
                                                if (!run_config(c, comm))
                                                    g_failures++;
                                            }
            }
    ccl::barrier(comm).wait();
    if (g_rank == 0) {
        for (int op = 0; op < OP_LAST; op++)
            std::cout << OP_NAMES[op] << ": " << per_op[op] << " configurations" << std::endl;
        std::cout << "functional: " << g_configs << " configurations, " << g_failures << " failed: "
                  << (g_failures ? "FAILED" : "PASSED") << std::endl;
    }
    return g_failures ? 1 : 0;
}
