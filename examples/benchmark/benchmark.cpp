// Collective benchmark through the public API, with the option set of the reference's tool
// (examples/benchmark/include/benchmark.hpp:46-106, doc/rst/source/benchmark-guide/benchmark.rst):
//
//   benchmark <rank> <size> <address-file> [options]          (no mpirun: ranks are plain processes)
//
//   -b, --backend host|cuda        where the buffers live (cuda needs a build with -DCCL_BENCH_CUDA)   [host]
//   -i, --iters N                  timed iterations                                                    [16]
//   -w, --warmup_iters N           untimed iterations                                                  [16]
//   -j, --iter_policy off|auto     auto halves the iteration count for every doubling above 256 KiB    [auto]
//   -n, --buf_count N              operations in flight per iteration, each with its own buffers       [1]
//   -f, --min_elem_count N         smallest element count                                              [0]
//   -t, --max_elem_count N         largest element count (powers of two in between)                    [128]
//   -y, --elem_counts a,b,c        explicit list of element counts
//   -c, --check off|last|all       compare the results with the closed form                            [last]
//   -p, --cache 0|1                persistent operations (to_cache + match_id)                         [1]
//   -q, --inplace 0|1              send buffer == recv buffer                                          [0]
//   -l, --coll list|all            allgather,allgatherv,allreduce,alltoall,alltoallv,bcast,reduce,reduce_scatter
//   -d, --dtype list|all           int8,int32,int64,uint64,float16,float32,float64,bfloat16           [float32]
//   -r, --reduction list|all       sum,prod,min,max                                                    [sum]
//   -o, --csv_filepath FILE        also write the rows to FILE (rank 0)
//   -x, --ext off|auto|on          on: add wait_t_avg (time from the return of the call to completion)  [auto]
//
// Output, one row per collective x datatype x reduction x count (times in microseconds):
//   coll,dtype,reduction,elem_count,bytes,repetitions,t_min,t_max,t_avg,stddev_pct[,wait_t_avg]
// t_min / t_max: mean over the iterations of the fastest / slowest rank of each iteration; t_avg: mean over
// ranks and iterations; stddev: of the per-iteration rank average, in percent of t_avg.
// The old positional form `benchmark <rank> <size> <file> <coll> <min> <max> <iters> <warmup>` still works.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <numeric>
#include <sstream>
#include <string>
#include <vector>

#ifdef CCL_BENCH_CUDA
#include <cuda_runtime.h>
#endif

#include "oneapi/ccl.hpp"
#include "store.hpp"

namespace {

struct options {
    std::string backend = "host";
    int iters = 16, warmup = 16;
    bool iter_auto = true;
    int buf_count = 1;
    size_t min_count = 0, max_count = 128;
    std::vector<size_t> counts;
    std::string check = "last";
    bool cache = true, inplace = false;
    std::vector<std::string> colls{ "allreduce" }, dtypes{ "float32" }, reductions{ "sum" };
    std::string csv;
    std::string ext = "auto";
};

const char* ALL_COLLS[] = { "allgather", "allgatherv", "allreduce", "alltoall", "alltoallv", "bcast", "reduce", "reduce_scatter" };
const char* ALL_DTYPES[] = { "int8", "int32", "int64", "uint64", "float16", "float32", "float64", "bfloat16" };
const char* ALL_REDUCTIONS[] = { "sum", "prod", "min", "max" };

std::vector<std::string> split(const std::string& s) {
    std::vector<std::string> out;
    std::stringstream ss(s);
    std::string tok;
    while (std::getline(ss, tok, ','))
        if (!tok.empty())
            out.push_back(tok == "reduce-scatter" ? "reduce_scatter" : (tok == "broadcast" ? "bcast" : tok));
    return out;
}

template <size_t K>
std::vector<std::string> list_or_all(const std::string& v, const char* (&all)[K]) {
    if (v == "all")
        return std::vector<std::string>(all, all + K);
    auto out = split(v);
    for (auto& x : out)
        if (std::find(all, all + K, x) == all + K) {
            std::cerr << "unknown value '" << x << "'\n";
            std::exit(2);
        }
    return out;
}

void usage(const char* app) {
    std::cerr << "usage: " << app
              << " <rank> <size> <address-file> [-b host|cuda] [-i iters] [-w warmup] [-j off|auto] [-n buf_count]\n"
                 "       [-f min_elem_count] [-t max_elem_count] [-y counts] [-c off|last|all] [-p 0|1] [-q 0|1]\n"
                 "       [-l colls|all] [-d dtypes|all] [-r reductions|all] [-o csv] [-x off|auto|on]\n";
}

bool parse(int argc, char** argv, options& o) {
    for (int i = 4; i < argc; i++) {
        std::string a = argv[i];
        auto is = [&](const char* s, const char* l) { return a == s || a == l; };
        if (is("-h", "--help"))
            return false;
        if (i + 1 >= argc) {
            std::cerr << "option " << a << " needs a value\n";
            return false;
        }
        const std::string v = argv[++i];
        if (is("-b", "--backend"))
            o.backend = v == "sycl" ? "cuda" : v;
        else if (is("-i", "--iters"))
            o.iters = std::atoi(v.c_str());
        else if (is("-w", "--warmup_iters"))
            o.warmup = std::atoi(v.c_str());
        else if (is("-j", "--iter_policy"))
            o.iter_auto = v == "auto";
        else if (is("-n", "--buf_count"))
            o.buf_count = std::max(1, std::atoi(v.c_str()));
        else if (is("-f", "--min_elem_count"))
            o.min_count = std::strtoull(v.c_str(), nullptr, 10);
        else if (is("-t", "--max_elem_count"))
            o.max_count = std::strtoull(v.c_str(), nullptr, 10);
        else if (is("-y", "--elem_counts"))
            for (auto& c : split(v))
                o.counts.push_back(std::strtoull(c.c_str(), nullptr, 10));
        else if (is("-c", "--check"))
            o.check = v;
        else if (is("-p", "--cache"))
            o.cache = v != "0";
        else if (is("-q", "--inplace"))
            o.inplace = v != "0";
        else if (is("-l", "--coll"))
            o.colls = list_or_all(v, ALL_COLLS);
        else if (is("-d", "--dtype"))
            o.dtypes = list_or_all(v, ALL_DTYPES);
        else if (is("-r", "--reduction"))
            o.reductions = list_or_all(v, ALL_REDUCTIONS);
        else if (is("-o", "--csv_filepath"))
            o.csv = v;
        else if (is("-x", "--ext"))
            o.ext = v;
        else {
            std::cerr << "unknown option " << a << "\n";
            return false;
        }
    }
    if (o.counts.empty()) {
        // min, the powers of two above it, max
        o.counts.push_back(o.min_count);
        for (size_t c = 1; c < o.max_count; c *= 2)
            if (c > o.min_count)
                o.counts.push_back(c);
        if (o.max_count > o.min_count)
            o.counts.push_back(o.max_count);
    }
    return true;
}

// ---- datatypes: values are small integers, exact in every type --------------------------------------
struct dtype_info {
    const char* name;
    ccl::datatype dt;
    size_t size;
};
const dtype_info DTYPES[] = { { "int8", ccl::datatype::int8, 1 },       { "int32", ccl::datatype::int32, 4 },
                              { "int64", ccl::datatype::int64, 8 },     { "uint64", ccl::datatype::uint64, 8 },
                              { "float16", ccl::datatype::float16, 2 }, { "float32", ccl::datatype::float32, 4 },
                              { "float64", ccl::datatype::float64, 8 }, { "bfloat16", ccl::datatype::bfloat16, 2 } };

const dtype_info& dtype_of(const std::string& name) {
    for (auto& d : DTYPES)
        if (name == d.name)
            return d;
    std::cerr << "unknown datatype " << name << "\n";
    std::exit(2);
}

uint16_t to_half(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000;
    const int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    if (exp <= 0)
        return (uint16_t)sign;
    if (exp >= 31)
        return (uint16_t)(sign | 0x7c00);
    return (uint16_t)(sign | ((uint32_t)exp << 10) | ((x & 0x7fffff) >> 13));
}
float from_half(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
    const uint32_t x = exp == 0 ? sign : (sign | ((exp - 15 + 127) << 23) | (man << 13));
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

void put(void* base, size_t i, const dtype_info& d, long v) {
    char* p = (char*)base + i * d.size;
    switch (d.dt) {
        case ccl::datatype::int8: *(int8_t*)p = (int8_t)v; break;
        case ccl::datatype::int32: *(int32_t*)p = (int32_t)v; break;
        case ccl::datatype::int64: *(int64_t*)p = (int64_t)v; break;
        case ccl::datatype::uint64: *(uint64_t*)p = (uint64_t)v; break;
        case ccl::datatype::float16: *(uint16_t*)p = to_half((float)v); break;
        case ccl::datatype::float32: *(float*)p = (float)v; break;
        case ccl::datatype::float64: *(double*)p = (double)v; break;
        case ccl::datatype::bfloat16: {
            const float f = (float)v;
            uint32_t x;
            std::memcpy(&x, &f, 4);
            *(uint16_t*)p = (uint16_t)(x >> 16);
            break;
        }
        default: break;
    }
}
long get(const void* base, size_t i, const dtype_info& d) {
    const char* p = (const char*)base + i * d.size;
    switch (d.dt) {
        case ccl::datatype::int8: return *(const int8_t*)p;
        case ccl::datatype::int32: return *(const int32_t*)p;
        case ccl::datatype::int64: return (long)*(const int64_t*)p;
        case ccl::datatype::uint64: return (long)*(const uint64_t*)p;
        case ccl::datatype::float16: return std::lround(from_half(*(const uint16_t*)p));
        case ccl::datatype::float32: return std::lround(*(const float*)p);
        case ccl::datatype::float64: return std::lround(*(const double*)p);
        case ccl::datatype::bfloat16: {
            const uint32_t x = (uint32_t) * (const uint16_t*)p << 16;
            float f;
            std::memcpy(&f, &x, 4);
            return std::lround(f);
        }
        default: return 0;
    }
}

ccl::reduction reduction_of(const std::string& r) {
    return r == "prod" ? ccl::reduction::prod : r == "min" ? ccl::reduction::min : r == "max" ? ccl::reduction::max
                                                                                              : ccl::reduction::sum;
}

// element i of the send buffer of rank p, buffer b; products stay below 2^size
long fill_value(int p, int b, size_t i, const std::string& red) {
    if (red == "prod")
        return 1 + (long)((p + b + i) % 2);
    return 1 + (long)((p + b + i) % 3);
}
long reduced(int size, int b, size_t i, const std::string& red) {
    long acc = fill_value(0, b, i, red);
    for (int p = 1; p < size; p++) {
        const long v = fill_value(p, b, i, red);
        acc = red == "prod" ? acc * v : red == "min" ? std::min(acc, v) : red == "max" ? std::max(acc, v) : acc + v;
    }
    return acc;
}

// ---- buffers on the host or on the device --------------------------------------------------------------
struct buffer {
    std::vector<char> host; // always present: filled and checked here
    void* dev = nullptr; // backend cuda
    void* ptr() { return dev ? dev : (void*)host.data(); }
};

#ifdef CCL_BENCH_CUDA
cudaStream_t g_stream = nullptr;
#endif

void allocate(buffer& b, size_t bytes, bool cuda) {
    b.host.assign(std::max<size_t>(bytes, 1), 0);
    (void)cuda;
#ifdef CCL_BENCH_CUDA
    if (cuda)
        cudaMalloc(&b.dev, std::max<size_t>(bytes, 16));
#endif
}
void release(buffer& b) {
#ifdef CCL_BENCH_CUDA
    if (b.dev)
        cudaFree(b.dev);
#endif
    b.dev = nullptr;
}
void to_device(buffer& b) {
#ifdef CCL_BENCH_CUDA
    if (b.dev) {
        cudaMemcpyAsync(b.dev, b.host.data(), b.host.size(), cudaMemcpyHostToDevice, g_stream);
        cudaStreamSynchronize(g_stream);
    }
#else
    (void)b;
#endif
}
void to_host(buffer& b) {
#ifdef CCL_BENCH_CUDA
    if (b.dev) {
        cudaMemcpyAsync(b.host.data(), b.dev, b.host.size(), cudaMemcpyDeviceToHost, g_stream);
        cudaStreamSynchronize(g_stream);
    }
#else
    (void)b;
#endif
}

} // namespace

namespace {

struct sizes {
    size_t send_elems, recv_elems;
};
sizes elems_of(const std::string& coll, size_t count, int size) {
    if (coll == "allgather" || coll == "allgatherv")
        return { count, count * (size_t)size };
    if (coll == "alltoall" || coll == "alltoallv")
        return { count * (size_t)size, count * (size_t)size };
    if (coll == "reduce_scatter")
        return { count * (size_t)size, count };
    return { count, count };
}

template <class Attr>
Attr make_attr(bool cache, const std::string& id) {
    auto a = ccl::create_operation_attr<Attr>();
    if (cache) {
        a.template set<ccl::operation_attr_id::to_cache>(true);
        a.template set<ccl::operation_attr_id::match_id>(ccl::string_class(id));
    }
    return a;
}

#define WITH_STREAM(call_with, call_without) (stream ? (call_with) : (call_without))

ccl::event start_one(const std::string& coll, const dtype_info& d, const std::string& red, size_t count, void* send,
                     void* recv, const ccl::communicator& comm, const ccl::stream* stream, bool cache,
                     const std::string& id) {
    const int N = comm.size();
    const ccl::reduction r = reduction_of(red);
    if (coll == "allreduce") {
        auto a = make_attr<ccl::allreduce_attr>(cache, id);
        return WITH_STREAM(ccl::allreduce(send, recv, count, d.dt, r, comm, *stream, a),
                           ccl::allreduce(send, recv, count, d.dt, r, comm, a));
    }
    if (coll == "reduce") {
        auto a = make_attr<ccl::reduce_attr>(cache, id);
        return WITH_STREAM(ccl::reduce(send, recv, count, d.dt, r, 0, comm, *stream, a),
                           ccl::reduce(send, recv, count, d.dt, r, 0, comm, a));
    }
    if (coll == "bcast") {
        auto a = make_attr<ccl::broadcast_attr>(cache, id);
        return WITH_STREAM(ccl::broadcast(recv, count, d.dt, 0, comm, *stream, a),
                           ccl::broadcast(recv, count, d.dt, 0, comm, a));
    }
    if (coll == "allgather") {
        auto a = make_attr<ccl::allgather_attr>(cache, id);
        return WITH_STREAM(ccl::allgather(send, recv, count, d.dt, comm, *stream, a),
                           ccl::allgather(send, recv, count, d.dt, comm, a));
    }
    if (coll == "allgatherv") {
        auto a = make_attr<ccl::allgatherv_attr>(cache, id);
        const ccl::vector_class<size_t> counts(N, count);
        return WITH_STREAM(ccl::allgatherv(send, count, recv, counts, d.dt, comm, *stream, a),
                           ccl::allgatherv(send, count, recv, counts, d.dt, comm, a));
    }
    if (coll == "alltoall") {
        auto a = make_attr<ccl::alltoall_attr>(cache, id);
        return WITH_STREAM(ccl::alltoall(send, recv, count, d.dt, comm, *stream, a),
                           ccl::alltoall(send, recv, count, d.dt, comm, a));
    }
    if (coll == "alltoallv") {
        auto a = make_attr<ccl::alltoallv_attr>(cache, id);
        const ccl::vector_class<size_t> counts(N, count);
        return WITH_STREAM(ccl::alltoallv(send, counts, recv, counts, d.dt, comm, *stream, a),
                           ccl::alltoallv(send, counts, recv, counts, d.dt, comm, a));
    }
    auto a = make_attr<ccl::reduce_scatter_attr>(cache, id);
    return WITH_STREAM(ccl::reduce_scatter(send, recv, count, d.dt, r, comm, *stream, a),
                       ccl::reduce_scatter(send, recv, count, d.dt, r, comm, a));
}

// expected value of element i of the recv buffer
long expected(const std::string& coll, const std::string& red, int rank, int size, int b, size_t count, size_t i) {
    if (coll == "allreduce" || coll == "reduce")
        return reduced(size, b, i, red);
    if (coll == "bcast")
        return fill_value(0, b, i, red);
    if (coll == "allgather" || coll == "allgatherv")
        return fill_value((int)(i / count), b, i % count, red);
    if (coll == "alltoall" || coll == "alltoallv")
        return fill_value((int)(i / count), b, (size_t)rank * count + i % count, red);
    return reduced(size, b, (size_t)rank * count + i, red); // reduce_scatter
}

struct row {
    std::string coll, dtype, red;
    size_t count, bytes;
    int reps;
    double t_min, t_max, t_avg, stddev, wait_avg;
};

} // namespace

int main(int argc, char** argv) {
    if (argc < 4) {
        usage(argv[0]);
        return 2;
    }
    const int rank = std::atoi(argv[1]), size = std::atoi(argv[2]);
    options o;
    const bool legacy = argc > 4 && argv[4][0] != '-';
    if (legacy) { // <coll> <min> <max> <iters> <warmup>, powers of two, fixed iteration count, no check
        o.colls = split(argv[4]);
        const size_t lo = argc > 5 ? std::strtoull(argv[5], nullptr, 10) : 1;
        const size_t hi = argc > 6 ? std::strtoull(argv[6], nullptr, 10) : (1u << 20);
        for (size_t c = std::max<size_t>(lo, 1); c <= hi; c *= 2)
            o.counts.push_back(c);
        o.iters = argc > 7 ? std::atoi(argv[7]) : 16;
        o.warmup = argc > 8 ? std::atoi(argv[8]) : 16;
        o.iter_auto = false;
        o.check = "off";
        o.cache = false;
    }
    else if (!parse(argc, argv, o)) {
        usage(argv[0]);
        return 2;
    }
    const bool cuda = o.backend == "cuda";
#ifdef CCL_BENCH_CUDA
    if (cuda) {
        int ndev = 0;
        cudaGetDeviceCount(&ndev);
        if (ndev < size) { // ranks that wait on one another must not share a GPU
            std::cout << "needs one GPU per rank" << std::endl;
            return 0;
        }
        cudaSetDevice(rank);
        cudaStreamCreate(&g_stream);
    }
#else
    if (cuda) {
        std::cerr << "this binary was built without -DCCL_BENCH_CUDA: only -b host\n";
        return 2;
    }
#endif
    ccl::init();
    auto kvs = bootstrap_kvs(rank, argv[3]);
    auto comm = ccl::create_communicator(size, rank, kvs);
    const ccl::stream* stream = nullptr; // host buffers: the overloads without a stream
#ifdef CCL_BENCH_CUDA
    ccl::stream stream_obj = ccl::create_stream();
    if (cuda) {
        stream_obj = ccl::create_stream((CUstream_st*)g_stream);
        stream = &stream_obj;
    }
#endif
    const bool show_wait = o.ext == "on";
    std::vector<row> rows;
    long failures = 0;
    if (rank == 0)
        std::cout << (legacy ? "#coll,count,bytes,t_min_us,t_max_us,t_avg_us,stddev_pct"
                             : "#coll,dtype,reduction,elem_count,bytes,repetitions,t_min,t_max,t_avg,stddev_pct")
                  << (show_wait && !legacy ? ",wait_t_avg" : "") << std::endl;
    for (const std::string& coll : o.colls) {
        const bool reduces = coll == "allreduce" || coll == "reduce" || coll == "reduce_scatter";
        for (const std::string& dname : o.dtypes) {
            const dtype_info& d = dtype_of(dname);
            for (const std::string& red : reduces ? o.reductions : std::vector<std::string>{ "sum" }) {
                for (size_t count : o.counts) {
                    const sizes sz = elems_of(coll, count, size);
                    const size_t bytes = count * d.size;
                    int reps = o.iters;
                    if (o.iter_auto) // half the repetitions for every doubling above 256 KiB
                        for (size_t n = bytes >> 18; n && reps > 1; n >>= 1)
                            reps = std::max(1, reps / 2);
                    std::vector<buffer> send(o.buf_count), recv(o.buf_count);
                    std::vector<void*> sp(o.buf_count), rp(o.buf_count);
                    for (int b = 0; b < o.buf_count; b++) {
                        allocate(send[b], sz.send_elems * d.size, cuda);
                        allocate(recv[b], sz.recv_elems * d.size, cuda);
                    }
                    auto fill = [&](int b) {
                        // in place: the input sits where the operation defines it, inside the larger buffer
                        buffer& in = send[b];
                        buffer& out = recv[b];
                        sp[b] = in.ptr();
                        rp[b] = out.ptr();
                        for (size_t i = 0; i < sz.send_elems; i++)
                            put(in.host.data(), i, d, fill_value(rank, b, i, red));
                        if (coll == "bcast") // the operation works on the recv buffer alone
                            for (size_t i = 0; i < count; i++)
                                put(out.host.data(), i, d, rank == 0 ? fill_value(0, b, i, red) : 0);
                        if (o.inplace) {
                            if (coll == "allgather" || coll == "allgatherv") {
                                std::memcpy(out.host.data() + (size_t)rank * count * d.size, in.host.data(), count * d.size);
                                sp[b] = (char*)out.ptr() + (size_t)rank * count * d.size;
                            }
                            else if (coll == "reduce_scatter")
                                rp[b] = (char*)in.ptr() + (size_t)rank * count * d.size;
                            else if (coll != "bcast")
                                rp[b] = in.ptr();
                        }
                        to_device(in);
                        to_device(out);
                    };
                    auto verify = [&](int b) {
                        // the bytes the operation wrote, wherever the in-place form put them
                        buffer& holder = (o.inplace && coll != "bcast" && coll != "allgather" && coll != "allgatherv")
                                             ? send[b]
                                             : recv[b];
                        to_host(holder);
                        const char* base = holder.host.data();
                        if (o.inplace && coll == "reduce_scatter")
                            base += (size_t)rank * count * d.size;
                        if (coll == "reduce" && rank != 0)
                            return;
                        for (size_t i = 0; i < sz.recv_elems; i++) {
                            const long want = expected(coll, red, rank, size, b, count, i);
                            const long got = get(base, i, d);
                            if (got != want) {
                                if (failures++ < 5)
                                    std::cout << "CHECK FAILED rank " << rank << ": " << coll << " " << dname << " " << red
                                              << " count " << count << " buffer " << b << " [" << i << "] = " << got
                                              << ", expected " << want << std::endl;
                                return;
                            }
                        }
                    };
                    for (int b = 0; b < o.buf_count; b++)
                        fill(b);
                    std::vector<std::string> ids(o.buf_count); // match_id of the persistent operation per buffer
                    for (int b = 0; b < o.buf_count; b++)
                        ids[b] = coll + "/" + dname + "/" + red + "/" + std::to_string(count) + "/" + std::to_string(b);
                    std::vector<double> total(reps), waited(reps);
                    for (int it = 0; it < o.warmup + reps; it++) {
                        if (o.inplace && it > 0)
                            for (int b = 0; b < o.buf_count; b++)
                                fill(b);
                        ccl::barrier(comm).wait();
                        std::vector<ccl::event> evs;
                        evs.reserve(o.buf_count);
                        const auto t0 = std::chrono::steady_clock::now();
                        for (int b = 0; b < o.buf_count; b++)
                            evs.push_back(start_one(coll, d, red, count, sp[b], rp[b], comm, stream, o.cache, ids[b]));
                        const auto t_call = std::chrono::steady_clock::now();
                        for (auto& e : evs)
                            e.wait();
                        const auto t1 = std::chrono::steady_clock::now();
                        if (it >= o.warmup) {
                            total[it - o.warmup] = std::chrono::duration<double, std::micro>(t1 - t0).count();
                            waited[it - o.warmup] = std::chrono::duration<double, std::micro>(t1 - t_call).count();
                        }
                        const bool last = it == o.warmup + reps - 1;
                        if (count > 0 && (o.check == "all" || (o.check == "last" && last)))
                            for (int b = 0; b < o.buf_count; b++)
                                verify(b);
                    }
                    for (int b = 0; b < o.buf_count; b++) {
                        release(send[b]);
                        release(recv[b]);
                    }
                    // every rank's per-iteration times meet on every rank; rank 0 reports
                    std::vector<double> mine(2 * (size_t)reps), all(2 * (size_t)reps * size);
                    std::copy(total.begin(), total.end(), mine.begin());
                    std::copy(waited.begin(), waited.end(), mine.begin() + reps);
                    ccl::allgather(mine.data(), all.data(), mine.size(), comm).wait();
                    row r{ coll, dname, red, count, bytes, reps, 0, 0, 0, 0, 0 };
                    std::vector<double> per_iter(reps);
                    for (int it = 0; it < reps; it++) {
                        double lo = 1e300, hi = 0, sum = 0, wsum = 0;
                        for (int p = 0; p < size; p++) {
                            const double t = all[(size_t)p * 2 * reps + it];
                            lo = std::min(lo, t);
                            hi = std::max(hi, t);
                            sum += t;
                            wsum += all[(size_t)p * 2 * reps + reps + it];
                        }
                        r.t_min += lo / reps;
                        r.t_max += hi / reps;
                        per_iter[it] = sum / size;
                        r.t_avg += per_iter[it] / reps;
                        r.wait_avg += wsum / size / reps;
                    }
                    double var = 0;
                    for (double t : per_iter)
                        var += (t - r.t_avg) * (t - r.t_avg);
                    r.stddev = r.t_avg > 0 ? 100.0 * std::sqrt(var / reps) / r.t_avg : 0;
                    rows.push_back(r);
                    if (rank == 0) {
                        if (legacy)
                            std::cout << coll << "," << count << "," << bytes << "," << r.t_min << "," << r.t_max << ","
                                      << r.t_avg << "," << r.stddev << std::endl;
                        else {
                            std::cout << coll << "," << dname << "," << red << "," << count << "," << bytes << "," << reps
                                      << "," << r.t_min << "," << r.t_max << "," << r.t_avg << "," << r.stddev;
                            if (show_wait)
                                std::cout << "," << r.wait_avg;
                            std::cout << std::endl;
                        }
                    }
                }
            }
        }
    }
    if (rank == 0 && !o.csv.empty()) {
        std::ofstream f(o.csv);
        f << "#ranks,collective,reduction,dtype,elem_count,bytes,repetitions,t_min,t_max,t_avg,stddev_pct,wait_t_avg\n";
        for (auto& r : rows)
            f << size << "," << r.coll << "," << r.red << "," << r.dtype << "," << r.count << "," << r.bytes << "," << r.reps
              << "," << r.t_min << "," << r.t_max << "," << r.t_avg << "," << r.stddev << "," << r.wait_avg << "\n";
    }
    ccl::barrier(comm).wait();
    if (rank == 0 && o.check != "off")
        std::cout << (failures ? "FAILED" : "PASSED") << std::endl;
    return failures ? 1 : 0;
}
