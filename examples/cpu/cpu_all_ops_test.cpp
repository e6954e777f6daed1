// Every operation of the public API on host buffers, typed overloads, in place and out of place,
// two iterations with re-allocated buffers (the schedule cache must not reuse stale pointers):
//   cpu_all_ops_test <rank> <size> <address-file>
// Plays the role of the reference's functional tests (tests/functional/*_test.cpp, oracle
// test_impl.hpp:241-324: deterministic fill from rank and buffer index, closed-form expected values)
// as one binary that prints PASSED / FAILED per operation.
#include <cmath>
#include <cstdlib>
#include <iostream>
#include <memory>
#include <numeric>
#include <string>
#include <vector>

#include "oneapi/ccl.hpp"
#include "store.hpp"

namespace {
int g_rank = 0, g_size = 1, g_fail = 0;

void report(const std::string& what, bool ok) {
    if (!ok)
        g_fail++;
    if (g_rank == 0 || !ok)
        std::cout << what << ": " << (ok ? "PASSED" : "FAILED") << (ok ? "" : " on rank " + std::to_string(g_rank))
                  << std::endl;
}

template <class T>
T tri(int n) { // 1 + 2 + ... + n
    return (T)(n * (n + 1) / 2);
}
} // namespace

template <class T>
void run_ops(const ccl::communicator& comm, const std::string& tname, int iteration) {
    const int R = g_rank, N = g_size;
    const size_t count = iteration == 0 ? 1033 : 4099; // odd counts, different per iteration
    const std::string tag = tname + "/it" + std::to_string(iteration);
    // fresh allocations every iteration ("dynamic pointer" mode of the reference tests)
    std::unique_ptr<T[]> a(new T[count * N]), b(new T[count * N]);

    // allreduce, out of place then in place
    for (size_t i = 0; i < count; i++)
        a[i] = (T)(R + 1 + (i % 3));
    ccl::allreduce(a.get(), b.get(), count, ccl::reduction::sum, comm).wait();
    bool ok = true;
    for (size_t i = 0; i < count; i++)
        ok = ok && b[i] == (T)(tri<T>(N) + (T)(N * (i % 3)));
    ccl::allreduce(a.get(), a.get(), count, ccl::reduction::max, comm).wait();
    for (size_t i = 0; i < count; i++)
        ok = ok && a[i] == (T)(N + (i % 3));
    report("allreduce " + tag, ok);

    // reduce to the last rank
    for (size_t i = 0; i < count; i++) {
        a[i] = (T)(R + 1);
        b[i] = (T)0;
    }
    ccl::reduce(a.get(), b.get(), count, ccl::reduction::sum, N - 1, comm).wait();
    ok = true;
    if (R == N - 1)
        for (size_t i = 0; i < count; i++)
            ok = ok && b[i] == tri<T>(N);
    report("reduce " + tag, ok);

    // broadcast: in-place form and send/recv form
    for (size_t i = 0; i < count; i++)
        a[i] = (T)(R == 0 ? (i % 7) : 99);
    ccl::broadcast(a.get(), count, 0, comm).wait();
    ok = true;
    for (size_t i = 0; i < count; i++)
        ok = ok && a[i] == (T)(i % 7);
    for (size_t i = 0; i < count; i++)
        b[i] = (T)98;
    ccl::broadcast(a.get(), b.get(), count, N - 1, comm).wait();
    for (size_t i = 0; i < count; i++)
        ok = ok && b[i] == (T)(i % 7);
    report("broadcast " + tag, ok);

    // allgather and allgatherv (one buffer, then one buffer per rank)
    for (size_t i = 0; i < count; i++)
        a[i] = (T)(R * 2 + 1);
    ccl::allgather(a.get(), b.get(), count, comm).wait();
    ok = true;
    for (int p = 0; p < N; p++)
        for (size_t i = 0; i < count; i++)
            ok = ok && b[p * count + i] == (T)(p * 2 + 1);
    std::vector<size_t> counts(N);
    size_t total = 0;
    for (int p = 0; p < N; p++) {
        counts[p] = 5 + 3 * p;
        total += counts[p];
    }
    std::vector<T> mine(counts[R], (T)(R + 10)), all(total, (T)0);
    ccl::allgatherv(mine.data(), mine.size(), all.data(), counts, comm).wait();
    size_t off = 0;
    for (int p = 0; p < N; p++) {
        for (size_t i = 0; i < counts[p]; i++)
            ok = ok && all[off + i] == (T)(p + 10);
        off += counts[p];
    }
    std::vector<std::vector<T>> parts(N);
    std::vector<T*> ptrs(N);
    for (int p = 0; p < N; p++) {
        parts[p].assign(counts[p], (T)0);
        ptrs[p] = parts[p].data();
    }
    ccl::allgatherv(mine.data(), mine.size(), ptrs, counts, comm).wait();
    for (int p = 0; p < N; p++)
        for (size_t i = 0; i < counts[p]; i++)
            ok = ok && parts[p][i] == (T)(p + 10);
    report("allgather(v) " + tag, ok);

    // reduce_scatter
    for (int p = 0; p < N; p++)
        for (size_t i = 0; i < count; i++)
            a[p * count + i] = (T)(R + p + 1);
    ccl::reduce_scatter(a.get(), b.get(), count, ccl::reduction::sum, comm).wait();
    ok = true;
    for (size_t i = 0; i < count; i++)
        ok = ok && b[i] == (T)(tri<T>(N) + (T)(N * R));
    report("reduce_scatter " + tag, ok);

    // alltoall and alltoallv
    for (int p = 0; p < N; p++)
        for (size_t i = 0; i < count; i++)
            a[p * count + i] = (T)(R * 10 + p);
    ccl::alltoall(a.get(), b.get(), count, comm).wait();
    ok = true;
    for (int p = 0; p < N; p++)
        for (size_t i = 0; i < count; i++)
            ok = ok && b[p * count + i] == (T)(p * 10 + R);
    std::vector<size_t> sc(N), rc(N);
    size_t st = 0, rt = 0;
    for (int p = 0; p < N; p++) {
        sc[p] = 1 + (size_t)((R + p) % 4);
        rc[p] = 1 + (size_t)((p + R) % 4);
        st += sc[p];
        rt += rc[p];
    }
    std::vector<T> sv(st), rv(rt, (T)0);
    off = 0;
    for (int p = 0; p < N; p++)
        for (size_t i = 0; i < sc[p]; i++)
            sv[off++] = (T)(R * 10 + p);
    ccl::alltoallv(sv.data(), sc, rv.data(), rc, comm).wait();
    off = 0;
    for (int p = 0; p < N; p++)
        for (size_t i = 0; i < rc[p]; i++)
            ok = ok && rv[off++] == (T)(p * 10 + R);
    report("alltoall(v) " + tag, ok);

    // send / recv around a ring, plain and inside a group
    if (N > 1) {
        const int next = (R + 1) % N, prev = (R + N - 1) % N;
        std::vector<T> out(count, (T)(R + 1)), in(count, (T)0);
        ccl::event es, er;
        if (R % 2 == 0) {
            es = ccl::send(out.data(), count, next, comm);
            er = ccl::recv(in.data(), count, prev, comm);
        }
        else {
            er = ccl::recv(in.data(), count, prev, comm);
            es = ccl::send(out.data(), count, next, comm);
        }
        es.wait();
        er.wait();
        ok = true;
        for (size_t i = 0; i < count; i++)
            ok = ok && in[i] == (T)(prev + 1);
        std::fill(in.begin(), in.end(), (T)0);
        ccl::group_start();
        auto g1 = ccl::send(out.data(), count, prev, comm);
        auto g2 = ccl::recv(in.data(), count, next, comm);
        ccl::group_end();
        g1.wait();
        g2.wait();
        for (size_t i = 0; i < count; i++)
            ok = ok && in[i] == (T)(next + 1);
        report("send/recv " + tag, ok);
    }
    ccl::barrier(comm).wait();
}

int main(int argc, char** argv) {
    if (argc < 4) {
        std::cerr << "usage: " << argv[0] << " <rank> <size> <address-file>\n";
        return 2;
    }
    g_rank = std::atoi(argv[1]);
    g_size = std::atoi(argv[2]);
    ccl::init();
    auto kvs = bootstrap_kvs(g_rank, argv[3]);
    auto comm = ccl::create_communicator(g_size, g_rank, kvs);
    for (int it = 0; it < 2; it++) {
        run_ops<int>(comm, "int32", it);
        run_ops<float>(comm, "float32", it);
        run_ops<double>(comm, "float64", it);
        run_ops<int64_t>(comm, "int64", it);
        run_ops<uint8_t>(comm, "uint8", it);
    }
    // sub-communicator by colour, events tested instead of waited, dependencies
    auto sattr = ccl::create_comm_split_attr(ccl::attr_val<ccl::comm_split_attr_id::color>(g_rank % 2));
    auto half = ccl::split_communicator(comm, sattr);
    std::vector<int> x(100, 1), y(100, 0), z(100, 0);
    auto e1 = ccl::allreduce(x.data(), y.data(), x.size(), ccl::reduction::sum, half);
    while (!e1.test()) {
    }
    bool ok = y[0] == half.size();
    std::vector<ccl::event> deps;
    deps.push_back(ccl::allreduce(x.data(), y.data(), x.size(), ccl::reduction::sum, comm));
    ccl::allreduce(y.data(), z.data(), y.size(), ccl::reduction::sum, comm, ccl::default_allreduce_attr, deps).wait();
    ok = ok && z[99] == g_size * g_size;
    report("split / test / deps", ok);
    std::cout.flush();
    return g_fail ? 1 : 0;
}
