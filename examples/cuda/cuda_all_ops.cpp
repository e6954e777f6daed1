// Every operation of the public API on device buffers, one process per GPU:
//   cuda_all_ops <rank> <size> <address-file>
// Counterpart of the reference's examples/sycl/sycl_*_usm_test.cpp family (allgather, allgatherv, allreduce,
// alltoall, alltoallv, broadcast, reduce, reduce_scatter, each in place and out of place) as one binary, with a
// CUDA stream where the reference passes a SYCL queue.  Prints PASSED / FAILED per operation; float32 and
// bfloat16 (as raw 16-bit patterns, exact for the small integers used).
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <string>
#include <vector>

#include "oneapi/ccl.hpp"
#include "store.hpp"

namespace {
int g_rank = 0, g_size = 1, g_fail = 0;
cudaStream_t g_st;

void report(const std::string& what, bool ok) {
    if (!ok)
        g_fail++;
    if (g_rank == 0 || !ok)
        std::cout << what << ": " << (ok ? "PASSED" : "FAILED") << (ok ? "" : " on rank " + std::to_string(g_rank))
                  << std::endl;
}

// element codec: float or bfloat16 bit pattern
template <class T>
T enc(float v);
template <>
float enc<float>(float v) {
    return v;
}
template <>
uint16_t enc<uint16_t>(float v) {
    uint32_t x;
    std::memcpy(&x, &v, 4);
    return (uint16_t)(x >> 16); // exact for integers below 256
}
template <class T>
float dec(T v);
template <>
float dec<float>(float v) {
    return v;
}
template <>
float dec<uint16_t>(uint16_t v) {
    const uint32_t x = (uint32_t)v << 16;
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

// a device buffer with a host mirror
template <class T>
struct dbuf {
    std::vector<T> host;
    T* dev = nullptr;
    explicit dbuf(size_t n) : host(n) { cudaMalloc(&dev, n * sizeof(T)); }
    ~dbuf() { cudaFree(dev); }
    void up() { cudaMemcpyAsync(dev, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice, g_st); }
    void down() {
        cudaMemcpyAsync(host.data(), dev, host.size() * sizeof(T), cudaMemcpyDeviceToHost, g_st);
        cudaStreamSynchronize(g_st);
    }
    void fill(float v) {
        for (auto& x : host)
            x = enc<T>(v);
    }
};

template <class T>
void run_ops(const ccl::communicator& comm, const ccl::stream& stream, ccl::datatype dt, const std::string& tname) {
    const int R = g_rank, N = g_size;
    const size_t count = 4099; // odd on purpose
    const float tri = (float)(N * (N + 1) / 2);

    { // allreduce: out of place, in place, fused 1/size scale
        dbuf<T> a(count), b(count);
        for (size_t i = 0; i < count; i++)
            a.host[i] = enc<T>((float)(R + 1 + (i % 3)));
        b.fill(0);
        a.up();
        b.up();
        ccl::allreduce(a.dev, b.dev, count, dt, ccl::reduction::sum, comm, stream).wait();
        b.down();
        bool ok = true;
        for (size_t i = 0; i < count; i++)
            ok = ok && dec<T>(b.host[i]) == tri + (float)(N * (i % 3));
        ccl::allreduce(a.dev, a.dev, count, dt, ccl::reduction::max, comm, stream).wait();
        a.down();
        for (size_t i = 0; i < count; i++)
            ok = ok && dec<T>(a.host[i]) == (float)(N + (i % 3));
        a.fill((float)(2 * N));
        a.up();
        auto attr = ccl::create_operation_attr<ccl::allreduce_attr>();
        attr.template set<ccl::device_attr_ext_id::scale>(1.0f / (float)N);
        ccl::allreduce(a.dev, a.dev, count, dt, ccl::reduction::sum, comm, stream, attr).wait();
        a.down();
        for (size_t i = 0; i < count; i++)
            ok = ok && dec<T>(a.host[i]) == (float)(2 * N);
        report("allreduce " + tname, ok);
    }
    { // reduce to the last rank
        dbuf<T> a(count), b(count);
        a.fill((float)(R + 1));
        b.fill(0);
        a.up();
        b.up();
        ccl::reduce(a.dev, b.dev, count, dt, ccl::reduction::sum, N - 1, comm, stream).wait();
        b.down();
        bool ok = true;
        if (R == N - 1)
            for (size_t i = 0; i < count; i++)
                ok = ok && dec<T>(b.host[i]) == tri;
        report("reduce " + tname, ok);
    }
    { // broadcast: in-place form from rank 0, send / recv form from the last rank
        dbuf<T> a(count), b(count);
        for (size_t i = 0; i < count; i++)
            a.host[i] = enc<T>(R == 0 ? (float)(i % 7) : 99.0f);
        a.up();
        ccl::broadcast(a.dev, count, dt, 0, comm, stream).wait();
        a.down();
        bool ok = true;
        for (size_t i = 0; i < count; i++)
            ok = ok && dec<T>(a.host[i]) == (float)(i % 7);
        b.fill(98);
        b.up();
        ccl::broadcast(a.dev, b.dev, count, dt, N - 1, comm, stream).wait();
        b.down();
        for (size_t i = 0; i < count; i++)
            ok = ok && dec<T>(b.host[i]) == (float)(i % 7);
        report("broadcast " + tname, ok);
    }
    { // allgather out of place and in place; allgatherv with unequal counts
        dbuf<T> a(count), b(count * N);
        a.fill((float)(R * 2 + 1));
        b.fill(0);
        a.up();
        b.up();
        ccl::allgather(a.dev, b.dev, count, dt, comm, stream).wait();
        b.down();
        bool ok = true;
        for (int p = 0; p < N; p++)
            for (size_t i = 0; i < count; i++)
                ok = ok && dec<T>(b.host[p * count + i]) == (float)(p * 2 + 1);
        b.fill(0);
        for (size_t i = 0; i < count; i++)
            b.host[R * count + i] = enc<T>((float)(R + 5));
        b.up();
        ccl::allgather(b.dev + R * count, b.dev, count, dt, comm, stream).wait(); // own block already in place
        b.down();
        for (int p = 0; p < N; p++)
            for (size_t i = 0; i < count; i++)
                ok = ok && dec<T>(b.host[p * count + i]) == (float)(p + 5);
        std::vector<size_t> counts(N);
        size_t total = 0;
        for (int p = 0; p < N; p++) {
            counts[p] = 5 + 3 * (size_t)p;
            total += counts[p];
        }
        dbuf<T> mine(counts[R]), all(total);
        mine.fill((float)(R + 10));
        all.fill(0);
        mine.up();
        all.up();
        ccl::allgatherv(mine.dev, counts[R], all.dev, counts, dt, comm, stream).wait();
        all.down();
        size_t off = 0;
        for (int p = 0; p < N; p++) {
            for (size_t i = 0; i < counts[p]; i++)
                ok = ok && dec<T>(all.host[off + i]) == (float)(p + 10);
            off += counts[p];
        }
        report("allgather(v) " + tname, ok);
    }
    { // reduce_scatter out of place and in place (recv = send + rank * recv_count)
        dbuf<T> a(count * N), b(count);
        for (int p = 0; p < N; p++)
            for (size_t i = 0; i < count; i++)
                a.host[p * count + i] = enc<T>((float)(R + p + 1));
        b.fill(0);
        a.up();
        b.up();
        ccl::reduce_scatter(a.dev, b.dev, count, dt, ccl::reduction::sum, comm, stream).wait();
        b.down();
        bool ok = true;
        for (size_t i = 0; i < count; i++)
            ok = ok && dec<T>(b.host[i]) == tri + (float)(N * R);
        ccl::reduce_scatter(a.dev, a.dev + R * count, count, dt, ccl::reduction::sum, comm, stream).wait();
        a.down();
        for (size_t i = 0; i < count; i++)
            ok = ok && dec<T>(a.host[R * count + i]) == tri + (float)(N * R);
        report("reduce_scatter " + tname, ok);
    }
    { // alltoall and alltoallv
        dbuf<T> a(count * N), b(count * N);
        for (int p = 0; p < N; p++)
            for (size_t i = 0; i < count; i++)
                a.host[p * count + i] = enc<T>((float)(R * 10 + p));
        b.fill(0);
        a.up();
        b.up();
        ccl::alltoall(a.dev, b.dev, count, dt, comm, stream).wait();
        b.down();
        bool ok = true;
        for (int p = 0; p < N; p++)
            for (size_t i = 0; i < count; i++)
                ok = ok && dec<T>(b.host[p * count + i]) == (float)(p * 10 + R);
        std::vector<size_t> sc(N), rc(N);
        size_t st = 0, rt = 0;
        for (int p = 0; p < N; p++) {
            sc[p] = 1 + (size_t)((R + p) % 4) * 100;
            rc[p] = 1 + (size_t)((p + R) % 4) * 100;
            st += sc[p];
            rt += rc[p];
        }
        dbuf<T> sv(st), rv(rt);
        size_t off = 0;
        for (int p = 0; p < N; p++)
            for (size_t i = 0; i < sc[p]; i++)
                sv.host[off++] = enc<T>((float)(R * 10 + p));
        rv.fill(0);
        sv.up();
        rv.up();
        ccl::alltoallv(sv.dev, sc, rv.dev, rc, dt, comm, stream).wait();
        rv.down();
        off = 0;
        for (int p = 0; p < N; p++)
            for (size_t i = 0; i < rc[p]; i++)
                ok = ok && dec<T>(rv.host[off++]) == (float)(p * 10 + R);
        report("alltoall(v) " + tname, ok);
    }
    if (N > 1) { // send / recv around a ring inside a group
        const int next = (R + 1) % N, prev = (R + N - 1) % N;
        dbuf<T> out(count), in(count);
        out.fill((float)(R + 1));
        in.fill(0);
        out.up();
        in.up();
        ccl::group_start();
        auto e1 = ccl::send(out.dev, count, dt, next, comm, stream);
        auto e2 = ccl::recv(in.dev, count, dt, prev, comm, stream);
        ccl::group_end();
        e1.wait();
        e2.wait();
        in.down();
        bool ok = true;
        for (size_t i = 0; i < count; i++)
            ok = ok && dec<T>(in.host[i]) == (float)(prev + 1);
        report("send/recv " + tname, ok);
    }
    ccl::barrier(comm, stream).wait();
}
} // namespace

int main(int argc, char** argv) {
    if (argc < 4) {
        std::cerr << "usage: " << argv[0] << " <rank> <size> <address-file>\n";
        return 2;
    }
    g_rank = std::atoi(argv[1]);
    g_size = std::atoi(argv[2]);
    int ndev = 0;
    cudaGetDeviceCount(&ndev);
    if (ndev == 0) {
        std::cout << "no CUDA device" << std::endl;
        return 0;
    }
    if (g_size > ndev) {
        // ranks that wait on one another must not share a GPU
        std::cout << "needs one GPU per rank" << std::endl;
        return 0;
    }
    cudaSetDevice(g_rank);
    cudaStreamCreate(&g_st);
    ccl::init();
    auto kvs = bootstrap_kvs(g_rank, argv[3]);
    auto comm = ccl::create_communicator(g_size, g_rank, kvs);
    auto stream = ccl::create_stream((CUstream_st*)g_st);
    run_ops<float>(comm, stream, ccl::datatype::float32, "float32");
    run_ops<uint16_t>(comm, stream, ccl::datatype::bfloat16, "bfloat16");
    std::cout.flush();
    return g_fail ? 1 : 0;
}
