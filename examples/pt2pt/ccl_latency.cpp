// Point-to-point latency between rank 0 and rank 1 (host buffers):
//   ccl_latency <rank> <size> <address-file> [min_bytes] [max_bytes] [iters]
// Ping-pong: rank 0 sends, rank 1 answers; the reported time is half the round trip, in
// microseconds, per message size (powers of two).  Same measurement as the reference's
// examples/pt2pt/src/ccl_latency.cpp (doc/rst/source/benchmark-guide/benchmark-point-to-point.rst:76-77).
#include <chrono>
#include <cstdlib>
#include <iostream>
#include <vector>

#include "oneapi/ccl.hpp"
#include "store.hpp"

int main(int argc, char** argv) {
    if (argc < 4) {
        std::cerr << "usage: " << argv[0] << " <rank> <size> <address-file> [min_bytes] [max_bytes] [iters]\n";
        return 2;
    }
    const int rank = std::atoi(argv[1]), size = std::atoi(argv[2]);
    const size_t lo = argc > 4 ? std::strtoull(argv[4], nullptr, 10) : 1;
    const size_t hi = argc > 5 ? std::strtoull(argv[5], nullptr, 10) : (1u << 20);
    const int iters = argc > 6 ? std::atoi(argv[6]) : 200;
    ccl::init();
    auto kvs = bootstrap_kvs(rank, argv[3]);
    auto comm = ccl::create_communicator(size, rank, kvs);
    if (size < 2) {
        std::cerr << "needs two ranks\n";
        return 2;
    }
    std::vector<char> buf(hi, (char)rank);
    if (rank == 0)
        std::cout << "#bytes,latency_usec" << std::endl;
    for (size_t n = lo ? lo : 1; n <= hi; n *= 2) {
        const int warm = iters / 10 + 1;
        std::chrono::steady_clock::time_point t0;
        for (int it = 0; it < warm + iters; it++) {
            if (it == warm)
                t0 = std::chrono::steady_clock::now();
            if (rank == 0) {
                ccl::send(buf.data(), n, ccl::datatype::int8, 1, comm).wait();
                ccl::recv(buf.data(), n, ccl::datatype::int8, 1, comm).wait();
            }
            else if (rank == 1) {
                ccl::recv(buf.data(), n, ccl::datatype::int8, 0, comm).wait();
                ccl::send(buf.data(), n, ccl::datatype::int8, 0, comm).wait();
            }
        }
        const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
        if (rank == 0)
            std::cout << n << "," << us / iters / 2.0 << std::endl;
    }
    ccl::barrier(comm).wait();
    if (rank == 0)
        std::cout << "PASSED" << std::endl;
    return 0;
}
