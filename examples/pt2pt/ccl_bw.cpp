// Point-to-point bandwidth from rank 0 to rank 1 (host buffers):
//   ccl_bw <rank> <size> <address-file> [min_bytes] [max_bytes] [iters] [window]
// Rank 0 posts `window` sends inside one group, rank 1 the matching receives, then a one-byte
// acknowledgement travels back; MB/s = window * bytes / time.  Same measurement as the reference's
// examples/pt2pt/src/ccl_bw.cpp (doc/rst/source/benchmark-guide/benchmark-point-to-point.rst:76-77).
#include <chrono>
#include <cstdlib>
#include <iostream>
#include <vector>

#include "oneapi/ccl.hpp"
#include "store.hpp"

int main(int argc, char** argv) {
    if (argc < 4) {
        std::cerr << "usage: " << argv[0] << " <rank> <size> <address-file> [min_bytes] [max_bytes] [iters] [window]\n";
        return 2;
    }
    const int rank = std::atoi(argv[1]), size = std::atoi(argv[2]);
    const size_t lo = argc > 4 ? std::strtoull(argv[4], nullptr, 10) : 1024;
    const size_t hi = argc > 5 ? std::strtoull(argv[5], nullptr, 10) : (4u << 20);
    const int iters = argc > 6 ? std::atoi(argv[6]) : 20;
    const int window = argc > 7 ? std::atoi(argv[7]) : 8;
    ccl::init();
    auto kvs = bootstrap_kvs(rank, argv[3]);
    auto comm = ccl::create_communicator(size, rank, kvs);
    if (size < 2) {
        std::cerr << "needs two ranks\n";
        return 2;
    }
    std::vector<std::vector<char>> bufs(window, std::vector<char>(hi, (char)(rank + 1)));
    char ack = 0;
    bool ok = true;
    if (rank == 0)
        std::cout << "#bytes,bandwidth_MBps" << std::endl;
    for (size_t n = lo ? lo : 1; n <= hi; n *= 2) {
        std::chrono::steady_clock::time_point t0;
        for (int it = 0; it < iters + 2; it++) {
            if (it == 2)
                t0 = std::chrono::steady_clock::now();
            std::vector<ccl::event> evs;
            if (rank < 2) {
                ccl::group_start();
                for (int w = 0; w < window; w++)
                    evs.push_back(rank == 0 ? ccl::send(bufs[w].data(), n, ccl::datatype::int8, 1, comm)
                                            : ccl::recv(bufs[w].data(), n, ccl::datatype::int8, 0, comm));
                ccl::group_end();
                for (auto& e : evs)
                    e.wait();
                if (rank == 0)
                    ccl::recv(&ack, 1, ccl::datatype::int8, 1, comm).wait();
                else
                    ccl::send(&ack, 1, ccl::datatype::int8, 0, comm).wait();
            }
        }
        const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (rank == 1)
            for (int w = 0; w < window; w++)
                ok = ok && bufs[w][0] == 1 && bufs[w][n - 1] == 1;
        if (rank == 0)
            std::cout << n << "," << (double)window * (double)n * iters / s / 1e6 << std::endl;
    }
    ccl::barrier(comm).wait();
    if (rank == 0)
        std::cout << "PASSED" << std::endl;
    return ok ? 0 : 1;
}
