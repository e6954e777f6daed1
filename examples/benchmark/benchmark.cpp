// Collective benchmark on host buffers through the public API (the reference ships an
// equivalent tool, examples/benchmark/src/benchmark.cpp:47-222: warm-up + timed
// iterations per message size, t_min / t_max / t_avg / stddev in microseconds).
//   benchmark <rank> <size> <address-file> [coll=allreduce] [min_count=1] [max_count=1048576] [iters=16] [warmup=16]
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <numeric>
#include <string>
#include <vector>

#include "oneapi/ccl.hpp"
#include "store.hpp"

int main(int argc, char** argv) {
    if (argc < 4) {
        std::cerr << "usage: " << argv[0] << " <rank> <size> <address-file> [coll] [min] [max] [iters] [warmup]\n";
        return 2;
    }
    const int rank = std::atoi(argv[1]), size = std::atoi(argv[2]);
    const std::string coll = argc > 4 ? argv[4] : "allreduce";
    const size_t min_count = argc > 5 ? std::strtoull(argv[5], nullptr, 10) : 1;
    const size_t max_count = argc > 6 ? std::strtoull(argv[6], nullptr, 10) : (1u << 20);
    const int iters = argc > 7 ? std::atoi(argv[7]) : 16;
    const int warmup = argc > 8 ? std::atoi(argv[8]) : 16;
    ccl::init();
    auto kvs = bootstrap_kvs(rank, argv[3]);
    auto comm = ccl::create_communicator(size, rank, kvs);
    if (rank == 0)
        std::cout << "#coll,count,bytes,t_min_us,t_max_us,t_avg_us,stddev_pct\n";
    for (size_t count = min_count; count <= max_count; count *= 2) {
        std::vector<float> send(count * size, 1.0f), recv(count * size, 0.0f);
        std::vector<double> samples;
        for (int it = 0; it < warmup + iters; it++) {
            ccl::barrier(comm).wait();
            auto t0 = std::chrono::steady_clock::now();
            if (coll == "allreduce")
                ccl::allreduce(send.data(), recv.data(), count, ccl::reduction::sum, comm).wait();
            else if (coll == "allgather")
                ccl::allgather(send.data(), recv.data(), count, comm).wait();
            else if (coll == "alltoall")
                ccl::alltoall(send.data(), recv.data(), count, comm).wait();
            else if (coll == "bcast")
                ccl::broadcast(send.data(), count, 0, comm).wait();
            else if (coll == "reduce")
                ccl::reduce(send.data(), recv.data(), count, ccl::reduction::sum, 0, comm).wait();
            else if (coll == "reduce_scatter")
                ccl::reduce_scatter(send.data(), recv.data(), count, ccl::reduction::sum, comm).wait();
            else {
                std::cerr << "unknown collective " << coll << "\n";
                return 2;
            }
            auto t1 = std::chrono::steady_clock::now();
            if (it >= warmup)
                samples.push_back(std::chrono::duration<double, std::micro>(t1 - t0).count());
        }
        double mn = *std::min_element(samples.begin(), samples.end());
        double mx = *std::max_element(samples.begin(), samples.end());
        double avg = std::accumulate(samples.begin(), samples.end(), 0.0) / samples.size();
        double var = 0;
        for (double s : samples)
            var += (s - avg) * (s - avg);
        double sd = std::sqrt(var / samples.size());
        if (rank == 0)
            std::cout << coll << "," << count << "," << count * sizeof(float) << "," << mn << "," << mx << "," << avg
                      << "," << (avg > 0 ? 100.0 * sd / avg : 0) << "\n";
    }
    return 0;
}
