// Times the host-buffer configuration of the baseline through the public C++ API: fp32 sum allreduce at
// 1 / 17 / 4096 / 1048576 elements, allgatherv with counts {1000, 1500, ...}, barrier; ranks are plain
// processes that meet through a key-value store address in a file (no mpirun).  The program uses only
// what the oneCCL specification offers, so the same source builds against this library and against
// the reference: the two columns of profiles/host_path_cpu_allreduce.md come from one binary each.
//
//   cpu_config1_timing <rank> <size> <address file> [iterations]
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <thread>
#include <vector>

#include "oneapi/ccl.hpp"

static std::shared_ptr<ccl::kvs> meet(int rank, const std::string& path) {
    if (rank == 0) {
        auto kvs = ccl::create_main_kvs();
        auto addr = kvs->get_address();
        std::string tmp = path + ".tmp";
        {
            std::ofstream f(tmp, std::ios::binary);
            f.write((const char*)addr.data(), addr.size());
        }
        std::rename(tmp.c_str(), path.c_str());
        return kvs;
    }
    ccl::kvs::address_type addr;
    for (int tries = 0;; tries++) {
        std::ifstream f(path, std::ios::binary);
        if (f && f.read((char*)addr.data(), addr.size()))
            break;
        if (tries > 6000) {
            std::fprintf(stderr, "address file never appeared\n");
            std::exit(2);
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(10));
    }
    return ccl::create_kvs(addr);
}

template <class F>
static void timed(const char* what, size_t count, int iters, const ccl::communicator& comm, F&& op) {
    for (int i = 0; i < std::max(4, iters / 4); i++)
        op();
    ccl::barrier(comm);
    std::vector<double> us(iters);
    for (int i = 0; i < iters; i++) {
        auto t0 = std::chrono::steady_clock::now();
        op();
        us[i] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    }
    std::sort(us.begin(), us.end());
    double sum = 0;
    for (double v : us)
        sum += v;
    if (comm.rank() == 0)
        std::printf("%-12s count %8zu  t_min %10.1f us  t_med %10.1f us  t_avg %10.1f us\n", what, count, us[0],
                    us[iters / 2], sum / iters);
}

int main(int argc, char** argv) {
    if (argc < 4) {
        std::fprintf(stderr, "usage: %s <rank> <size> <address file> [iterations]\n", argv[0]);
        return 2;
    }
    const int rank = std::atoi(argv[1]), size = std::atoi(argv[2]);
    const int iters = argc > 4 ? std::atoi(argv[4]) : 64;
    ccl::init();
    auto kvs = meet(rank, argv[3]);
    auto comm = ccl::create_communicator(size, rank, kvs);
    bool ok = true;
    for (size_t count : { (size_t)1, (size_t)17, (size_t)4096, (size_t)1048576 }) {
        std::vector<float> send(count), recv(count);
        for (size_t i = 0; i < count; i++)
            send[i] = (float)((i % 13) + rank);
        timed("allreduce", count, count > 100000 ? std::max(8, iters / 4) : iters, comm, [&] {
            ccl::allreduce(send.data(), recv.data(), count, ccl::reduction::sum, comm).wait();
        });
        for (size_t i = 0; i < count; i += std::max<size_t>(1, count / 97)) {
            const float ref = (float)((i % 13) * size + size * (size - 1) / 2);
            ok = ok && std::fabs(recv[i] - ref) < 1e-3f;
        }
    }
    std::vector<size_t> counts(size);
    size_t total = 0;
    for (int p = 0; p < size; p++) {
        counts[p] = p == 0 ? 1000 : (p == 1 ? 1500 : 700);
        total += counts[p];
    }
    std::vector<float> mine(counts[rank], (float)(rank + 1)), all(total);
    timed("allgatherv", total, iters, comm,
          [&] { ccl::allgatherv(mine.data(), counts[rank], all.data(), counts, comm).wait(); });
    size_t off = 0;
    for (int p = 0; p < size; p++) {
        ok = ok && all[off] == (float)(p + 1) && all[off + counts[p] - 1] == (float)(p + 1);
        off += counts[p];
    }
    timed("barrier", 0, iters, comm, [&] { ccl::barrier(comm); });
    if (rank == 0)
        std::printf(ok ? "PASSED\n" : "FAILED\n");
    return ok ? 0 : 1;
}
