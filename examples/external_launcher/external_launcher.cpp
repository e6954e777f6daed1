// Launch without mpirun or any process manager: every process is started by hand (or by a job
// scheduler) with its rank, the world size and a place to find the KVS address.
//   external_launcher <size> <rank> <address-file> [repeats]
// The communicator is created and destroyed `repeats` times (default 10) over fresh key-value
// stores, as a long-running service re-forming its group would do.  Same scenario as the
// reference's examples/external_launcher/external_launcher.cpp:23-27 (which re-initialises ten
// times) with its file store (examples/include/store.hpp); local rank / size come from
// CCL_LOCAL_RANK / CCL_LOCAL_SIZE with CCL_PROCESS_LAUNCHER=none, as its run_binary.sh sets them.
#include <cstdlib>
#include <iostream>
#include <numeric>
#include <vector>

#include "oneapi/ccl.hpp"
#include "store.hpp"

int main(int argc, char** argv) {
    if (argc < 4) {
        std::cerr << "usage: " << argv[0] << " <size> <rank> <address-file> [repeats]\n";
        return 2;
    }
    const int size = std::atoi(argv[1]), rank = std::atoi(argv[2]);
    const std::string path = argv[3];
    const int repeats = argc > 4 ? std::atoi(argv[4]) : 10;
    ccl::init();
    bool ok = true;
    for (int it = 0; it < repeats; it++) {
        // one address file per incarnation: nobody can pick up the previous store
        auto kvs = bootstrap_kvs(rank, path + "." + std::to_string(it));
        auto comm = ccl::create_communicator(size, rank, kvs);
        std::vector<float> send(1 << 12), recv(send.size(), 0.f);
        std::iota(send.begin(), send.end(), (float)(rank + it));
        ccl::allreduce(send.data(), recv.data(), send.size(), ccl::reduction::sum, comm).wait();
        for (size_t i = 0; i < send.size(); i++) {
            const float want = (float)size * (float)(i + it) + (float)size * (float)(size - 1) / 2.f;
            ok = ok && recv[i] == want;
        }
        std::vector<int> all(size, -1);
        int mine = rank * 10 + it;
        ccl::allgather(&mine, all.data(), 1, comm).wait();
        for (int p = 0; p < size; p++)
            ok = ok && all[p] == p * 10 + it;
        ccl::barrier(comm).wait();
    }
    if (rank == 0)
        std::cout << (ok ? "PASSED" : "FAILED") << " after " << repeats << " communicator incarnations" << std::endl;
    return ok ? 0 : 1;
}
