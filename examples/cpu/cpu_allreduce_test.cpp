// Host-buffer allreduce through the public API, launched as N plain processes:
//   cpu_allreduce_test <rank> <size> <address-file>
// Same flow as the reference's examples/cpu/cpu_allreduce_test.cpp (init, kvs,
// communicator, allreduce, check), with a file instead of MPI_Bcast for the address.
#include <cstdlib>
#include <iostream>
#include <vector>

#include "oneapi/ccl.hpp"
#include "store.hpp"

int main(int argc, char** argv) {
    if (argc < 4) {
        std::cerr << "usage: " << argv[0] << " <rank> <size> <address-file>\n";
        return 2;
    }
    const int rank = std::atoi(argv[1]), size = std::atoi(argv[2]);
    const size_t count = 4096;
    ccl::init();
    auto kvs = bootstrap_kvs(rank, argv[3]);
    auto comm = ccl::create_communicator(size, rank, kvs);

    std::vector<int> send_buf(count, comm.rank() + 1), recv_buf(count, 0);
    ccl::allreduce(send_buf.data(), recv_buf.data(), count, ccl::reduction::sum, comm).wait();
    bool ok = true;
    for (size_t i = 0; i < count; i++)
        ok = ok && recv_buf[i] == size * (size + 1) / 2;

    // operation attributes: cached schedule named by match_id, run twice
    auto attr = ccl::create_operation_attr<ccl::allreduce_attr>();
    attr.set<ccl::operation_attr_id::to_cache>(true);
    attr.set<ccl::operation_attr_id::match_id>(std::string("tensor_a"));
    std::vector<float> a(1000, 1.0f * (rank + 1)), b(1000);
    for (int it = 0; it < 2; it++) {
        ccl::allreduce(a.data(), b.data(), a.size(), ccl::reduction::max, comm, attr).wait();
        ok = ok && b[999] == (float)size;
    }

    // allgatherv with unequal counts and a barrier
    std::vector<size_t> counts(size);
    size_t total = 0;
    for (int p = 0; p < size; p++) {
        counts[p] = 10 + p;
        total += counts[p];
    }
    std::vector<double> mine(counts[rank], rank), all(total, -1);
    ccl::allgatherv(mine.data(), mine.size(), all.data(), counts, comm).wait();
    size_t off = 0;
    for (int p = 0; p < size; p++) {
        for (size_t i = 0; i < counts[p]; i++)
            ok = ok && all[off + i] == p;
        off += counts[p];
    }
    ccl::barrier(comm).wait();

    // custom datatype moved with broadcast
    auto dattr = ccl::create_datatype_attr(ccl::attr_val<ccl::datatype_attr_id::size>((size_t)12));
    ccl::datatype triple = ccl::register_datatype(dattr);
    std::vector<char> blob(12 * 5, (char)(rank == 0 ? 7 : 0));
    ccl::broadcast(blob.data(), 5, triple, 0, comm).wait();
    ok = ok && blob[59] == 7 && ccl::get_datatype_size(triple) == 12;
    ccl::deregister_datatype(triple);

    if (rank == 0)
        std::cout << (ok ? "PASSED" : "FAILED") << std::endl;
    return ok ? 0 : 1;
}
