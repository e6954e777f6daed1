// C binding over the public C++ API of an installed oneCCL, used only by `bench.py --impl reference`.
//
// The reference library has no CUDA path and no Python binding, so the benchmark's reference arm keeps
// the model on the GPU with stock PyTorch and hands the gradients to the reference the only way it can
// take them on this hardware: as host buffers, through ccl::allreduce on a communicator created from the
// library's own key-value store.  Nothing of this repository's runtime is linked here; the file
// compiles against <prefix>/include and links <prefix>/lib/libccl.so of the reference installation.
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>

#include "oneapi/ccl.hpp"

namespace {
ccl::shared_ptr_class<ccl::kvs> g_kvs;
std::unique_ptr<ccl::communicator> g_comm;
std::string g_err;

template <class F>
int guard(F&& f) {
    try {
        f();
        return 0;
    }
    catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}
} // namespace

extern "C" {

const char* refshim_last_error() {
    return g_err.c_str();
}

// rank 0: start the key-value store server and return its 256-byte address
int refshim_main_kvs(unsigned char* addr_out) {
    return guard([&] {
        ccl::init();
        g_kvs = ccl::create_main_kvs();
        ccl::kvs::address_type a = g_kvs->get_address();
        std::memcpy(addr_out, a.data(), a.size());
    });
}

int refshim_addr_size() {
    return (int)ccl::kvs::address_type().size();
}

// every rank: connect to the store (rank 0 passes the address it produced) and create the communicator
int refshim_init(int size, int rank, const unsigned char* addr) {
    return guard([&] {
        ccl::init();
        if (!g_kvs) {
            ccl::kvs::address_type a;
            std::memcpy(a.data(), addr, a.size());
            g_kvs = ccl::create_kvs(a);
        }
        g_comm.reset(new ccl::communicator(ccl::create_communicator(size, rank, g_kvs)));
    });
}

// in-place sum over all ranks of a host buffer; dtype 0 = float32, 1 = bfloat16
int refshim_allreduce(void* buf, size_t count, int dtype) {
    return guard([&] {
        ccl::allreduce(buf, buf, count, dtype == 1 ? ccl::datatype::bfloat16 : ccl::datatype::float32,
                       ccl::reduction::sum, *g_comm)
            .wait();
    });
}

int refshim_barrier() {
    return guard([&] { ccl::barrier(*g_comm); });
}

void refshim_finalize() {
    g_comm.reset();
    g_kvs.reset();
}
}
