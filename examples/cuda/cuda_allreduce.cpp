// Device-buffer allreduce through the public API: one process per GPU,
//   cuda_allreduce <rank> <size> <address-file>
// Counterpart of the reference's examples/sycl/sycl_allreduce_usm_test.cpp with a CUDA stream
// in place of the SYCL queue: the stream passed to ccl::create_stream selects the device path.
#include <cuda_runtime.h>

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
    int ndev = 0;
    cudaGetDeviceCount(&ndev);
    if (ndev == 0) {
        std::cout << "no CUDA device" << std::endl;
        return 0;
    }
    cudaSetDevice(rank % ndev);
    const size_t count = 1 << 20;
    ccl::init();
    auto kvs = bootstrap_kvs(rank, argv[3]);
    auto comm = ccl::create_communicator(size, rank, kvs);
    cudaStream_t st;
    cudaStreamCreate(&st);
    auto stream = ccl::create_stream((CUstream_st*)st);
    float* buf = nullptr;
    cudaMalloc(&buf, count * sizeof(float));
    std::vector<float> host(count, (float)(rank + 1));
    cudaMemcpyAsync(buf, host.data(), count * sizeof(float), cudaMemcpyHostToDevice, st);
    auto attr = ccl::create_operation_attr<ccl::allreduce_attr>();
    attr.set<ccl::device_attr_ext_id::scale>(1.0f / size); // fused 1/world scale
    ccl::allreduce(buf, buf, count, ccl::reduction::sum, comm, stream, attr).wait();
    cudaMemcpy(host.data(), buf, count * sizeof(float), cudaMemcpyDeviceToHost);
    const float expect = (size + 1) / 2.0f;
    bool ok = true;
    for (size_t i = 0; i < count; i += 4097)
        ok = ok && std::abs(host[i] - expect) < 1e-5f;
    ccl::barrier(comm).wait();
    if (rank == 0)
        std::cout << (ok ? "PASSED" : "FAILED") << std::endl;
    cudaFree(buf);
    return ok ? 0 : 1;
}
