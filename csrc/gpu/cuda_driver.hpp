// Runtime-resolved CUDA driver entry points.
//
// The library links the static CUDA runtime only, so that it loads on hosts
// without a driver (CPU-only ranks, build checks).  Driver functions needed
// for virtual memory, shareable handles, NVLS multicast and tensor maps are
// looked up through cudaGetDriverEntryPoint on first use.  This is the CUDA
// counterpart of the reference's dlopen'd Level Zero table
// (src/common/api_wrapper/ze_api_wrapper.hpp).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <string>

#include "core/log.hpp"

namespace cclx {
namespace gpu {

struct driver_api {
    decltype(&cuGetErrorString) GetErrorString = nullptr;
    decltype(&cuDeviceGet) DeviceGet = nullptr;
    decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
    decltype(&cuCtxGetCurrent) CtxGetCurrent = nullptr;
    decltype(&cuMemGetAddressRange) MemGetAddressRange = nullptr;
    decltype(&cuPointerGetAttributes) PointerGetAttributes = nullptr;
    decltype(&cuMemCreate) MemCreate = nullptr;
    decltype(&cuMemRelease) MemRelease = nullptr;
    decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
    decltype(&cuMemAddressFree) MemAddressFree = nullptr;
    decltype(&cuMemMap) MemMap = nullptr;
    decltype(&cuMemUnmap) MemUnmap = nullptr;
    decltype(&cuMemSetAccess) MemSetAccess = nullptr;
    decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
    decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
    decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
    decltype(&cuMulticastCreate) MulticastCreate = nullptr;
    decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
    decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
    decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
    decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
    decltype(&cuTensorMapEncodeTiled) TensorMapEncodeTiled = nullptr;
    bool loaded = false;
    std::string error;
};

// Loads the table once; returns a table with loaded == false (and `error` set)
// when no driver is present.
const driver_api& driver();

std::string cu_error_string(CUresult r);

} // namespace gpu
} // namespace cclx

#define CUDA_CHECK(expr) \
    do { \
        cudaError_t _e = (expr); \
        if (_e != cudaSuccess) \
            CCL_THROW("CUDA error ", cudaGetErrorName(_e), " (", cudaGetErrorString(_e), ") at ", #expr); \
    } while (0)

#define CU_CHECK(expr) \
    do { \
        CUresult _r = (expr); \
        if (_r != CUDA_SUCCESS) \
            CCL_THROW("CUDA driver error ", ::cclx::gpu::cu_error_string(_r), " at ", #expr); \
    } while (0)
