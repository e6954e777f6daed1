#include "gpu/cuda_driver.hpp"

#include <mutex>

namespace cclx {
namespace gpu {

namespace {

template <class F>
bool load_one(const char* name, F& fn, std::string& err) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
        (void)cudaGetLastError();
        err += std::string(name) + " ";
        return false;
    }
    fn = reinterpret_cast<F>(p);
    return true;
}

driver_api table;
std::once_flag once;

} // namespace

const driver_api& driver() {
    std::call_once(once, [] {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
            (void)cudaGetLastError();
            table.error = "no CUDA device / driver";
            return;
        }
        bool ok = true;
        std::string miss;
#define LOAD(sym) ok = load_one("cu" #sym, table.sym, miss) && ok
        LOAD(GetErrorString);
        LOAD(DeviceGet);
        LOAD(DeviceGetAttribute);
        LOAD(CtxGetCurrent);
        LOAD(MemGetAddressRange);
        LOAD(PointerGetAttributes);
        LOAD(MemCreate);
        LOAD(MemRelease);
        LOAD(MemAddressReserve);
        LOAD(MemAddressFree);
        LOAD(MemMap);
        LOAD(MemUnmap);
        LOAD(MemSetAccess);
        LOAD(MemGetAllocationGranularity);
        LOAD(MemExportToShareableHandle);
        LOAD(MemImportFromShareableHandle);
        LOAD(TensorMapEncodeTiled);
#undef LOAD
        // multicast entry points are optional (absent on old drivers)
        std::string opt;
        load_one("cuMulticastCreate", table.MulticastCreate, opt);
        load_one("cuMulticastAddDevice", table.MulticastAddDevice, opt);
        load_one("cuMulticastBindMem", table.MulticastBindMem, opt);
        load_one("cuMulticastUnbind", table.MulticastUnbind, opt);
        load_one("cuMulticastGetGranularity", table.MulticastGetGranularity, opt);
        table.loaded = ok;
        if (!ok)
            table.error = "missing driver symbols: " + miss;
    });
    return table;
}

std::string cu_error_string(CUresult r) {
    const char* s = nullptr;
    if (table.GetErrorString && table.GetErrorString(r, &s) == CUDA_SUCCESS && s)
        return std::string(s) + " (" + std::to_string((int)r) + ")";
    return "CUresult " + std::to_string((int)r);
}

} // namespace gpu
} // namespace cclx
