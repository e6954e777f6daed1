// Local rank and local size from a PMIx server (CCL_PROCESS_LAUNCHER=pmix), the library opened at run time.
//
// The reference asks PMIx for exactly these two values (src/common/api_wrapper/pmix_api_wrapper.cpp:27-68,
// entry-point table in pmix_api_wrapper.hpp:30-44; the library is CCL_PMIX_LIBRARY_PATH, else libpmix.so).
// Here the part of PMIx's binary interface that this needs is declared in pmix_client.cpp, so that the build
// has no PMIx dependency.
#pragma once
#include <string>

namespace cclx {

// True with the two values when a PMIx library could be opened, PMIx_Init succeeded (the process was started
// by a PMIx-aware launcher) and both keys were served; `why` says what failed otherwise.
bool pmix_local_coord(const std::string& lib_path, int& local_rank, int& local_size, std::string& why);

} // namespace cclx
