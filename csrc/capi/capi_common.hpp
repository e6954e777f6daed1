// Helpers of the flat C API: exception-to-error-code translation.
#pragma once
#include <exception>
#include <string>

namespace cclx {
namespace capi {

void set_last_error(const std::string& msg);

template <class F>
int guard(F&& f) {
    try {
        f();
        return 0;
    }
    catch (const std::exception& e) {
        set_last_error(e.what());
        return -1;
    }
    catch (...) {
        set_last_error("unknown exception");
        return -1;
    }
}

} // namespace capi
} // namespace cclx

#define CCLX_API extern "C" __attribute__((visibility("default")))
