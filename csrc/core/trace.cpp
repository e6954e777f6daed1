#include "core/trace.hpp"

#include <nvtx3/nvToolsExt.h>
#include <sys/syscall.h>
#include <unistd.h>

#include "core/env.hpp"

namespace cclx {

namespace {
nvtxDomainHandle_t domain() {
    static nvtxDomainHandle_t d = nvtxDomainCreateA("ccl_b200::API");
    return d;
}
} // namespace

int trace_level() {
    static const int level = env_data::get().itt_level;
    return level;
}

void trace_push(const char* name, uint64_t payload) {
    nvtxEventAttributes_t a = {};
    a.version = NVTX_VERSION;
    a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
    a.messageType = NVTX_MESSAGE_TYPE_ASCII;
    a.message.ascii = name;
    a.payloadType = NVTX_PAYLOAD_TYPE_UNSIGNED_INT64;
    a.payload.ullValue = payload;
    nvtxDomainRangePushEx(domain(), &a);
}

void trace_pop() {
    nvtxDomainRangePop(domain());
}

void trace_mark(const char* name) {
    nvtxEventAttributes_t a = {};
    a.version = NVTX_VERSION;
    a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
    a.messageType = NVTX_MESSAGE_TYPE_ASCII;
    a.message.ascii = name;
    nvtxDomainMarkEx(domain(), &a);
}

void trace_name_thread(const char* name) {
    if (trace_level() > 0)
        nvtxNameOsThreadA((uint32_t)syscall(SYS_gettid), name);
}

} // namespace cclx
