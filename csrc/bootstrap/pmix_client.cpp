#include "bootstrap/pmix_client.hpp"

#include <dlfcn.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace cclx {

namespace {

// --- the part of PMIx's public binary interface used below (pmix_common.h of PMIx 2 to 5) ---
constexpr int PMIX_MAX_NSLEN = 255;
struct pmix_proc_t {
    char nspace[PMIX_MAX_NSLEN + 1];
    uint32_t rank;
};
constexpr uint32_t PMIX_RANK_WILDCARD = UINT32_MAX - 1;
constexpr int PMIX_SUCCESS = 0;
// data type codes of pmix_value_t::type
constexpr uint16_t PMIX_INT = 6, PMIX_INT16 = 8, PMIX_INT32 = 9, PMIX_UINT = 11, PMIX_UINT16 = 13, PMIX_UINT32 = 14,
                   PMIX_UINT64 = 15;
struct pmix_value_t {
    uint16_t type;
    union { // the full union holds pointers and size_t as well: 8-byte aligned, the integer members overlay its start
        int integer;
        int16_t int16;
        int32_t int32;
        unsigned int uint;
        uint16_t uint16;
        uint32_t uint32;
        uint64_t uint64;
        void* ptr;
        char pad[24];
    } data;
};
constexpr const char* KEY_LOCAL_SIZE = "pmix.local.size"; // PMIX_LOCAL_SIZE, asked of the wildcard rank
constexpr const char* KEY_LOCAL_RANK = "pmix.lrank"; // PMIX_LOCAL_RANK, asked of this process

typedef int (*init_fn)(pmix_proc_t*, void*, size_t);
typedef int (*get_fn)(const pmix_proc_t*, const char*, const void*, size_t, pmix_value_t**);
typedef int (*finalize_fn)(const void*, size_t);
typedef const char* (*strerror_fn)(int);
typedef void (*value_destruct_fn)(pmix_value_t*);

bool as_int(const pmix_value_t& v, int& out) {
    switch (v.type) {
        case PMIX_INT: out = v.data.integer; return true;
        case PMIX_INT16: out = v.data.int16; return true;
        case PMIX_INT32: out = v.data.int32; return true;
        case PMIX_UINT: out = (int)v.data.uint; return true;
        case PMIX_UINT16: out = v.data.uint16; return true;
        case PMIX_UINT32: out = (int)v.data.uint32; return true;
        case PMIX_UINT64: out = (int)v.data.uint64; return true;
        default: return false;
    }
}

} // namespace

bool pmix_local_coord(const std::string& lib_path, int& local_rank, int& local_size, std::string& why) {
    std::vector<std::string> names;
    if (!lib_path.empty())
        names.push_back(lib_path);
    else {
        names.push_back("libpmix.so.2");
        names.push_back("libpmix.so");
    }
    void* h = nullptr;
    for (auto& n : names) {
        h = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (h)
            break;
        const char* err = dlerror();
        why += std::string(err ? err : "dlopen failed") + "; ";
    }
    if (!h)
        return false;
    init_fn init = (init_fn)dlsym(h, "PMIx_Init");
    get_fn get = (get_fn)dlsym(h, "PMIx_Get");
    finalize_fn fin = (finalize_fn)dlsym(h, "PMIx_Finalize");
    strerror_fn serr = (strerror_fn)dlsym(h, "PMIx_Error_string");
    value_destruct_fn vdes = (value_destruct_fn)dlsym(h, "PMIx_Value_destruct"); // a function from PMIx 4.2 on
    if (!init || !get || !fin) {
        why += "PMIx entry points missing";
        dlclose(h);
        return false;
    }
    auto text = [&](int rc) { return std::string(serr ? serr(rc) : "error") + " (" + std::to_string(rc) + ")"; };
    pmix_proc_t me;
    std::memset(&me, 0, sizeof(me));
    int rc = init(&me, nullptr, 0);
    if (rc != PMIX_SUCCESS) {
        why += "PMIx_Init: " + text(rc);
        dlclose(h);
        return false;
    }
    bool ok = true;
    auto ask = [&](const pmix_proc_t& whom, const char* key, int& out) {
        pmix_value_t* val = nullptr;
        const int r = get(&whom, key, nullptr, 0, &val);
        if (r != PMIX_SUCCESS || !val) {
            why += std::string("PMIx_Get(") + key + "): " + text(r) + "; ";
            ok = false;
            return;
        }
        if (!as_int(*val, out)) {
            why += std::string("PMIx_Get(") + key + "): value of type " + std::to_string(val->type) + "; ";
            ok = false;
        }
        if (vdes)
            vdes(val);
        std::free(val);
    };
    pmix_proc_t all = me;
    all.rank = PMIX_RANK_WILDCARD;
    int lr = -1, ls = -1;
    ask(all, KEY_LOCAL_SIZE, ls);
    ask(me, KEY_LOCAL_RANK, lr);
    fin(nullptr, 0);
    // the library stays loaded: it may have registered exit handlers
    if (ok && lr >= 0 && ls > 0 && lr < ls) {
        local_rank = lr;
        local_size = ls;
        return true;
    }
    if (ok)
        why += "implausible values: local rank " + std::to_string(lr) + ", local size " + std::to_string(ls);
    return false;
}

} // namespace cclx
