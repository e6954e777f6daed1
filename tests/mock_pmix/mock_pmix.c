/* A stand-in for libpmix with the two calls the library makes (there is no PMIx in the image): PMIx_Init names
 * the process, PMIx_Get serves "pmix.local.size" (asked of the wildcard rank, as uint32) and "pmix.lrank" (asked
 * of the process itself, as uint16) from MOCK_PMIX_LOCAL_SIZE / MOCK_PMIX_LOCAL_RANK.  MOCK_PMIX_FAIL_INIT=1
 * makes PMIx_Init fail the way it does for a process that no PMIx-aware launcher started.
 *
 * Build: cc -shared -fPIC -O1 -o libmockpmix.so mock_pmix.c */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    char nspace[256];
    uint32_t rank;
} pmix_proc_t;

typedef struct {
    uint16_t type;
    union {
        uint16_t uint16;
        uint32_t uint32;
        void* ptr;
        char pad[24];
    } data;
} pmix_value_t;

#define PMIX_SUCCESS 0
#define PMIX_ERR_UNREACH (-25)
#define PMIX_ERR_NOT_FOUND (-46)
#define PMIX_RANK_WILDCARD (UINT32_MAX - 1)
#define PMIX_UINT16 13
#define PMIX_UINT32 14

static uint32_t my_rank;

int PMIx_Init(pmix_proc_t* proc, void* info, size_t ninfo) {
    (void)info;
    (void)ninfo;
    if (getenv("MOCK_PMIX_FAIL_INIT"))
        return PMIX_ERR_UNREACH;
    const char* r = getenv("MOCK_PMIX_RANK");
    my_rank = r ? (uint32_t)atoi(r) : 0;
    if (proc) {
        memset(proc, 0, sizeof(*proc));
        strcpy(proc->nspace, "mock-job");
        proc->rank = my_rank;
    }
    return PMIX_SUCCESS;
}

int PMIx_Get(const pmix_proc_t* proc, const char* key, const void* info, size_t ninfo, pmix_value_t** val) {
    (void)info;
    (void)ninfo;
    if (!proc || strcmp(proc->nspace, "mock-job") != 0)
        return PMIX_ERR_NOT_FOUND;
    pmix_value_t* v = (pmix_value_t*)calloc(1, sizeof(*v));
    if (strcmp(key, "pmix.local.size") == 0 && proc->rank == PMIX_RANK_WILDCARD) {
        const char* s = getenv("MOCK_PMIX_LOCAL_SIZE");
        v->type = PMIX_UINT32;
        v->data.uint32 = s ? (uint32_t)atoi(s) : 1;
    }
    else if (strcmp(key, "pmix.lrank") == 0 && proc->rank == my_rank) {
        const char* s = getenv("MOCK_PMIX_LOCAL_RANK");
        v->type = PMIX_UINT16;
        v->data.uint16 = s ? (uint16_t)atoi(s) : 0;
    }
    else {
        free(v);
        return PMIX_ERR_NOT_FOUND;
    }
    *val = v;
    return PMIX_SUCCESS;
}

int PMIx_Finalize(const void* info, size_t ninfo) {
    (void)info;
    (void)ninfo;
    return PMIX_SUCCESS;
}

const char* PMIx_Error_string(int rc) {
    return rc == PMIX_ERR_UNREACH ? "UNREACHABLE" : (rc == PMIX_ERR_NOT_FOUND ? "NOT-FOUND" : "ERROR");
}
