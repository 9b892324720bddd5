// NCCL binding for the cross-shard sums (per-level histograms, child row counts).  NCCL is resolved at run
// time with dlopen so that the library has no link-time dependency on it: single-GPU use never touches
// NCCL, and in a torch process the NCCL that torch already loaded is the one that gets picked up.
// The reference has no multi-GPU path (ext/EvoTreesCUDAExt.jl:7-12 selects one CUDA backend).
#include "evb_internal.cuh"
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

namespace {

typedef struct { char internal[128]; } nccl_uid;
typedef void *nccl_comm;
enum { NCCL_INT32 = 2, NCCL_FLOAT64 = 8, NCCL_SUM = 0 };

struct NcclApi {
    void *lib = nullptr;
    int (*GetUniqueId)(nccl_uid *) = nullptr;
    int (*CommInitRank)(nccl_comm *, int, nccl_uid, int) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    int (*CommDestroy)(nccl_comm) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    int (*CommGetAsyncError)(nccl_comm, int *) = nullptr;
};
NcclApi g_nccl;

int32_t load_nccl() {
    if (g_nccl.lib) return EVB_OK;
    const char *env = getenv("EVB_NCCL_LIB");
    const char *names[] = {env, "libnccl.so.2", "libnccl.so"};
    void *lib = nullptr;
    for (const char *nm : names) {
        if (!nm || !*nm) continue;
        lib = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (lib) break;
    }
    if (!lib) {
        evb_set_error("cannot load NCCL (set EVB_NCCL_LIB to the path of libnccl.so.2): %s", dlerror());
        return EVB_ERR_NCCL;
    }
    NcclApi a;
    a.lib = lib;
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(lib, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(lib, "ncclCommInitRank");
    a.AllReduce = (decltype(a.AllReduce))dlsym(lib, "ncclAllReduce");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(lib, "ncclCommDestroy");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(lib, "ncclGetErrorString");
    a.CommGetAsyncError = (decltype(a.CommGetAsyncError))dlsym(lib, "ncclCommGetAsyncError");
    if (!a.GetUniqueId || !a.CommInitRank || !a.AllReduce || !a.CommDestroy || !a.GetErrorString) {
        evb_set_error("NCCL library lacks a required symbol");
        return EVB_ERR_NCCL;
    }
    g_nccl = a;
    return EVB_OK;
}

int32_t nccl_fail(int rc, const char *what) {
    evb_set_error("NCCL error in %s: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?");
    return EVB_ERR_NCCL;
}

} // namespace

int32_t evb_nccl_unique_id(uint8_t id[128]) {
    EVB_CHECK(load_nccl());
    nccl_uid u;
    int rc = g_nccl.GetUniqueId(&u);
    if (rc != 0) return nccl_fail(rc, "ncclGetUniqueId");
    memcpy(id, u.internal, 128);
    return EVB_OK;
}

// Records the id; the communicator itself is created by the first collective (evb_nccl_ensure).  Creating it costs
// from 0.3 s (2 ranks) to 2 s (8 ranks), and a handle on the peer-access path never issues an NCCL collective.
int32_t evb_nccl_init(evb_handle *h, const uint8_t id[128], int rank, int world) {
    EVB_CHECK(load_nccl());
    memcpy(h->nccl_id, id, 128);
    h->nccl_pending = true;
    h->rank = rank;
    h->world = world;
    return EVB_OK;
}

// All ranks reach their first collective at the same point of the same launch sequence, so they all create the
// communicator together.
static int32_t evb_nccl_ensure(evb_handle *h) {
    if (h->nccl_comm) return EVB_OK;
    if (!h->nccl_pending) { evb_set_error("NCCL collective without evb_comm_init"); return EVB_ERR_NCCL; }
    nccl_uid u;
    memcpy(u.internal, h->nccl_id, 128);
    nccl_comm comm = nullptr;
    int rc = g_nccl.CommInitRank(&comm, h->world, u, h->rank);
    if (rc != 0) return nccl_fail(rc, "ncclCommInitRank");
    h->nccl_comm = comm;
    h->nccl_pending = false;
    return EVB_OK;
}

int32_t evb_nccl_allreduce_f64(evb_handle *h, double *buf, size_t count) {
    EVB_CHECK(evb_nccl_ensure(h));
    int rc = g_nccl.AllReduce(buf, buf, count, NCCL_FLOAT64, NCCL_SUM, (nccl_comm)h->nccl_comm, h->st);
    if (rc != 0) return nccl_fail(rc, "ncclAllReduce(f64)");
    return EVB_OK;
}

int32_t evb_nccl_allreduce_i32(evb_handle *h, const int32_t *src, int32_t *dst, size_t count) {
    EVB_CHECK(evb_nccl_ensure(h));
    int rc = g_nccl.AllReduce(src, dst, count, NCCL_INT32, NCCL_SUM, (nccl_comm)h->nccl_comm, h->st);
    if (rc != 0) return nccl_fail(rc, "ncclAllReduce(i32)");
    return EVB_OK;
}

// Asynchronous communicator errors (a peer that died, a network fault) are polled on the host before a
// tree is enqueued, so a broken communicator turns into an error code instead of a hang.
int32_t evb_nccl_check(evb_handle *h) {
    if (!h->nccl_comm || !g_nccl.CommGetAsyncError) return EVB_OK;
    int async = 0;
    int rc = g_nccl.CommGetAsyncError((nccl_comm)h->nccl_comm, &async);
    if (rc != 0) return nccl_fail(rc, "ncclCommGetAsyncError");
    if (async != 0) return nccl_fail(async, "communicator (asynchronous error)");
    return EVB_OK;
}

void evb_nccl_destroy(evb_handle *h) {
    if (h->nccl_comm && g_nccl.CommDestroy) g_nccl.CommDestroy((nccl_comm)h->nccl_comm);
    h->nccl_comm = nullptr;
}
