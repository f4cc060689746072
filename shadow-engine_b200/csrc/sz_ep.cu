// Expert parallelism: the NCCL side.  One communicator per process (one process per GPU); NCCL is loaded with dlopen when
// sz_ep_init or sz_ep_unique_id is first called, so a single-GPU user never needs the library.  The only collective on the
// data path is the all-reduce of a layer's fixed-point output (int64 sum): activations are replicated, so the dispatch is empty.
#include "sz_common.cuh"

#include <dlfcn.h>
#include <string.h>

namespace {
typedef struct { char internal[128]; } NcclId;   // ncclUniqueId
typedef void* NcclComm;
typedef int (*fn_get_id)(NcclId*);
typedef int (*fn_init)(NcclComm*, int, NcclId, int);
typedef int (*fn_allreduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*fn_destroy)(NcclComm);
typedef const char* (*fn_errstr)(int);
const int kNcclInt64 = 4, kNcclSum = 0;          // ncclDataType_t / ncclRedOp_t values of nccl.h

struct Ep {
    void* lib = nullptr;
    fn_get_id get_id = nullptr;
    fn_init init = nullptr;
    fn_allreduce allreduce = nullptr;
    fn_destroy destroy = nullptr;
    fn_errstr errstr = nullptr;
    NcclComm comm = nullptr;
    int rank = 0, world = 0;
    int graph_refs = 0;  // recorded passes (CUDA graphs) that contain a collective of this communicator
} g_ep;

int load_nccl() {
    if (g_ep.lib) return SZ_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        g_ep.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_ep.lib) break;
    }
    if (!g_ep.lib) return sz_fail(SZ_E_CUDA, "cannot load NCCL: %s", dlerror());
    g_ep.get_id = (fn_get_id)dlsym(g_ep.lib, "ncclGetUniqueId");
    g_ep.init = (fn_init)dlsym(g_ep.lib, "ncclCommInitRank");
    g_ep.allreduce = (fn_allreduce)dlsym(g_ep.lib, "ncclAllReduce");
    g_ep.destroy = (fn_destroy)dlsym(g_ep.lib, "ncclCommDestroy");
    g_ep.errstr = (fn_errstr)dlsym(g_ep.lib, "ncclGetErrorString");
    if (!g_ep.get_id || !g_ep.init || !g_ep.allreduce || !g_ep.destroy || !g_ep.errstr) return sz_fail(SZ_E_CUDA, "NCCL lacks a symbol this library binds");
    return SZ_OK;
}
}  // namespace

extern "C" int sz_ep_unique_id(uint8_t id[128]) {
    if (!id) return sz_fail(SZ_E_ARG, "null id");
    int rc = load_nccl();
    if (rc) return rc;
    NcclId u;
    const int e = g_ep.get_id(&u);
    if (e) return sz_fail(SZ_E_CUDA, "ncclGetUniqueId: %s", g_ep.errstr(e));
    memcpy(id, u.internal, 128);
    return SZ_OK;
}

extern "C" int sz_ep_init(int rank, int world, const uint8_t id[128]) {
    if (world < 1 || rank < 0 || rank >= world) return sz_fail(SZ_E_ARG, "rank %d of %d", rank, world);
    if (g_ep.world) return sz_fail(SZ_E_ARG, "sz_ep_init: already initialised (%d ranks)", g_ep.world);
    if (world == 1) { g_ep.rank = 0; g_ep.world = 1; return SZ_OK; }  // one rank: nothing to exchange, NCCL is not needed
    if (!id) return sz_fail(SZ_E_ARG, "null id");
    int rc = load_nccl();
    if (rc) return rc;
    NcclId u;
    memcpy(u.internal, id, 128);
    const int e = g_ep.init(&g_ep.comm, world, u, rank);
    if (e) return sz_fail(SZ_E_CUDA, "ncclCommInitRank: %s", g_ep.errstr(e));
    g_ep.rank = rank; g_ep.world = world;
    return SZ_OK;
}

extern "C" int sz_ep_world(void) { return g_ep.world; }

int sz_ep_graph_refs(int delta) { return g_ep.graph_refs += delta; }

// NCCL waits inside ncclCommDestroy until every graph that recorded one of the communicator's collectives is gone, so a destroy
// with such a session alive would never return: it is refused instead.
extern "C" int sz_ep_destroy(void) {
    if (g_ep.comm && g_ep.graph_refs > 0)
        return sz_fail(SZ_E_ARG, "sz_ep_destroy: %d recorded pass(es) of live sessions still hold the communicator; destroy the sessions first",
                       g_ep.graph_refs);
    if (g_ep.comm) g_ep.destroy(g_ep.comm);
    g_ep.comm = nullptr;
    g_ep.world = 0;
    g_ep.rank = 0;
    return SZ_OK;
}

int sz_ep_allreduce_i64(long long* buf, size_t count, cudaStream_t st) {
    if (g_ep.world <= 1) return SZ_OK;
    const int e = g_ep.allreduce(buf, buf, count, kNcclInt64, kNcclSum, g_ep.comm, st);
    if (e) return sz_fail(SZ_E_CUDA, "ncclAllReduce: %s", g_ep.errstr(e));
    sz_trace_mark("ep_allreduce", st);
    return SZ_OK;
}
