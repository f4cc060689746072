// Expert parallelism: the NCCL side.  One communicator per process (one process per GPU); NCCL is loaded with dlopen when
// sz_ep_init or sz_ep_unique_id is first called, so a single-GPU user never needs the library.  The only collective on the
// data path is the all-reduce of a layer's fixed-point output (int64 sum): activations are replicated, so the dispatch is empty.
#include "sz_common.cuh"

#include <dlfcn.h>
#include <stdlib.h>
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
int g_ep_generation = 0;  // bumped whenever the exchange set-up changes (communicator up / down, buffers attached / detached)

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
    if (world == 1) { g_ep.rank = 0; g_ep.world = 1; g_ep_generation++; return SZ_OK; }  // one rank: nothing to exchange, NCCL is not needed
    if (!id) return sz_fail(SZ_E_ARG, "null id");
    int rc = load_nccl();
    if (rc) return rc;
    NcclId u;
    memcpy(u.internal, id, 128);
    const int e = g_ep.init(&g_ep.comm, world, u, rank);
    if (e) return sz_fail(SZ_E_CUDA, "ncclCommInitRank: %s", g_ep.errstr(e));
    g_ep.rank = rank; g_ep.world = world;
    g_ep_generation++;
    return SZ_OK;
}

extern "C" int sz_ep_world(void) { return g_ep.world; }
// Sessions compare this with the value they recorded their passes under: a pass recorded under another exchange set-up is dropped.
int sz_ep_generation(void) { return g_ep_generation; }

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
    g_ep_generation++;
    return SZ_OK;
}

int sz_ep_allreduce_i64(long long* buf, size_t count, cudaStream_t st) {
    if (g_ep.world <= 1) return SZ_OK;
    const int e = g_ep.allreduce(buf, buf, count, kNcclInt64, kNcclSum, g_ep.comm, st);
    if (e) return sz_fail(SZ_E_CUDA, "ncclAllReduce: %s", g_ep.errstr(e));
    sz_trace_mark("ep_allreduce", st);
    return SZ_OK;
}

// ---- exchange over peer memory ------------------------------------------------------------------------------------------------------
#include "sz_moe.cuh"

namespace {
struct P2p {
    int rank = 0, world = 0;
    int hidden = 0;
    int polls = SZ_EP_SPIN_LIMIT;   // how often a finish block polls a counter before it gives up
    u8* buf[SZ_EP_MAX_RANKS] = {};
    int graph_refs = 0;             // recorded passes of live sessions whose kernels hold these buffer addresses
} g_p2p;

bool p2p_attached(uint64_t ptr) {
    for (int r = 0; r < g_p2p.world; r++)
        if ((uint64_t)g_p2p.buf[r] == ptr) return true;
    return false;
}
}  // namespace

// A recorded pass bakes the buffer addresses, the rank and the poll budget into its kernels' arguments: while one is alive the
// attachment must not change and the buffers must stay mapped (a replay would store into freed or unmapped peer memory).
int sz_ep_p2p_graph_refs(int delta) { return g_p2p.graph_refs += delta; }

// Sums the ranks' rows of the current slot into y.  grid: any; block 256.  Thread 0 of every block waits for the sources (a bounded
// number of polls; on running out it raises the header's error word and the block goes on with what is there, so the kernel always
// ends).  The last block to finish closes the exchange: epoch + 1, target + blocks of the combine kernel.
__global__ void __launch_bounds__(256)
sz_ep_finish_kernel(u8* __restrict__ mine, int world, long long row_elems, unsigned long long nb, int n, float* __restrict__ y, int poll_limit) {
    __shared__ int s_last;
    sz_pdl_wait();
    sz_pdl_trigger();
    SzEpHeader* hdr = (SzEpHeader*)mine;
    const unsigned long long want = hdr->target + nb;
    const int slot = (int)(hdr->epoch & 1ull);
    if (threadIdx.x < world) {
        volatile unsigned long long* c = sz_ep_arrive(mine, threadIdx.x);
        int polls = 0;
        bool ok = false;
        while (polls < poll_limit && *(volatile unsigned int*)&hdr->error == 0) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(c));
            if (v >= want) { ok = true; break; }
            polls++;
            __nanosleep(polls < 4096 ? 32 : 1000);   // quick at first, then about a microsecond a poll
        }
        if (!ok) atomicExch(&hdr->error, 1u);
    }
    __syncthreads();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        long long f = 0;
        for (int r = 0; r < world; r++) f += __ldcg(sz_ep_slot(mine, world, row_elems, slot, r) + i);
        y[i] = (float)((double)f * (1.0 / 1099511627776.0));
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&hdr->ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        hdr->ticket = 0;
        hdr->target = want;
        hdr->epoch = hdr->epoch + 1;
    }
}

extern "C" int sz_ep_p2p_bytes(int world, int hidden, int64_t* bytes) {
    if (!bytes || world < 1 || world > SZ_EP_MAX_RANKS || hidden < 1) return sz_fail(SZ_E_ARG, "sz_ep_p2p_bytes: %d ranks, hidden %d", world, hidden);
    *bytes = SZ_EP_HDR_BYTES + (int64_t)2 * world * SZ_MAX_VERIFY * hidden * 8;
    return SZ_OK;
}

// The exchange buffer has to be an allocation of its own (CUDA IPC exports whole allocations), made once at start-up.
extern "C" int sz_ep_p2p_alloc(int64_t bytes, uint64_t* ptr) {
    if (!ptr || bytes <= 0) return sz_fail(SZ_E_ARG, "sz_ep_p2p_alloc: bad argument");
    void* p = nullptr;
    SZ_CUDA(cudaMalloc(&p, (size_t)bytes));
    SZ_CUDA(cudaMemset(p, 0, (size_t)bytes));
    SZ_CUDA(cudaDeviceSynchronize());
    *ptr = (uint64_t)p;
    return SZ_OK;
}
extern "C" int sz_ep_p2p_free(uint64_t ptr) {
    if (ptr && p2p_attached(ptr)) return sz_fail(SZ_E_ARG, "sz_ep_p2p_free: the buffer is attached to the exchange; sz_ep_p2p_detach first");
    if (ptr) SZ_CUDA(cudaFree((void*)ptr));
    return SZ_OK;
}
extern "C" int sz_ep_ipc_export(uint64_t ptr, uint8_t handle[64]) {
    if (!ptr || !handle) return sz_fail(SZ_E_ARG, "sz_ep_ipc_export: null argument");
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    SZ_CUDA(cudaIpcGetMemHandle(&h, (void*)ptr));
    memcpy(handle, &h, 64);
    return SZ_OK;
}
extern "C" int sz_ep_ipc_import(const uint8_t handle[64], uint64_t* ptr) {
    if (!ptr || !handle) return sz_fail(SZ_E_ARG, "sz_ep_ipc_import: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void* p = nullptr;
    SZ_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = (uint64_t)p;
    return SZ_OK;
}
extern "C" int sz_ep_ipc_close(uint64_t ptr) {
    if (ptr && p2p_attached(ptr)) return sz_fail(SZ_E_ARG, "sz_ep_ipc_close: the mapping is attached to the exchange; sz_ep_p2p_detach first");
    if (ptr) SZ_CUDA(cudaIpcCloseMemHandle((void*)ptr));
    return SZ_OK;
}

// bufs[r]: rank r's exchange buffer as this process addresses it (its own allocation for r == rank, an imported mapping otherwise;
// on one GPU, for tests, simply other local allocations).  Expert-parallel layers then exchange over these buffers instead of NCCL.
extern "C" int sz_ep_p2p_attach(int rank, int world, int hidden, const uint64_t* bufs) {
    if (!bufs || world < 1 || world > SZ_EP_MAX_RANKS || rank < 0 || rank >= world || hidden < 1)
        return sz_fail(SZ_E_ARG, "sz_ep_p2p_attach: rank %d of %d, hidden %d", rank, world, hidden);
    for (int r = 0; r < world; r++)
        if (!bufs[r] || (bufs[r] & 255)) return sz_fail(SZ_E_ARG, "sz_ep_p2p_attach: buffer %d is null or not 256-byte aligned", r);
    if (g_p2p.graph_refs > 0)
        return sz_fail(SZ_E_ARG, "sz_ep_p2p_attach: %d recorded pass(es) of live sessions hold the current attachment; destroy the sessions first", g_p2p.graph_refs);
    g_ep_generation++;
    g_p2p.rank = rank; g_p2p.world = world; g_p2p.hidden = hidden;
    {
        // the poll budget of a wait: about two seconds by default (a peer may be busy recording a graph or loading a module);
        // SZ_EP_WAIT_POLLS overrides it (the test of a wait that runs out uses a small one)
        const char* e = getenv("SZ_EP_WAIT_POLLS");
        const long v = e ? atol(e) : 0;
        g_p2p.polls = v > 0 && v < 2000000000L ? (int)v : SZ_EP_SPIN_LIMIT;
    }
    for (int r = 0; r < SZ_EP_MAX_RANKS; r++) g_p2p.buf[r] = r < world ? (u8*)bufs[r] : nullptr;
    return SZ_OK;
}
extern "C" int sz_ep_p2p_detach(void) {
    if (g_p2p.graph_refs > 0)
        return sz_fail(SZ_E_ARG, "sz_ep_p2p_detach: %d recorded pass(es) of live sessions hold the attachment; destroy the sessions first", g_p2p.graph_refs);
    g_p2p = P2p();
    g_ep_generation++;
    return SZ_OK;
}
extern "C" int sz_ep_p2p_world(void) { return g_p2p.world; }

// 0: no wait of this rank's exchanges ever ran out.  Synchronises the device.
extern "C" int sz_ep_p2p_status(int* error) {
    if (!error) return sz_fail(SZ_E_ARG, "null argument");
    *error = 0;
    if (!g_p2p.world) return SZ_OK;
    SzEpHeader h;
    SZ_CUDA(cudaMemcpy(&h, g_p2p.buf[g_p2p.rank], sizeof(h), cudaMemcpyDeviceToHost));
    *error = (int)h.error;
    return SZ_OK;
}

// for sz_moe.cu: the push descriptor of the attached exchange (world 0: none), and the finish launch
int sz_ep_p2p_push(int hidden, SzEpPush* p) {
    memset(p, 0, sizeof(*p));
    if (!g_p2p.world) return SZ_OK;
    if (hidden != g_p2p.hidden) return sz_fail(SZ_E_ARG, "the exchange buffers were sized for hidden %d, the layer has %d", g_p2p.hidden, hidden);
    for (int r = 0; r < g_p2p.world; r++) p->buf[r] = g_p2p.buf[r];
    p->world = g_p2p.world; p->me = g_p2p.rank;
    p->row_elems = (long long)SZ_MAX_VERIFY * hidden;
    return SZ_OK;
}
int sz_ep_p2p_finish(int m, int hidden, unsigned long long combine_blocks, float* y, cudaStream_t st);
int sz_moe_combine_blocks(const sz_moe_layer* L, int m);  // sz_moe.cu

// The finish half on its own, for hosts (and tests) that run the two halves of an exchange apart: sz_moe_verify_partial pushes,
// this adds up.  The layer says how many blocks the combine kernel of the push had.
extern "C" int sz_moe_finish_exchange(const sz_moe_layer* L, int m, uint64_t y, uint64_t stream) {
    if (!L || !y || m < 1 || m > SZ_MAX_VERIFY) return sz_fail(SZ_E_ARG, "sz_moe_finish_exchange: bad argument");
    if (!g_p2p.world) return sz_fail(SZ_E_ARG, "sz_moe_finish_exchange: no exchange attached");
    if (L->hidden != g_p2p.hidden) return sz_fail(SZ_E_ARG, "the exchange buffers were sized for hidden %d, the layer has %d", g_p2p.hidden, L->hidden);
    return sz_ep_p2p_finish(m, L->hidden, (unsigned long long)sz_moe_combine_blocks(L, m), (float*)y, (cudaStream_t)stream);
}

int sz_ep_p2p_finish(int m, int hidden, unsigned long long combine_blocks, float* y, cudaStream_t st) {
    const int n = m * hidden;
    SZ_CUDA(sz_launch("ep_finish", sz_ep_finish_kernel, dim3((n + 1023) / 1024), dim3(256), 0, st, true, g_p2p.buf[g_p2p.rank], g_p2p.world,
                      (long long)SZ_MAX_VERIFY * hidden, combine_blocks, n, y, g_p2p.polls));
    return SZ_OK;
}

SZ_TIMELINE_READER(ep)
