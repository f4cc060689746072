// sz_moe_verify_static: the MoE verify step for callers that cannot hand the library a scratch buffer.
//
// sz_moe_verify wants scratch memory from its caller.  Some hosts have none to give: an engine that hands every byte of device
// memory to its own arena at start-up (the reference's session owns all of its device buffers and its kernels never allocate),
// or a plugin loaded into a process whose rules forbid touching the CUDA allocator after initialisation, because a cudaMalloc
// there would stall every stream of the device or fail outright.  For them the scratch lives in this file, in a fixed array in
// device memory that exists on every GPU that loads the library, from load until the process exits.
#include "sz_moe.cuh"

#include <mutex>

#define SZ_STATIC_SCRATCH_BYTES (4 << 20)  // 4 MiB per GPU: every layer shape whose sz_moe_scratch_bytes fits is served
#define SZ_STATIC_MAX_DEVICES 64

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress - it is not a device address, and a
// kernel handed `sz_static_scratch` from the host would read and write the wrong memory.
static __device__ __align__(256) unsigned char sz_static_scratch[SZ_STATIC_SCRATCH_BYTES];

static std::mutex g_static_mu;
static void* g_static_ptr[SZ_STATIC_MAX_DEVICES];  // per device: the array's address in that device's memory, once set up

// Once per device, with that device current: asks the runtime where the array lives on this GPU and clears its control words.
// The clear is synchronous (cudaMemset, then a device synchronise), so that it is ordered before work on ANY stream, not only the
// first caller's.  `again` looks the array up anew (after a cudaDeviceReset the cached address is stale) and clears again.
static int sz_static_setup(int dev, bool again, void** out) {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (again || !g_static_ptr[dev]) {
        void* p = nullptr;
        g_static_ptr[dev] = nullptr;
        const cudaError_t rc = cudaGetSymbolAddress(&p, sz_static_scratch);
        if (rc != cudaSuccess || !p) return sz_fail(SZ_E_CUDA, "cudaGetSymbolAddress(sz_static_scratch): %s", cudaGetErrorString(rc));
        SZ_CUDA(cudaMemset(p, 0, 256));
        SZ_CUDA(cudaDeviceSynchronize());
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return SZ_OK;
}

static int sz_static_device(const char* who, int* dev) {
    SZ_CUDA(cudaGetDevice(dev));
    if (*dev < 0 || *dev >= SZ_STATIC_MAX_DEVICES) return sz_fail(SZ_E_ARG, "%s: device ordinal %d is out of range", who, *dev);
    return SZ_OK;
}

// The static twin of sz_moe_scratch_init: clears the array's control words (counters, the error word) on the current device and
// looks its address up again.  After a call that sz_moe_static_status reported as failed, and after a cudaDeviceReset.
extern "C" int sz_moe_static_reset(void) {
    int dev = 0;
    int rc = sz_static_device("sz_moe_static_reset", &dev);
    if (rc) return rc;
    void* p = nullptr;
    return sz_static_setup(dev, true, &p);
}

// *error = the array's error word on the current device: nonzero once a kernel's bounded wait on an asynchronous copy ran out (the
// y of that call is not valid).  Synchronises `stream`.
extern "C" int sz_moe_static_status(int* error, uint64_t stream) {
    if (!error) return sz_fail(SZ_E_ARG, "sz_moe_static_status: null result pointer");
    int dev = 0;
    int rc = sz_static_device("sz_moe_static_status", &dev);
    if (rc) return rc;
    void* p = nullptr;
    if ((rc = sz_static_setup(dev, false, &p))) return rc;
    unsigned int word = 0;
    SZ_CUDA(cudaMemcpyAsync(&word, (const unsigned char*)p + 4, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SZ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    *error = (int)word;
    return SZ_OK;
}

extern "C" int sz_moe_static_scratch_max(int64_t* bytes) {
    if (!bytes) return sz_fail(SZ_E_ARG, "null result pointer");
    *bytes = SZ_STATIC_SCRATCH_BYTES;
    return SZ_OK;
}

extern "C" int sz_moe_verify_static(const sz_moe_layer* L, uint64_t x, int m, uint64_t y, uint64_t route_idx, uint64_t route_w,
                                    uint64_t stream) {
    int64_t need = 0;
    const int rc = sz_moe_scratch_bytes(L, m, &need);  // also validates the layer and m
    if (rc) return rc;
    if (need > SZ_STATIC_SCRATCH_BYTES)
        return sz_fail(SZ_E_SCRATCH, "sz_moe_verify_static: this layer with %d rows needs %lld bytes of scratch, the built-in array has %d; "
                       "use sz_moe_verify with a caller-provided buffer", m, (long long)need, SZ_STATIC_SCRATCH_BYTES);
    int dev = 0;
    const int rd = sz_static_device("sz_moe_verify_static", &dev);
    if (rd) return rd;
    void* scratch = nullptr;
    const int rs = sz_static_setup(dev, false, &scratch);
    if (rs) return rs;
    return sz_moe_verify(L, x, m, y, route_idx, route_w, (uint64_t)scratch, SZ_STATIC_SCRATCH_BYTES, stream);
}
