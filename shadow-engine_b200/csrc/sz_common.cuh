// Shared device/host helpers for the shadowzero_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/shadowzero_b200.h"

typedef uint8_t u8;
typedef uint16_t u16;
typedef uint32_t u32;
typedef uint64_t u64;

// ---- host side: errors ------------------------------------------------------------------------------------------------
void sz_set_error(const char* fmt, ...);
int sz_fail(int code, const char* fmt, ...);
#define SZ_CUDA(expr)                                                                                   \
    do {                                                                                                \
        cudaError_t e_ = (expr);                                                                        \
        if (e_ != cudaSuccess) return sz_fail(SZ_E_CUDA, "%s: %s", #expr, cudaGetErrorString(e_));      \
    } while (0)

static inline bool sz_aligned16(u64 p) { return (p & 15) == 0; }

// Per-kernel timing (sz_trace_begin): records the next caller-provided event on `stream` under `name`.  No-op when tracing is off.
void sz_trace_mark(const char* name, cudaStream_t stream);
bool sz_trace_active();

// Launch with the programmatic-dependent-launch attribute: the kernel may start while its predecessor on the stream drains;
// every such kernel calls sz_pdl_wait() before it touches anything the predecessor wrote.
template <typename... KArgs, typename... Args>
static inline cudaError_t sz_launch(const char* name, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    sz_trace_mark(name, stream);
    return rc;
}

// ---- device side --------------------------------------------------------------------------------------------------------
#ifdef __CUDACC__

// Phase stamps, debug builds only (-DSZ_PHASES): thread 0 of a block keeps clock64() readings in registers and one chosen block
// writes them out at the end; sz_phase_read_<file> copies them to the host.  Compiled out otherwise.
#ifdef SZ_PHASES
static __device__ long long sz_phase_t[16][16];
#define SZ_PH_DECL long long _ph[12]; int _phn = 0; (void)_ph; (void)_phn
#define SZ_PH() do { if (threadIdx.x == 0 && _phn < 12) { _ph[_phn++] = clock64(); } } while (0)
#define SZ_PH_FLUSH(kid, cond) do { if (threadIdx.x == 0 && (cond)) { for (int _i = 0; _i < 12; _i++) sz_phase_t[kid][_i] = _i < _phn ? _ph[_i] : 0; } } while (0)
#else
#define SZ_PH_DECL do {} while (0)
#define SZ_PH() do {} while (0)
#define SZ_PH_FLUSH(kid, cond) do {} while (0)
#endif

// Wait for the kernels this one depends on (no-op when launched without the PDL attribute).
#ifdef SZ_PHASES
// debug builds: block 0 of every kernel logs (source line of the wait, time before it, time after it) - a device-side timeline of a
// pass, valid inside CUDA graphs too.  One log per translation unit; sz_timeline_read_<file> copies it out.
static __device__ unsigned long long sz_tl[3 * 4096];
static __device__ unsigned int sz_tl_n;
__device__ __forceinline__ unsigned long long sz_gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void sz_pdl_wait_at(int line) {
    const bool log = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0;
    const unsigned long long t0 = log ? sz_gtime() : 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (log) {
        const unsigned int i = atomicAdd(&sz_tl_n, 1u);
        if (i < 4096) { sz_tl[3 * i] = (unsigned long long)line; sz_tl[3 * i + 1] = t0; sz_tl[3 * i + 2] = sz_gtime(); }
    }
}
#define sz_pdl_wait() sz_pdl_wait_at(__LINE__)
#define SZ_TIMELINE_READER(name)                                                                                                  \
    extern "C" int sz_timeline_read_##name(unsigned long long* out, unsigned int* n, int reset) {                                 \
        if (cudaMemcpyFromSymbol(n, sz_tl_n, 4) != cudaSuccess) return 1;                                                         \
        if (cudaMemcpyFromSymbol(out, sz_tl, sizeof(unsigned long long) * 3 * 4096) != cudaSuccess) return 1;                     \
        if (reset) { const unsigned int z = 0; if (cudaMemcpyToSymbol(sz_tl_n, &z, 4) != cudaSuccess) return 1; }                 \
        return 0;                                                                                                                 \
    }
#else
__device__ __forceinline__ void sz_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define SZ_TIMELINE_READER(name)
#endif
// Let the next kernel on the stream begin its prologue.
__device__ __forceinline__ void sz_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A 16-byte read-only load the compiler must leave where it is written: a plain __ldg may be sunk to its first use, which for a
// prefetch placed ahead of griddepcontrol.wait would put it after the wait.  Volatile asm statements keep their order.
__device__ __forceinline__ uint4 sz_ldg16_here(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// 2- and 4-byte forms of the same (read-only data: weights, or what a kernel two or more launches back wrote).
__device__ __forceinline__ u32 sz_ldg32_here(const void* p) {
    u32 v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ u16 sz_ldg16b_here(const void* p) {
    u16 v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ double sz_ldg64f_here(const double* p) {
    double v;
    asm volatile("ld.global.nc.f64 %0, [%1];" : "=d"(v) : "l"(p));
    return v;
}

// The same for a 4-byte load of data that other kernels write (an ordinary global load, kept where it is written).
__device__ __forceinline__ float sz_ld32_here(const float* p) {
    float v;
    asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ float sz_f16_to_f32(u16 h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ float sz_bf16_to_f32(u16 b) { return __uint_as_float((u32)b << 16); }

__device__ __forceinline__ float sz_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double sz_warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// sigmoid as the CPU reference computes it: in f64, then narrowed (crates/shadowzero-model/src/forward.rs:262-264).
// The CPU reference takes the sigmoid in f64 and rounds (forward.rs:262-264).  A double-precision exp and divide cost about a
// microsecond of dependent latency each on this part, which is the whole budget of a kernel here, so this is the f32 form: it
// differs from the rounded f64 value by an ulp or two, the same size as the f32 accumulation noise of the dot products around it.
__device__ __forceinline__ float sz_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
// 1 / sqrt(v) to about 1e-14 relative: the f32 estimate refined by one Newton step in f64.  A correctly rounded f64 square root
// and divide cost several hundred cycles of dependent latency; this is four multiply-adds.
__device__ __forceinline__ double sz_rsqrt64(double v) {
    const double r = (double)rsqrtf((float)v);
    return r * fma(-0.5 * v, r * r, 1.5);
}

__device__ __forceinline__ float sz_silu(float x) { return x * sz_sigmoid(x); }

// ---- mbarrier + bulk async copy (TMA engine, untiled form) ---------------------------------------------------------------
__device__ __forceinline__ u32 sz_smem_addr(const void* p) { return (u32)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void sz_mbar_init(u64* bar, u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sz_smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void sz_mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void sz_mbar_expect_tx(u64* bar, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sz_smem_addr(bar)), "r"(bytes) : "memory");
}
// Bounded wait on a phase: gives up after `limit` polls and returns false (the caller records an error and leaves).
__device__ __forceinline__ bool sz_mbar_wait(u64* bar, u32 phase, u32 limit = 20000000u) {
    u32 ok = 0;
    for (u32 i = 0; i < limit; i++) {
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(ok)
            : "r"(sz_smem_addr(bar)), "r"(phase)
            : "memory");
        if (ok) return true;
    }
    return false;
}
// global -> shared bulk copy; src and dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void sz_bulk_g2s(void* dst, const void* src, u32 bytes, u64* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sz_smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(sz_smem_addr(bar))
                 : "memory");
}

#endif  // __CUDACC__
