// Top-64 of each row of logits, shared by the session's dense head and the screened (proxy) head.
#pragma once

#include "sz_common.cuh"

#ifdef __CUDACC__

// ---- top-64 of each row of logits: largest first, ties to the lower id, NaN as -inf (the order of kernels/forward.cu:3565-3625).
// A key packs (orderable value bits, ~id) so that one 64-bit descending sort gives that order.
#define SZ_TK_N 4096
__device__ __forceinline__ u64 sz_tk_key(float v, u32 id) {
    if (v != v) v = -INFINITY;
    if (v == 0.0f) v = 0.0f;  // -0 ties with +0 in the reference's comparison (va == vb): one key for both (decoded as +0)
    u32 b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((u64)b << 32) | (u64)(0xffffffffu - id);
}
__device__ __forceinline__ void sz_tk_unkey(u64 k, float& v, u32& id) {
    u32 b = (u32)(k >> 32);
    b = (b & 0x80000000u) ? (b & 0x7fffffffu) : ~b;
    v = __uint_as_float(b);
    id = 0xffffffffu - (u32)k;
}
// A key for a slot that holds no logit (past the end of a row): below every real key (whose high word is at least 0x007fffff) and
// different for every slot, so that keys never tie - the selection below counts on that.  Decoded as (-inf, id 0xffffffff).
__device__ __forceinline__ u64 sz_tk_pad(int slot) { return (u64)(0xfffu - ((u32)slot & 0xfffu)); }
__device__ __forceinline__ bool sz_tk_is_pad(u64 k) { return (k >> 32) == 0; }
// The 64 best of up to 16 * 256 keys held 16 a thread, written sorted (descending) to dst[0..64).  Instead of sorting everything:
// the 64th best of the 256 per-thread maxima is a floor under the 64th best key (64 keys are at least that large), so only keys at
// or above it can be among the winners - at most 64 threads x 16 keys, typically ~70 - and only those are sorted.
// sm: 256 keys (the maxima); cand: 1024 keys; cnt: one counter.  All 256 threads call it.
__device__ __forceinline__ void sz_tk_select(const u64* key, u64* sm, u64* cand, int* cnt, u64* dst) {
    const int t = threadIdx.x;
    u64 mx = key[0];
#pragma unroll
    for (int i = 1; i < 16; i++) mx = key[i] > mx ? key[i] : mx;
    sm[t] = mx;
    if (t == 0) *cnt = 0;
    __syncthreads();
    // rank of this thread's maximum among the 256 (keys are distinct; the thread number would break a tie)
    int rank = 0;
    for (int i = 0; i < 256; i += 2) {
        const ulonglong2 o = *(const ulonglong2*)(sm + i);
        rank += (o.x > mx || (o.x == mx && i < t)) + (o.y > mx || (o.y == mx && i + 1 < t));
    }
    __syncthreads();
    if (rank == 63) sm[0] = mx;
    __syncthreads();
    const u64 floor64 = sm[0];
#pragma unroll
    for (int i = 0; i < 16; i++)
        if (key[i] >= floor64) {
            const int at = atomicAdd(cnt, 1);
            if (at < 1024) cand[at] = key[i];  // (distinct keys: at most 64 threads x 16 keys reach the floor)
        }
    __syncthreads();
    const int c = *cnt < 1024 ? *cnt : 1024;  // 64 <= c <= 1024
    int p = 64;
    while (p < c) p <<= 1;
    for (int i = c + t; i < p; i += 256) cand[i] = 0ull;  // below every real key
    __syncthreads();
    for (int k = 2; k <= p; k <<= 1)
        for (int jj = k >> 1; jj > 0; jj >>= 1) {
            for (int i = t; i < p; i += 256) {
                const int l = i ^ jj;
                if (l > i) {
                    const bool up = (i & k) == 0;
                    const u64 a = cand[i], b = cand[l];
                    if (up ? (b > a) : (a > b)) { cand[i] = b; cand[l] = a; }
                }
            }
            __syncthreads();
        }
    if (t < 64) dst[t] = cand[t];
}

// grid (nb, m): slice blk of row j -> its 64 best keys, sorted, at tmp[(j * nb + blk) * 64].
// sel != null: the row holds the logits of sel[0] blocks of 128 outputs, packed; element i belongs to token
// sel[1 + i / 128] * 128 + i % 128 (the packed rows of crates/shadowzero-cuda/src/session.rs:5950-5995, kernels/forward.cu:4635-4657).
static __global__ void __launch_bounds__(256)
sz_topk_slices_kernel(const float* __restrict__ logits, int vocab, int ls, int nb, u64* __restrict__ tmp, const u32* __restrict__ sel) {
    __shared__ __align__(16) u64 sm[256];
    __shared__ u64 cand[1024];
    __shared__ int cnt;
    sz_pdl_wait();
    sz_pdl_trigger();
    const int blk = blockIdx.x, j = blockIdx.y;
    const float* r = logits + (size_t)j * ls;
    const int n = sel ? (int)__ldcg(sel) * 128 : vocab;
    u64 key[16];
#pragma unroll
    for (int q = 0; q < 16; q++) {
        const int i = blk * SZ_TK_N + threadIdx.x + 256 * q;
        const u32 id = sel ? (i < n ? __ldcg(sel + 1 + (i >> 7)) * 128u + (u32)(i & 127) : 0u) : (u32)i;
        key[q] = i < n ? sz_tk_key(__ldcg(r + i), id) : sz_tk_pad(threadIdx.x + 256 * q);
    }
    sz_tk_select(key, sm, cand, &cnt, tmp + ((size_t)j * nb + blk) * 64);
}
// grid (m): out row j = 64 value bit patterns then 64 ids (crates/shadowzero-cuda/src/session.rs:6034-6039); nb * 64 <= 4096
static __global__ void __launch_bounds__(256)
sz_topk_merge_kernel(const u64* __restrict__ tmp, int nb, u32* __restrict__ out) {
    __shared__ __align__(16) u64 sm[256];
    __shared__ u64 cand[1024];
    __shared__ u64 best[64];
    __shared__ int cnt;
    sz_pdl_wait();
    sz_pdl_trigger();
    const int j = blockIdx.x;
    u64 key[16];
#pragma unroll
    for (int q = 0; q < 16; q++) {
        const int i = threadIdx.x + 256 * q;
        key[q] = i < nb * 64 ? __ldcg(tmp + (size_t)j * nb * 64 + i) : sz_tk_pad(i);
        if (sz_tk_is_pad(key[q])) key[q] = sz_tk_pad(i);  // a slice's empty slots: distinct again among all slices
    }
    sz_tk_select(key, sm, cand, &cnt, best);
    __syncthreads();
    if (threadIdx.x < 64) {
        float v; u32 id;
        sz_tk_unkey(best[threadIdx.x], v, id);
        if (sz_tk_is_pad(best[threadIdx.x])) { v = -INFINITY; id = 0xffffffffu; }  // fewer than 64 logits in the row
        out[(size_t)j * 128 + threadIdx.x] = __float_as_uint(v);
        out[(size_t)j * 128 + 64 + threadIdx.x] = id;
    }
}

#endif  // __CUDACC__
