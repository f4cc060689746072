// Weight-format decoders (device).  Layouts: Q8_0 and IQ3_S as ggml defines them (reference decoders:
// crates/shadowzero-model/src/quant.rs:148-159,174-179); EXL3 as crates/shadowzero-model/src/exl3.rs:1-22 describes it.
#pragma once

#include "sz_common.cuh"

#ifdef __CUDACC__

// The IQ3_S codebook in constant memory (for uniform or test access) - kernels that gather from it per lane copy it
// into shared memory first.
__constant__ u32 c_iq3s_grid[512] = {
#include "iq3s_grid.inc"
};

__device__ __forceinline__ u16 sz_ld16(const u8* p) { return *(const u16*)p; }  // p is 2-byte aligned

// ---- Q8_0: 34-byte block = f16 d, 32 x i8 ----------------------------------------------------------------------------------
// weight i of the block at `b` (2-byte aligned): d * q, one f32 multiply (quant.rs:174-179)
__device__ __forceinline__ float sz_q8_0_at(const u8* b, int i) {
    return sz_f16_to_f32(sz_ld16(b)) * (float)(int8_t)b[2 + i];
}

// ---- IQ3_S: 110-byte superblock of 256 weights ---------------------------------------------------------------------------------
// weight e of the superblock at `b`, the operations in the reference's order: (d * (1 + 2 s)) * grid * sign
__device__ __forceinline__ float sz_iq3_s_at(const u8* b, int e, const u32* grid) {
    const float d = sz_f16_to_f32(sz_ld16(b));
    const int j = e >> 2;
    const int idx = b[2 + j] | (((b[66 + (j >> 3)] >> (j & 7)) & 1) << 8);
    const int g = e >> 5;
    const int s = (b[106 + (g >> 1)] >> (4 * (g & 1))) & 15;
    const float db = d * (float)(1 + 2 * s);
    const float mag = (float)((grid[idx] >> (8 * (e & 3))) & 0xff);
    const float v = db * mag;
    return ((b[74 + (e >> 3)] >> (e & 7)) & 1) ? -v : v;
}

// ---- EXL3 -------------------------------------------------------------------------------------------------------------------------
// Codebook "mul1": the four bytes of state * 0x83DCD12D summed onto 0x6400 give an f16 in [1024, 2048); one f16 fma maps it to
// about [-10.4, 10.4] (exl3.rs:84-92).  Returns the f16.
__device__ __forceinline__ __half sz_exl3_cb2_h(u32 state) {
    const u32 x = state * 0x83DCD12Du;
    const u32 sum = __dp4a(x, 0x01010101u, 0x6400u);
    return __hfma(__ushort_as_half((u16)sum), __ushort_as_half((u16)0x1eee), __ushort_as_half((u16)0xc931));
}
__device__ __forceinline__ float sz_exl3_cb2(u32 state) { return __half2float(sz_exl3_cb2_h(state)); }

// A tile of K bits a weight is 8 K u32 words, one cyclic bit stream, most significant bit of word 0 first; weight t's
// 16-bit state ends at bit (t + 1) K.  Lane L decodes weights 8 L .. 8 L + 7, whose windows are consecutive in the ring.
template <int K>
struct SzExl3Tile {
    static constexpr int WORDS = 8 * K;       // u32 words of a tile
    static constexpr int RING = 256 * K;      // bits
    static constexpr int SPAN = 16 + 7 * K;   // bits from the start of window 0 to the end of window 7
    static constexpr int NA = (SPAN + 31) / 32 + 1;  // words of the span once it starts at bit 0, plus one to peek
    static constexpr int NW = NA + 1;                // words loaded: the span at any bit offset

    // What depends on the lane only: the (wrapped) word offsets of its span and the bit offset inside the first word.  A kernel that
    // decodes many tiles computes this once.
    struct Lane { int wi[NW]; int off; };
    __device__ __forceinline__ static Lane lane_setup(int lane) {
        Lane L;
        const int sb = ((8 * lane + 1) * K - 16 + RING) % RING;
        const int w0 = sb >> 5;
        L.off = sb & 31;
#pragma unroll
        for (int i = 0; i < NW; i++) {
            int wi = w0 + i;
            wi = wi >= WORDS ? wi - WORDS : wi;
            wi = wi >= WORDS ? wi - WORDS : wi;
            L.wi[i] = wi;
        }
        return L;
    }
    __device__ __forceinline__ static void states_pre(const u32* tile, const Lane& L, u32* st) {
        u32 w[NW];
#pragma unroll
        for (int i = 0; i < NW; i++) w[i] = tile[L.wi[i]];
        u32 a[NA];
#pragma unroll
        for (int i = 0; i < NA; i++) a[i] = __funnelshift_l(w[i + 1], w[i], L.off);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int pos = j * K;
            const int wi = pos >> 5, sh = pos & 31;
            st[j] = (sh <= 16 ? (a[wi] >> (16 - sh)) : __funnelshift_l(a[wi + 1], a[wi], sh) >> 16) & 0xffffu;
        }
    }

    // the 8 states of lane `lane`; `tile` points at the tile's words (4-byte aligned, any address space)
    __device__ __forceinline__ static void states(const u32* tile, int lane, u32* st) {
        const int sb = ((8 * lane + 1) * K - 16 + RING) % RING;  // first bit of window 0
        const int w0 = sb >> 5, off = sb & 31;
        u32 w[NW];
#pragma unroll
        for (int i = 0; i < NW; i++) {
            int wi = w0 + i;
            wi = wi >= WORDS ? wi - WORDS : wi;
            wi = wi >= WORDS ? wi - WORDS : wi;  // K = 1: the ring (8 words) is shorter than the words peeked
            w[i] = tile[wi];
        }
        // shift the lane's span to bit 0 once, so every window below sits at a compile-time position
        u32 a[NA];
#pragma unroll
        for (int i = 0; i < NA; i++) a[i] = __funnelshift_l(w[i + 1], w[i], off);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int pos = j * K;
            const int wi = pos >> 5, sh = pos & 31;
            st[j] = (sh <= 16 ? (a[wi] >> (16 - sh)) : __funnelshift_l(a[wi + 1], a[wi], sh) >> 16) & 0xffffu;
        }
    }
};

// Position p = 8 L + j of a tile sits at input row 2 (L % 4) + (j & 1) + 8 ((j >> 1) & 1), output column
// (L >> 2) + 8 (j >> 2) (exl3.rs:105-110; 2 (L >> 3) + ((L >> 2) & 1) is L >> 2).
__device__ __forceinline__ int sz_exl3_row(int lane, int j) { return 2 * (lane & 3) + (j & 1) + 8 * ((j >> 1) & 1); }
__device__ __forceinline__ int sz_exl3_col(int lane, int j) { return (lane >> 2) + 8 * (j >> 2); }

// In-place Walsh-Hadamard transform (Sylvester order) of 128 floats spread over a warp: lane L holds v[e] = element L + 32 e.
// Unnormalised; the caller multiplies by 1 / sqrt(128).
__device__ __forceinline__ void sz_wht128_warp(float* v, int lane) {
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float p = __shfl_xor_sync(0xffffffffu, v[e], m);
            v[e] = (lane & m) ? p - v[e] : v[e] + p;
        }
    }
    float a = v[0], b = v[1], c = v[2], d = v[3];
    v[0] = a + b; v[1] = a - b; v[2] = c + d; v[3] = c - d;   // stage h = 32
    a = v[0]; b = v[1]; c = v[2]; d = v[3];
    v[0] = a + c; v[2] = a - c; v[1] = b + d; v[3] = b - d;   // stage h = 64
}
#define SZ_RSQRT128 0.08838835f  // the constant the reference multiplies by (exl3.rs:595)

#endif  // __CUDACC__
