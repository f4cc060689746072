// The output projection over an EXL3 output.weight, with the reference's 2-bit screening proxy ("Q2_P") and sparse rescore:
//   rotate the rows of the pass into the trellis' basis and quantise them to int8 per 128-block        (kernels/exl3.cu:609-625,
//                                                                                                     kernels/forward.cu:4369-4420)
//   score every output against a 2-bit copy of the rotated weights, keep each 128-output block's best  (forward.cu:4428-4495)
//   keep the k best blocks of every row of the pass, their union as an ascending list                 (forward.cu:4536-4632)
//   evaluate only those blocks from the real EXL3 weights                                             (exl3.cu:349-480, SPARSE)
//   top-64 over the packed logits                                                                      (forward.cu:4635-4680)
// The proxy itself is built once from the weights (exl3.cu:915-987).  Everything up to the block list is integer or ordered f32
// arithmetic and is bit-for-bit what the CPU restatement computes; the logits come from the same tensor-core decode as the experts.
#pragma once

#include "sz_moe_exl3.cuh"
#include "sz_topk.cuh"

#ifdef __CUDACC__

#define SZ_HEAD_PICK_KEYS 8  // keys a thread of the pick kernel holds: 256 * 8 = 2048 blocks = 262144 outputs at most

// ---- the proxy, once: 128 x 128 blocks of W_rot = H_out(W_hat) * svh / 128 as 2-bit codes {-3, -1, 1, 3} * scale ------------------------
// grid (n_ob, n_b), 256 threads; warp w decodes tile column w of the block, one tile row at a time.
// w_q2: uint4 [(ob * 2 n_b + 2 b + hb) * 128 + r], word wi, bits (bi * 8 + sl * 2) = code of input hb * 64 + wi * 16 + sl * 4 + bi;
// w_sc: f16 [(ob * n_b + b) * 128 + r] = half the quantiser's step.
template <int K>
static __global__ void __launch_bounds__(256)
sz_head_build_kernel(const u8* __restrict__ blob, int rows, int cols, u8* __restrict__ w_q2, u16* __restrict__ w_sc) {
    __shared__ float ws[16][132];
    __shared__ u16 wh[128][132];
    const int ob = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_b = cols >> 7, nt = rows >> 4;
    const u16* svh = (const u16*)(blob + 2 * (size_t)cols);
    const u32* tr = (const u32*)(blob + 2 * (size_t)cols + 2 * (size_t)rows + 4);
    for (int kk = 0; kk < 8; kk++) {
        const u32* tile = tr + ((size_t)(b * 8 + kk) * nt + ob * 8 + warp) * (8 * K);
        u32 st[8];
        SzExl3Tile<K>::states(tile, lane, st);
#pragma unroll
        for (int j = 0; j < 8; j++) ws[sz_exl3_row(lane, j)][warp * 16 + sz_exl3_col(lane, j)] = sz_exl3_cb2(st[j]);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int r_in = warp + 8 * u;
            float rv[4];
#pragma unroll
            for (int e = 0; e < 4; e++) rv[e] = ws[r_in][lane + 32 * e];
            sz_wht128_warp(rv, lane);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int c_out = lane + 32 * e;
                const float val = __fmul_rn(__fmul_rn(rv[e], 0.0078125f), sz_f16_to_f32(svh[ob * 128 + c_out]));
                wh[c_out][kk * 16 + r_in] = __half_as_ushort(__float2half_rn(val));
            }
        }
        __syncthreads();
    }
    if (tid < 128) {
        const int r = tid;
        float sq = 0.0f;
        for (int c = 0; c < 128; c++) {
            const float fv = sz_f16_to_f32(wh[r][c]);
            sq = __fmaf_rn(fv, fv, sq);
        }
        const float delta = __fmul_rn(0.9957f, __fsqrt_rn(__fmul_rn(sq, 0.0078125f)));
        const u16 sh = __half_as_ushort(__float2half_rn(__fmul_rn(0.5f, delta)));
        const float thr = 2.0f * sz_f16_to_f32(sh);
        w_sc[((size_t)ob * n_b + b) * 128 + r] = sh;
        for (int hb = 0; hb < 2; hb++) {
            u32 words[4];
#pragma unroll
            for (int wi = 0; wi < 4; wi++) {
                const int c0 = hb * 64 + wi * 16;
                u32 pw = 0;
#pragma unroll
                for (int sl = 0; sl < 4; sl++)
#pragma unroll
                    for (int bi = 0; bi < 4; bi++) {
                        const float fv = sz_f16_to_f32(wh[r][c0 + sl * 4 + bi]);
                        const u32 q = (fv >= 0.0f) ? (fv >= thr ? 3u : 2u) : (fv <= -thr ? 0u : 1u);
                        pw |= q << (bi * 8 + sl * 2);
                    }
                words[wi] = pw;
            }
            ((uint4*)w_q2)[((size_t)ob * (n_b * 2) + b * 2 + hb) * 128 + r] = make_uint4(words[0], words[1], words[2], words[3]);
        }
    }
}

// ---- rows of the pass into the trellis' basis, and their int8 form ---------------------------------------------------------------------
// A warp a (row, 128-block): xr = H(x * suh), not normalised.  With `quant`: codes q = round(xr / sc), sc = max|xr| / 127, four to a
// word in element order; x_sc = sc; x_corr = -3 sc sum(q) (the proxy's codes are 0..3 for the levels -3, -1, 1, 3).
static __global__ void __launch_bounds__(256)
sz_head_rotate_kernel(const u8* __restrict__ blob, const float* __restrict__ x, int xs, int cols, int m, float* __restrict__ xr,
                      u32* __restrict__ xq, float* __restrict__ x_sc, float* __restrict__ x_corr, int quant) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_b = cols >> 7;
    const int job = blockIdx.x * 8 + warp;
    const bool live = job < m * n_b;
    const int j = live ? job / n_b : 0, b = live ? job % n_b : 0;
    float s[4];
#pragma unroll
    for (int e = 0; e < 4; e++) s[e] = sz_f16_to_f32(__ldg((const u16*)blob + b * 128 + lane + 32 * e));  // weights: ahead of the wait
    sz_pdl_wait();
    sz_pdl_trigger();
    if (!live) return;
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; e++) v[e] = __fmul_rn(__ldcg(x + (size_t)j * xs + b * 128 + lane + 32 * e), s[e]);
    sz_wht128_warp(v, lane);
#pragma unroll
    for (int e = 0; e < 4; e++) xr[(size_t)j * cols + b * 128 + lane + 32 * e] = v[e];
    if (!quant) return;
    float am = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, off));
    const float sc = am > 0.0f ? __fdiv_rn(am, 127.0f) : 0.0f;
    const float inv = sc > 0.0f ? __fdiv_rn(1.0f, sc) : 0.0f;
    int tot = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int q = __float2int_rn(fmaxf(-127.0f, fminf(127.0f, __fmul_rn(v[e], inv))));
        tot += q;
        const u32 byte = (u32)q & 0xffu;
        const u32 b0 = __shfl_sync(0xffffffffu, byte, (lane & ~3) | 0), b1 = __shfl_sync(0xffffffffu, byte, (lane & ~3) | 1);
        const u32 b2 = __shfl_sync(0xffffffffu, byte, (lane & ~3) | 2), b3 = __shfl_sync(0xffffffffu, byte, (lane & ~3) | 3);
        if ((lane & 3) == 0) xq[((size_t)j * n_b + b) * 32 + (lane >> 2) + 8 * e] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    }
    tot = __reduce_add_sync(0xffffffffu, tot);
    if (lane == 0) {
        x_sc[(size_t)j * n_b + b] = sc;
        x_corr[(size_t)j * n_b + b] = __fmul_rn(__fmul_rn(-3.0f, (float)tot), sc);
    }
}

// ---- the screen: bmax[j][ob] = the best proxy score of block ob's 128 outputs for row j ----------------------------------------------------
// grid n_ob, 128 threads (thread = output), dynamic shared memory m * n_b * (128 + 8) bytes.  The integer dot products of a 128-block
// are exact; the f32 sum over the blocks runs in block order with the reference's two fused multiply-adds a block.
template <int M>
static __global__ void __launch_bounds__(128)
sz_head_proxy_kernel(const u8* __restrict__ w_q2, const u16* __restrict__ w_sc, const u32* __restrict__ xq, const float* __restrict__ x_sc,
                     const float* __restrict__ x_corr, float* __restrict__ bmax, int n_ob, int cols, int m) {
    extern __shared__ __align__(16) u8 smem_raw[];
    const int n_b = cols >> 7;
    int* s_xq = (int*)smem_raw;                       // [m][n_b * 32]
    float* s_sc2 = (float*)(s_xq + (size_t)m * n_b * 32);  // [m][n_b]: 2 * x_sc
    float* s_corr = s_sc2 + m * n_b;                  // [m][n_b]
    __shared__ float s_wmax[4][M];
    const int ob = blockIdx.x, tid = threadIdx.x;
    const uint4* wq = (const uint4*)w_q2 + (size_t)ob * (n_b * 2) * 128 + tid;
    const u16* ws = w_sc + (size_t)ob * n_b * 128 + tid;
    const uint4 first0 = sz_ldg16_here(wq), first1 = sz_ldg16_here(wq + 128);  // the weights do not depend on the pass
    sz_pdl_wait();
    sz_pdl_trigger();
    for (int i = tid; i < m * n_b * 32; i += 128) s_xq[i] = (int)__ldcg(xq + i);
    for (int i = tid; i < m * n_b; i += 128) { s_sc2[i] = 2.0f * __ldcg(x_sc + i); s_corr[i] = __ldcg(x_corr + i); }
    __syncthreads();
    float acc[M];
#pragma unroll
    for (int j = 0; j < M; j++) acc[j] = 0.0f;
#pragma unroll 2
    for (int b = 0; b < n_b; b++) {
        uint4 qw[2];
        qw[0] = b == 0 ? first0 : __ldg(wq + (size_t)(b * 2) * 128);
        qw[1] = b == 0 ? first1 : __ldg(wq + (size_t)(b * 2 + 1) * 128);
        const float wsc = sz_f16_to_f32(__ldg(ws + (size_t)b * 128));
        int ia[M];
#pragma unroll
        for (int j = 0; j < M; j++) ia[j] = 0;
#pragma unroll
        for (int hb = 0; hb < 2; hb++) {
            const u32 words[4] = {qw[hb].x, qw[hb].y, qw[hb].z, qw[hb].w};
#pragma unroll
            for (int wi = 0; wi < 4; wi++) {
                const u32 w = words[wi];
                const int u0 = (int)(w & 0x03030303u), u1 = (int)((w >> 2) & 0x03030303u);
                const int u2 = (int)((w >> 4) & 0x03030303u), u3 = (int)((w >> 6) & 0x03030303u);
                const int xbase = b * 32 + hb * 16 + wi * 4;
#pragma unroll
                for (int j = 0; j < M; j++) {
                    if (M == 1 || j < m) {
                        const int4 xv = *(const int4*)(s_xq + (size_t)j * n_b * 32 + xbase);
                        ia[j] = __dp4a(xv.x, u0, ia[j]);   // the codes are 0..3: the signed form gives the unsigned product
                        ia[j] = __dp4a(xv.y, u1, ia[j]);
                        ia[j] = __dp4a(xv.z, u2, ia[j]);
                        ia[j] = __dp4a(xv.w, u3, ia[j]);
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < M; j++)
            if (M == 1 || j < m) acc[j] = __fmaf_rn(wsc, __fmaf_rn(s_sc2[j * n_b + b], (float)ia[j], s_corr[j * n_b + b]), acc[j]);
    }
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
    for (int j = 0; j < M; j++) {
        float mx = acc[j];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (lane == 0) s_wmax[warp][j] = mx;
    }
    __syncthreads();
    if (tid < M && tid < m) bmax[(size_t)tid * n_ob + ob] = fmaxf(fmaxf(s_wmax[0][tid], s_wmax[1][tid]), fmaxf(s_wmax[2][tid], s_wmax[3][tid]));
}

// ---- the block list: the k best blocks of every row (value descending, index ascending, NaN below everything), their union ascending --------
// grid m, 256 threads.  A row's k-th best key is found bit by bit (the largest threshold that k keys still reach: a count a bit);
// every key at or above it sets its block's bit in `seen`.  The last block to finish (a ticket in ctrl[0]) turns the bits into
// sel[1 ..], sel[0] = how many (at most max_sel), and clears bits and ticket for the next pass.
static __global__ void __launch_bounds__(256)
sz_head_pick_kernel(const float* __restrict__ bmax, int n_ob, int k_use, int max_sel, u32* __restrict__ seen, u32* __restrict__ ctrl,
                    u32* __restrict__ sel) {
    __shared__ int cnts[2][8];
    __shared__ int offs[64];
    __shared__ int s_last;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    sz_pdl_wait();
    sz_pdl_trigger();
    const float* r = bmax + (size_t)blockIdx.x * n_ob;
    u64 key[SZ_HEAD_PICK_KEYS];
#pragma unroll
    for (int q = 0; q < SZ_HEAD_PICK_KEYS; q++) {
        const int i = t + 256 * q;
        float v = i < n_ob ? __ldcg(r + i) : 0.0f;
        if (v != v) v = -3.0e38f;
        key[q] = i < n_ob ? sz_tk_key(v, (u32)i) : 0ull;  // 0 is below every real key
    }
    const int k = k_use < n_ob ? k_use : n_ob;
    // every real key has bits 31..12 set (block numbers are below 4096): the threshold keeps them set and the search covers the rest
    u64 T = 0x00000000fffff000ull;
    int it = 0;
    for (int bit = 63; bit >= 0; bit--) {
        if (bit < 32 && bit >= 12) continue;
        const u64 cand = T | (1ull << bit);
        int c = 0;
#pragma unroll
        for (int q = 0; q < SZ_HEAD_PICK_KEYS; q++) c += key[q] >= cand;
        c = __reduce_add_sync(0xffffffffu, c);
        if (lane == 0) cnts[it & 1][warp] = c;
        __syncthreads();
        int tot = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) tot += cnts[it & 1][w];
        if (tot >= k) T = cand;
        it++;
    }
#pragma unroll
    for (int q = 0; q < SZ_HEAD_PICK_KEYS; q++)
        if (key[q] >= T && key[q] != 0ull) {
            const u32 i = (u32)(t + 256 * q);
            atomicOr(&seen[i >> 5], 1u << (i & 31));
        }
    __threadfence();
    __syncthreads();
    if (t == 0) s_last = atomicAdd(&ctrl[0], 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int n_words = (n_ob + 31) >> 5;  // at most 64
    u32 mask = 0;
    if (t < n_words) mask = atomicExch(&seen[t], 0u);
    if (t < 64) offs[t] = __popc(mask);
    __syncthreads();
    int pos = 0, total = 0;
    for (int w = 0; w < 64; w++) {
        const int c = offs[w];
        pos += w < t ? c : 0;
        total += c;
    }
    if (t < n_words)
        while (mask) {
            const int bit = __ffs((int)mask) - 1;
            mask &= mask - 1;
            if (pos < max_sel) sel[1 + pos] = (u32)(t * 32 + bit);
            pos++;
        }
    if (t == 0) {
        sel[0] = (u32)(total < max_sel ? total : max_sel);
        ctrl[0] = 0;
    }
}

// ---- the logits of whole 128-output blocks from the EXL3 weights -----------------------------------------------------------------------------
// A block of 8 warps takes one 128-output block (sel: the slot-th block of the list; null: block number = slot) and walks the input
// in 128-blocks: a unit is 8 tile rows of 8 tiles, one tile column a warp, fetched by bulk copies into a ring of stages while the
// previous ones are decoded (a tile is the A fragment of mma.m16n8k16, the rows of the pass are the B operand in f16 high and low
// parts, as for the experts).  The whole input range belongs to one block, so the sums stay in registers; the output rotation, the
// 1/sqrt(128) and svh follow, and row j's 128 logits go to logits[j * ls + slot * 128 ..].
// The decode of two tiles in lockstep (the steps of sz_exl3_afrag, written alternately): a warp issues in order, so the second tile's
// step fills the wait for the first's result.  The asm statements are not volatile: pure functions of their inputs, free to move.
__device__ __forceinline__ void sz_mma16816_free(float* c, const u32* a, u32 b0, u32 b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void sz_bytesum4_free(const u32* x, u32 sel0, u32 sel1, u32* c) {
    c[0] = 0x6400u; c[1] = 0x6400u; c[2] = 0x6400u; c[3] = 0x6400u;
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(x[0]), "r"(x[2]), "r"(x[1]), "r"(x[3]), "r"(sel0), "r"(sel1));
}
template <int K>
__device__ __forceinline__ void sz_exl3_afrag2(const u32* tileA, const u32* tileB, int lane, const typename SzExl3Tile<K>::Lane& LS, u32* aA, u32* aB) {
    u32 sA[8], sB[8];
    SzExl3Tile<K>::states_pre(tileA, LS, sA);
    SzExl3Tile<K>::states_pre(tileB, LS, sB);
    const __half2 kinv = __halves2half2(__ushort_as_half((u16)0x1eee), __ushort_as_half((u16)0x1eee));
    const __half2 kbias = __halves2half2(__ushort_as_half((u16)0xc931), __ushort_as_half((u16)0xc931));
    const int n = lane >> 2, q = lane & 3;
    const u32 sel0 = ((n & 1) == 0 && (n >> 1) == q) ? 0x01010101u : 0u;
    const u32 sel1 = ((n & 1) == 1 && (n >> 1) == q) ? 0x01010101u : 0u;
#pragma unroll
    for (int i = 0; i < 8; i++) { sA[i] *= 0x83DCD12Du; sB[i] *= 0x83DCD12Du; }
    u32 cA[8], cB[8];
    sz_bytesum4_free(sA, sel0, sel1, cA);
    sz_bytesum4_free(sB, sel0, sel1, cB);
    sz_bytesum4_free(sA + 4, sel0, sel1, cA + 4);
    sz_bytesum4_free(sB + 4, sel0, sel1, cB + 4);
    u32 pA[4], pB[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const u32 ka = __byte_perm(cA[2 * i], cA[2 * i + 1], 0x5410), kb = __byte_perm(cB[2 * i], cB[2 * i + 1], 0x5410);
        const __half2 ha = __hfma2(*(const __half2*)&ka, kinv, kbias), hb = __hfma2(*(const __half2*)&kb, kinv, kbias);
        pA[i] = *(const u32*)&ha;
        pB[i] = *(const u32*)&hb;
    }
    aA[0] = pA[0]; aA[1] = pA[2]; aA[2] = pA[1]; aA[3] = pA[3];
    aB[0] = pB[0]; aB[1] = pB[2]; aB[2] = pB[1]; aB[3] = pB[3];
}

// MC = how many rows of the pass have B-fragment columns in shared memory (4 or 8): a pass of at most four rows keeps half the
// fragments, which lets a third block share the multiprocessor.
template <int K, int MC>
struct SzHeadX {
    using X = SzX3<K, 1>;
    static constexpr int OUT_BYTES = 8 * 128 * 4;
    static constexpr int FRAG_UNIT = 8 * 4 * MC;  // uint4 entries of one input block: 8 tile rows x (4 lanes a row of the pass)
    static size_t smem_bytes(int n_b) { return (size_t)SZ_X3_STAGES * X::STAGE_BYTES + (size_t)n_b * FRAG_UNIT * 16 + OUT_BYTES + SZ_X3_STAGES * 8 + 16; }
};

template <int K, int MC>
static __global__ void __launch_bounds__(SZ_X3_THREADS)
sz_head_exl3_kernel(const u8* __restrict__ blob, int rows, int cols, const float* __restrict__ xr, int m, const u32* __restrict__ sel,
                    float* __restrict__ logits, int ls, u32* __restrict__ err) {
    using X = SzX3<K, 1>;
    using HX = SzHeadX<K, MC>;
    static_assert(SZ_X3_STAGES == 4, "the loop below takes the ring two stages at a time");
    extern __shared__ __align__(128) u8 smem[];
    const int n_b = cols >> 7, nt = rows >> 4;
    u8* stages = smem;
    uint4* frags = (uint4*)(smem + SZ_X3_STAGES * X::STAGE_BYTES);                                  // [n_b][8 tile rows][4 MC]
    float* outs = (float*)(smem + SZ_X3_STAGES * X::STAGE_BYTES + (size_t)n_b * HX::FRAG_UNIT * 16);   // [8 rows][128]
    u64* bars = (u64*)((u8*)outs + HX::OUT_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < SZ_X3_STAGES; i++) sz_mbar_init(&bars[i], 1);
        sz_mbar_fence_init();
    }
    sz_pdl_wait();
    sz_pdl_trigger();
    const int slot = blockIdx.x;
    if (sel && slot >= (int)__ldcg(sel)) return;
    const int ob = sel ? (int)__ldcg(sel + 1 + slot) : slot;
    const u8* tr = blob + 2 * (size_t)cols + 2 * (size_t)rows + 4;
    const u64 drow = (u64)nt * X::TILE_BYTES;  // bytes between tile rows
    __syncthreads();                           // the barriers are initialised
    auto issue = [&](int i) {                  // thread 0: input block i into stage i % STAGES
        u64* bar = &bars[i % SZ_X3_STAGES];
        u8* dst = stages + (size_t)(i % SZ_X3_STAGES) * X::STAGE_BYTES;
        const u8* src = tr + (size_t)i * 8 * drow + (size_t)ob * X::ROW_BYTES;
        sz_mbar_expect_tx(bar, X::STAGE_BYTES);
#pragma unroll
        for (int kr = 0; kr < 8; kr++) sz_bulk_g2s(dst + kr * X::ROW_BYTES, src + kr * drow, X::ROW_BYTES, bar);
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < 2 && i < n_b; i++) issue(i);
    // warp t: row t of the pass, already rotated, as B fragments of every input block (rows beyond the pass are zero columns)
    if (warp < MC) {
        for (int b = 0; b < n_b; b++) {
            uint4* frag = frags + (size_t)b * HX::FRAG_UNIT;
            if (warp < m) {
                const int kk = lane & 15;
                const int q = (kk & 7) >> 1, reg = kk >> 3, half = kk & 1;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float val = __ldcg(xr + (size_t)warp * cols + b * 128 + lane + 32 * e) * SZ_RSQRT128;
                    const __half hi = __float2half_rn(val);
                    const __half lo = __float2half_rn(val - __half2float(hi));
                    const int kr = 2 * e + (lane >> 4);
                    u16* dst = (u16*)(frag + kr * (4 * MC) + 4 * warp + q);
                    dst[reg * 2 + half] = __half_as_ushort(hi);
                    dst[4 + reg * 2 + half] = __half_as_ushort(lo);
                }
            } else {
                frag[(lane >> 2) * (4 * MC) + 4 * warp + (lane & 3)] = make_uint4(0, 0, 0, 0);
            }
        }
    }
    __syncthreads();
    const typename SzExl3Tile<K>::Lane LS = SzExl3Tile<K>::lane_setup(lane);
    const bool has_b = lane < 4 * MC;   // lanes whose column of the B operand belongs to a row held in shared memory
    auto bfrag = [&](int unit, int kr) { return has_b ? frags[(size_t)unit * HX::FRAG_UNIT + kr * (4 * MC) + lane] : make_uint4(0, 0, 0, 0); };
    float accA[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f};
    int failed = 0;
    // two input blocks a round, decoded side by side into accumulators of their own: twice the independent work in flight a warp
    for (int i = 0; i < n_b; i += 2) {
        const bool two = i + 1 < n_b;
        if (threadIdx.x == 0) {  // the stages the previous round left
            if (i + 2 < n_b) issue(i + 2);
            if (i + 3 < n_b) issue(i + 3);
        }
        if (!sz_mbar_wait(&bars[i % SZ_X3_STAGES], (i / SZ_X3_STAGES) & 1)) failed = 1;
        if (two && !sz_mbar_wait(&bars[(i + 1) % SZ_X3_STAGES], ((i + 1) / SZ_X3_STAGES) & 1)) failed = 1;
        if (!failed) {
            const u8* sA = stages + (size_t)(i % SZ_X3_STAGES) * X::STAGE_BYTES + (size_t)warp * X::TILE_BYTES;
            const u8* sB = stages + (size_t)((i + 1) % SZ_X3_STAGES) * X::STAGE_BYTES + (size_t)warp * X::TILE_BYTES;
            if (two) {
#pragma unroll
                for (int kr = 0; kr < 8; kr++) {
                    const uint4 bA = bfrag(i, kr), bB = bfrag(i + 1, kr);
                    u32 aA[4], aB[4];
                    sz_exl3_afrag2<K>((const u32*)(sA + (size_t)kr * X::ROW_BYTES), (const u32*)(sB + (size_t)kr * X::ROW_BYTES), lane, LS, aA, aB);
                    sz_mma16816_free(accA, aA, bA.x, bA.y);
                    sz_mma16816_free(accB, aB, bB.x, bB.y);
                    sz_mma16816_free(accA, aA, bA.z, bA.w);
                    sz_mma16816_free(accB, aB, bB.z, bB.w);
                }
            } else {
#pragma unroll
                for (int kr = 0; kr < 8; kr++) {
                    const uint4 bA = bfrag(i, kr);
                    u32 aA[4];
                    sz_exl3_afrag<K>((const u32*)(sA + (size_t)kr * X::ROW_BYTES), lane, LS, aA);
                    sz_mma16816(accA, aA, bA.x, bA.y);
                    sz_mma16816(accA, aA, bA.z, bA.w);
                }
            }
        }
        if (__syncthreads_or(failed)) { failed = 1; break; }
    }
    if (failed) {
        if (threadIdx.x == 0) atomicExch(err, 1u);
        return;
    }
    {   // c0 = (output g, row 2q), c1 = (output g, row 2q + 1), c2 = (output g + 8, row 2q), c3 = (output g + 8, row 2q + 1)
        const int g = lane >> 2, q = lane & 3;
        outs[(2 * q) * 128 + warp * 16 + g] = accA[0] + accB[0];
        outs[(2 * q + 1) * 128 + warp * 16 + g] = accA[1] + accB[1];
        outs[(2 * q) * 128 + warp * 16 + g + 8] = accA[2] + accB[2];
        outs[(2 * q + 1) * 128 + warp * 16 + g + 8] = accA[3] + accB[3];
    }
    __syncthreads();
    if (warp < m) {
        const u16* svh = (const u16*)(blob + 2 * (size_t)cols) + (size_t)ob * 128;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = outs[warp * 128 + lane + 32 * e];
        sz_wht128_warp(v, lane);
#pragma unroll
        for (int e = 0; e < 4; e++)
            logits[(size_t)warp * ls + (size_t)slot * 128 + lane + 32 * e] = (v[e] * SZ_RSQRT128) * sz_f16_to_f32(__ldg(svh + lane + 32 * e));
    }
}

#endif  // __CUDACC__
