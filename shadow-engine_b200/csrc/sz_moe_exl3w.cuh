// EXL3 expert FFN for a verify pass, warp-specialised streaming form.
//
// Same units, same arithmetic and same fixed-point partial sums as the kernels of sz_moe_exl3.cuh (bit-identical results), another
// division of labour inside a block: eight CONSUMER warps do nothing but decode trellis tiles and issue tensor-core instructions,
// one PRODUCER warp keeps the ring of shared-memory stages full (cp.async.bulk) and prepares each unit's activation fragments.  The
// two sides meet only at mbarriers - a `full` barrier a stage (the copy's bytes have landed and the fragments are written) and an
// `empty` barrier a stage (all eight consumer warps are done with it) - so the consumers never stop at a block-wide barrier and
// never wait for the one thread that issues copies.  The decode itself is leaner: a lane's 8 windows of a tile span two 32-bit
// words at every bit rate this kernel takes (2, 3, 4 bits), so it loads two words instead of four, and the integer byte-sum MMA
// takes its 0x6400 start value from registers that are set once instead of being re-initialised for every tile.
#pragma once

#include "sz_moe_exl3.cuh"

#define SZ_XW_CONSUMERS 8
#define SZ_XW_THREADS (32 * (SZ_XW_CONSUMERS + 1))

// A unit: 8 tile rows (one 128-input block) x 8 TW tile columns (TW a consumer warp).  OCC: blocks a multiprocessor the kernel is
// built for (2 or 3); the ring takes as many stages as fit that share of shared memory, at most 6.
template <int K, int TW, int OCC>
struct SzXW {
    static constexpr int TILE_BYTES = 32 * K;
    static constexpr int ROW_BYTES = 8 * TW * TILE_BYTES;    // one tile row of the unit
    static constexpr int STAGE_BYTES = 8 * ROW_BYTES;        // the unit's trellis bytes
    static constexpr int FRAG_BYTES = 8 * 32 * 16;           // the unit's activation fragments: [8 tile rows][32 lanes] uint4
    static constexpr int BUDGET = (OCC == 3 ? 72 : 108) * 1024;
    static constexpr int FIT = BUDGET / (STAGE_BYTES + FRAG_BYTES);
    static constexpr int STAGES = FIT > 6 ? 6 : FIT;
    static_assert(STAGES >= 2, "the ring needs two stages");
    static constexpr int SMEM_BYTES = STAGES * (STAGE_BYTES + FRAG_BYTES) + 2 * STAGES * 8 + 16;
};

// Two-word form of SzExl3Tile<K>::states_pre: valid when the lane's span (16 + 7 K bits) starting at its bit offset inside the
// first word never crosses into a third word.  sb = first bit of window 0 = ((8 L + 1) K - 16) mod 256 K; for K = 2, 3, 4 the
// offsets sb mod 32 are {2, 18}, {3, 11, 19, 27} and {20}, and offset + span is at most 48, 64 and 64.
template <int K>
struct SzExl3Two {
    static_assert(K == 2 || K == 3 || K == 4, "the span of a lane's windows fits two words for 2, 3 and 4 bits a weight");
    static constexpr int WORDS = 8 * K, RING = 256 * K;
    struct Lane { int w0, w1, off; };
    __device__ __forceinline__ static Lane lane_setup(int lane) {
        Lane L;
        const int sb = ((8 * lane + 1) * K - 16 + RING) % RING;
        L.w0 = sb >> 5;
        L.w1 = L.w0 + 1 >= WORDS ? 0 : L.w0 + 1;
        L.off = sb & 31;
        return L;
    }
    __device__ __forceinline__ static void states(const u32* tile, const Lane& L, u32* st) {
        const u32 w0 = tile[L.w0], w1 = tile[L.w1];
        const u32 a0 = __funnelshift_l(w1, w0, L.off);   // the span from its first bit: 32 bits, then the rest
        const u32 a1 = w1 << L.off;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int pos = j * K;
            if (pos == 0) st[j] = a0 >> 16;
            else if (pos <= 16) st[j] = (a0 >> (16 - pos)) & 0xffffu;
            else st[j] = __funnelshift_l(a1, a0, pos) >> 16;
        }
    }
};

// Byte sums of four products on the integer tensor pipe (see sz_bytesum4), the 0x6400 start value read from `base` (four registers
// that hold it): the accumulator input is a separate operand, so nothing has to be re-initialised per call.
__device__ __forceinline__ void sz_bytesum4c(const u32* x, u32 sel0, u32 sel1, const u32* base, u32* c) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(x[0]), "r"(x[2]), "r"(x[1]), "r"(x[3]), "r"(sel0), "r"(sel1), "r"(base[0]), "r"(base[1]), "r"(base[2]), "r"(base[3]));
}

// What a consumer lane keeps for the whole kernel.
template <int K>
struct SzXWLane {
    typename SzExl3Two<K>::Lane L;
    u32 sel0, sel1;
    u32 base[4];
};
template <int K>
__device__ __forceinline__ SzXWLane<K> sz_xw_lane(int lane) {
    SzXWLane<K> s;
    s.L = SzExl3Two<K>::lane_setup(lane);
    const int n = lane >> 2, q = lane & 3;
    s.sel0 = ((n & 1) == 0 && (n >> 1) == q) ? 0x01010101u : 0u;
    s.sel1 = ((n & 1) == 1 && (n >> 1) == q) ? 0x01010101u : 0u;
    // (an opaque move: the compiler must keep four registers for the accumulator operand rather than re-materialise the constant)
#pragma unroll
    for (int i = 0; i < 4; i++) asm volatile("mov.u32 %0, 0x6400;" : "=r"(s.base[i]));
    return s;
}

// The lane's 8 weights of a tile as the A fragment of m16n8k16 (the same values, bit for bit, as sz_exl3_afrag).
template <int K>
__device__ __forceinline__ void sz_xw_afrag(const u32* tile, const SzXWLane<K>& S, u32* a) {
    u32 st[8];
    SzExl3Two<K>::states(tile, S.L, st);
    const __half2 kinv = __halves2half2(__ushort_as_half((u16)0x1eee), __ushort_as_half((u16)0x1eee));
    const __half2 kbias = __halves2half2(__ushort_as_half((u16)0xc931), __ushort_as_half((u16)0xc931));
    u32 x[8];
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = st[i] * 0x83DCD12Du;
    u32 c[8];
    sz_bytesum4c(x, S.sel0, S.sel1, S.base, c);
    sz_bytesum4c(x + 4, S.sel0, S.sel1, S.base, c + 4);
    u32 p[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const u32 packed = __byte_perm(c[2 * i], c[2 * i + 1], 0x5410);
        const __half2 h = __hfma2(*(const __half2*)&packed, kinv, kbias);
        p[i] = *(const u32*)&h;
    }
    a[0] = p[0]; a[1] = p[2]; a[2] = p[1]; a[3] = p[3];
}

// Decodes and multiplies one staged unit (8 tile rows x 8 NTC tile columns): warp w takes tile columns w NTC .. w NTC + NTC - 1.
// c[tc] = outputs (w NTC + tc) 16 + {g, g + 8} for rows 2 q, 2 q + 1.
// The decode loop is fully unrolled: rolled over the tile rows it ran 6% slower, and moving the byte-sum packing or the
// word-crossing windows from the ALU pipe to multiply-adds on the FMA pipe another 2 - 4% slower (measured on the benchmark's shape).
template <int K, int TW>
__device__ __forceinline__ void sz_xw_compute(const u8* stage, const uint4* frag, int warp, int lane, const SzXWLane<K>& S, float (*c)[4]) {
#pragma unroll
    for (int tc = 0; tc < TW; tc++) { c[tc][0] = 0.f; c[tc][1] = 0.f; c[tc][2] = 0.f; c[tc][3] = 0.f; }
    const u8* wbase = stage + (size_t)(warp * TW) * (32 * K);
    const uint4* fl = frag + lane;
#pragma unroll
    for (int kr = 0; kr < 8; kr++) {
        const uint4 b = fl[kr * 32];
#pragma unroll
        for (int tc = 0; tc < TW; tc++) {
            const u32* tile = (const u32*)(wbase + (size_t)(kr * 8 * TW + tc) * (32 * K));
            u32 a[4];
            sz_xw_afrag<K>(tile, S, a);
            sz_mma16816(c[tc], a, b.x, b.y);
            sz_mma16816(c[tc], a, b.z, b.w);
        }
    }
}

__device__ __forceinline__ void sz_mbar_arrive(u64* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sz_smem_addr(bar)) : "memory");
}

// One warp writes the B fragments of one row (see sz_x3_store_frag: the same layout, any warp may write any row t).
__device__ __forceinline__ void sz_xw_store_row(uint4* frag, int t, float* v, int lane) {
    sz_wht128_warp(v, lane);
    const int kk = lane & 15;
    const int q = (kk & 7) >> 1, reg = kk >> 3, half = kk & 1;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const float val = v[e] * SZ_RSQRT128;
        const __half hi = __float2half_rn(val);
        const __half lo = __float2half_rn(val - __half2float(hi));
        const int kr = 2 * e + (lane >> 4);
        u16* dst = (u16*)(frag + kr * 32 + 4 * t + q);
        dst[reg * 2 + half] = __half_as_ushort(hi);
        dst[4 + reg * 2 + half] = __half_as_ushort(lo);
    }
}
__device__ __forceinline__ void sz_xw_zero_row(uint4* frag, int t, int lane) {
    frag[(lane >> 2) * 32 + 4 * t + (lane & 3)] = make_uint4(0, 0, 0, 0);
}

// What the producer and the consumers of both kernels share: the stage ring and its barriers.
template <int K, int TW, int OCC>
struct SzXWRing {
    using X = SzXW<K, TW, OCC>;
    u8* stages;
    uint4* frags;
    u64 *full, *empty;
    __device__ __forceinline__ void init(u8* smem) {
        stages = smem;
        frags = (uint4*)(smem + X::STAGES * X::STAGE_BYTES);
        full = (u64*)(smem + X::STAGES * (X::STAGE_BYTES + X::FRAG_BYTES));
        empty = full + X::STAGES;
        if (threadIdx.x == 0) {
            for (int i = 0; i < X::STAGES; i++) { sz_mbar_init(&full[i], 2); sz_mbar_init(&empty[i], SZ_XW_CONSUMERS); }
            sz_mbar_fence_init();
        }
    }
    // lane 0 of the producer: the unit's 8 tile rows, `row_stride` bytes apart in the matrix, into stage st
    __device__ __forceinline__ void issue(int st, const u8* src, u64 row_stride) {
        u8* dst = stages + (size_t)st * X::STAGE_BYTES;
        sz_mbar_expect_tx(&full[st], X::STAGE_BYTES);
        if (row_stride == (u64)X::ROW_BYTES) {
            sz_bulk_g2s(dst, src, X::STAGE_BYTES, &full[st]);
        } else {
#pragma unroll
            for (int kr = 0; kr < 8; kr++) sz_bulk_g2s(dst + kr * X::ROW_BYTES, src + kr * row_stride, X::ROW_BYTES, &full[st]);
        }
    }
};

// The consumers' epilogue: the unit's partial sums into the fixed-point accumulators of the group's pairs.
template <int TW>
__device__ __forceinline__ void sz_xw_flush(const SzPlan* plan, int g, int D, int m, int top_k, long long* base, size_t pair_stride, int col0,
                                            int lane, const float (*c)[4]) {
    const int q = lane & 3, g8 = lane >> 2;
    int n, pair0;
    const u8* pairs;
    if (g < D) { n = plan->count[g]; pairs = plan->pairs[g]; pair0 = 0; }
    else { n = m; pairs = nullptr; pair0 = m * top_k; }
#pragma unroll
    for (int tt = 0; tt < 2; tt++) {
        const int t = 2 * q + tt;
        if (t < n) {
            const int pair = pairs ? pairs[t] : pair0 + t;
            long long* dst = base + (size_t)pair * pair_stride + col0 + g8;
#pragma unroll
            for (int tc = 0; tc < TW; tc++) {
                sz_fix_add(dst + tc * 16, c[tc][tt]);
                sz_fix_add(dst + tc * 16 + 8, c[tc][2 + tt]);
            }
        }
    }
}

// ---- gate / up --------------------------------------------------------------------------------------------------------------------
// Units: group x {gate, up} x input block x column chunk (8 TW tile columns of the FF / 16), the chunk fastest: the chunks of one
// input block share their activation fragments (made for the first, copied for the others).  A block takes a contiguous share of
// the units.  acc: i64 [pairs][2][FF], zero on entry.
template <int K, int NTC, int TW, int OCC>
__global__ void __launch_bounds__(SZ_XW_THREADS, OCC)
sz_xw_gateup_kernel(const SzPlan* __restrict__ plan, const u8* __restrict__ gate, u64 gstride, const u8* __restrict__ up, u64 ustride,
                    const u8* __restrict__ sh_gate, const u8* __restrict__ sh_up, const float* __restrict__ x, int m, int H, int top_k,
                    long long* __restrict__ acc, u32* __restrict__ ctrl, long long win_x, long long win_acc) {
    using X = SzXW<K, TW, OCC>;
    constexpr int FF = 128 * NTC, S = X::STAGES, NCH = NTC / TW;
    // grid.y > 1: block row w works on plan w of an array of plans, with its own inputs and sums (win_x, win_acc: elements from one
    // window's to the next's); a window without groups is left at once
    if (gridDim.y > 1) {
        plan += blockIdx.y; x += blockIdx.y * win_x; acc += blockIdx.y * win_acc;
        if (plan->n_groups == 0 && !sh_gate) return;
    }
    static_assert(NTC % TW == 0, "column chunks tile the matrix");
    extern __shared__ __align__(128) u8 smem[];
    SzXWRing<K, TW, OCC> R;
    R.init(smem);
    __shared__ __align__(16) SzPlan splan;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    sz_pdl_wait();
    sz_pdl_trigger();
    plan = sz_plan_stage(plan, &splan);
    __syncthreads();
    const int D = plan ? plan->n_groups : 0;
    const int NG = D + (sh_gate ? 1 : 0);
    const int NS = H / 128;
    const long long U = (long long)NG * 2 * NS * NCH;
    const int u0 = (int)(U * blockIdx.x / gridDim.x), u1 = (int)(U * (blockIdx.x + 1) / gridDim.x);
    const int count = u1 - u0;
    if (count <= 0) return;
    const size_t hdr = 2 * (size_t)H + 2 * (size_t)FF + 4;
    const u64 mrow = (u64)(8 * NTC) * X::TILE_BYTES;    // bytes of one tile row of the matrix
    int failed = 0;
    if (warp == SZ_XW_CONSUMERS) {
        // ---- producer: copies and fragments of unit i into stage i % S
        int prev_key = -1, prev_st = 0;
        // the unit's (group, matrix, input block, column chunk): divided out once, then stepped (the units of a block follow one another)
        int key = u0 / NCH, ch = u0 - key * NCH;                  // key = (g, mat, s)
        int g = key / (2 * NS), mat, s;
        { const int rem = key - g * 2 * NS; mat = rem / NS; s = rem - mat * NS; }
        for (int i = 0; i < count; i++) {
            const int st = i % S;
            if (i > 0) {
                if (++ch == NCH) { ch = 0; key++; if (++s == NS) { s = 0; if (++mat == 2) { mat = 0; g++; } } }
            }
            if (i >= S && !sz_mbar_wait(&R.empty[st], ((i / S) - 1) & 1)) { failed = 1; break; }
            const u8* blob;
            int n;
            const u8* rows;
            if (g < D) {
                const u64 e = (u64)plan->expert[g];
                blob = mat ? up + e * ustride : gate + e * gstride;
                n = plan->count[g]; rows = plan->rows[g];
            } else {
                blob = mat ? sh_up : sh_gate;
                n = m; rows = nullptr;
            }
            if (lane == 0) R.issue(st, blob + hdr + (size_t)s * 8 * mrow + (size_t)ch * X::ROW_BYTES, mrow);
            uint4* frag = R.frags + st * 256;
            if (key == prev_key) {
                const uint4* from = R.frags + prev_st * 256;   // that stage is still intact: its `empty` wait lies ahead of this warp
#pragma unroll
                for (int e = 0; e < 8; e++) frag[lane + 32 * e] = from[lane + 32 * e];
            } else {
                const u16* suh = (const u16*)blob + s * 128;
                float sc[4];
#pragma unroll
                for (int e = 0; e < 4; e++) sc[e] = sz_f16_to_f32(__ldg(suh + lane + 32 * e));
                // every row's loads are in flight before the first is used (a row at a time would pay the L2 latency once a row)
                float v[8][4];
#pragma unroll
                for (int t = 0; t < 8; t++) {
                    if (t < n) {
                        const int row = rows ? rows[t] : t;
#pragma unroll
                        for (int e = 0; e < 4; e++) v[t][e] = __ldg(x + (size_t)row * H + s * 128 + lane + 32 * e);
                    }
                }
#pragma unroll
                for (int t = 0; t < 8; t++) {
                    if (t < n) {
#pragma unroll
                        for (int e = 0; e < 4; e++) v[t][e] *= sc[e];
                        sz_xw_store_row(frag, t, v[t], lane);
                    } else {
                        sz_xw_zero_row(frag, t, lane);
                    }
                }
            }
            prev_key = key; prev_st = st;
            __syncwarp();
            if (lane == 0) sz_mbar_arrive(&R.full[st]);   // (release: the warp's fragment stores are ordered before it by the __syncwarp)
        }
    } else {
        // ---- consumers
        const SzXWLane<K> LS = sz_xw_lane<K>(lane);
        int key = u0 / NCH, ch = u0 - key * NCH;
        int g = key / (2 * NS), mat, s;
        { const int rem = key - g * 2 * NS; mat = rem / NS; s = rem - mat * NS; }
        for (int i = 0; i < count; i++) {
            const int st = i % S;
            if (i > 0) {
                if (++ch == NCH) { ch = 0; if (++s == NS) { s = 0; if (++mat == 2) { mat = 0; g++; } } }
            }
            if (!sz_mbar_wait(&R.full[st], (i / S) & 1)) { failed = 1; break; }
            float c[TW][4];
            sz_xw_compute<K, TW>(R.stages + (size_t)st * X::STAGE_BYTES, R.frags + st * 256, warp, lane, LS, c);
            __syncwarp();
            if (lane == 0) sz_mbar_arrive(&R.empty[st]);
            sz_xw_flush<TW>(plan, g, D, m, top_k, acc + (size_t)mat * FF, (size_t)2 * FF, (ch * 8 * TW + warp * TW) * 16, lane, c);
        }
    }
    if (failed && lane == 0) atomicExch(&ctrl[1], 1u);
}

// ---- down ---------------------------------------------------------------------------------------------------------------------------
// Units: group x input block (128 of FF) x output chunk (8 TW tile columns of the H / 16), the chunk fastest; 8 tile rows, strided.
// The input of a unit is the SwiGLU product of its pairs, finished by the producer warp from the gate / up sums: rotate back (H),
// scale by svh, silu(g) * u, then into the down trellis' basis (suh, H); the chunks of one (group, input block) follow one another
// and share it, so it is computed for the first and copied for the others.  out: i64 [pairs][H], zero on entry.
template <int K, int TW, int OCC>
__global__ void __launch_bounds__(SZ_XW_THREADS, OCC)
sz_xw_down_kernel(const SzPlan* __restrict__ plan, const u8* __restrict__ gate, u64 gstride, const u8* __restrict__ up, u64 ustride,
                  const u8* __restrict__ down, u64 dstride, const u8* __restrict__ sh_gate, const u8* __restrict__ sh_up,
                  const u8* __restrict__ sh_down, int m, int H, int FF, int top_k, const long long* __restrict__ acc,
                  long long* __restrict__ out, u32* __restrict__ ctrl, long long win_acc, long long win_out) {
    using X = SzXW<K, TW, OCC>;
    constexpr int S = X::STAGES;
    if (gridDim.y > 1) {   // (as the gate / up kernel)
        plan += blockIdx.y; acc += blockIdx.y * win_acc; out += blockIdx.y * win_out;
        if (plan->n_groups == 0 && !sh_down) return;
    }
    extern __shared__ __align__(128) u8 smem[];
    SzXWRing<K, TW, OCC> R;
    R.init(smem);
    __shared__ __align__(16) SzPlan splan;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the plan was finished two kernels ago (the kernel before this one waited for it before it let this one start): it can be read,
    // and the first copies issued, ahead of the wait; only the gate / up sums need the wait
    plan = sz_plan_stage(plan, &splan);
    __syncthreads();
    const int D = plan ? plan->n_groups : 0;
    const int NG = D + (sh_down ? 1 : 0);
    const int KB = FF / 128, NC = H / (128 * TW);
    const long long U = (long long)NG * KB * NC;
    const int u0 = (int)(U * blockIdx.x / gridDim.x), u1 = (int)(U * (blockIdx.x + 1) / gridDim.x);
    const int count = u1 - u0;
    const size_t hdr_d = 2 * (size_t)FF + 2 * (size_t)H + 4;
    const u64 drow = (u64)(H / 16) * X::TILE_BYTES;  // bytes of one tile row of the down matrix
    int failed = 0;
    if (warp == SZ_XW_CONSUMERS) {
        auto blobs = [&](int g, const u8** bg, const u8** bu, const u8** bd) {
            if (g < D) {
                const u64 e = (u64)plan->expert[g];
                *bg = gate + e * gstride; *bu = up + e * ustride; *bd = down + e * dstride;
            } else {
                *bg = sh_gate; *bu = sh_up; *bd = sh_down;
            }
        };
        auto issue = [&](int i) {   // lane 0: the row copies of the block's i-th unit
            const int u = u0 + i;
            const int g = u / (KB * NC), rem = u - g * KB * NC, kb = rem / NC, c = rem - kb * NC;
            const u8 *bg, *bu, *bd;
            blobs(g, &bg, &bu, &bd);
            R.issue(i % S, bd + hdr_d + (size_t)kb * 8 * drow + (size_t)c * X::ROW_BYTES, drow);
        };
        const int pre = count < S ? count : S;
        if (lane == 0)
            for (int i = 0; i < pre; i++) issue(i);
        sz_pdl_wait();
        sz_pdl_trigger();
        int prev_g = -1, prev_kb = -1, prev_st = 0;
        for (int i = 0; i < count; i++) {
            const int u = u0 + i, st = i % S;
            if (i >= S) {
                if (!sz_mbar_wait(&R.empty[st], ((i / S) - 1) & 1)) { failed = 1; break; }
                if (lane == 0) issue(i);
            }
            const int g = u / (KB * NC), rem = u - g * KB * NC, kb = rem / NC;
            uint4* frag = R.frags + st * 256;
            if (g == prev_g && kb == prev_kb) {
                const uint4* from = R.frags + prev_st * 256;   // the same input as the unit before: a copy (that stage is still intact: its
                                                                // `empty` wait lies ahead of this warp)
#pragma unroll
                for (int e = 0; e < 8; e++) frag[lane + 32 * e] = from[lane + 32 * e];
            } else {
                const u8 *bg, *bu, *bd;
                blobs(g, &bg, &bu, &bd);
                int n, pair0;
                const u8* pairs;
                if (g < D) { n = plan->count[g]; pairs = plan->pairs[g]; pair0 = 0; }
                else { n = m; pairs = nullptr; pair0 = m * top_k; }
                const u16* svg = (const u16*)(bg + 2 * (size_t)H) + kb * 128;
                const u16* svu = (const u16*)(bu + 2 * (size_t)H) + kb * 128;
                const u16* suh = (const u16*)bd + kb * 128;
                float sc[12];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int idx = lane + 32 * e;
                    sc[e] = sz_f16_to_f32(__ldg(svg + idx));
                    sc[4 + e] = sz_f16_to_f32(__ldg(svu + idx));
                    sc[8 + e] = sz_f16_to_f32(__ldg(suh + idx));
                }
                for (int t = 0; t < 8; t++) {
                    if (t < n) {
                        const int pair = pairs ? pairs[t] : pair0 + t;
                        const long long* a = acc + (size_t)pair * 2 * FF + kb * 128;
                        float gg[4], uu[4], v[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            gg[e] = (float)((double)__ldcg(a + lane + 32 * e) * SZ_FIX_INV);
                            uu[e] = (float)((double)__ldcg(a + FF + lane + 32 * e) * SZ_FIX_INV);
                        }
                        sz_wht128_warp(gg, lane);
                        sz_wht128_warp(uu, lane);
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float gv = (gg[e] * SZ_RSQRT128) * sc[e], uv = (uu[e] * SZ_RSQRT128) * sc[4 + e];
                            v[e] = (sz_silu(gv) * uv) * sc[8 + e];
                        }
                        sz_xw_store_row(frag, t, v, lane);
                    } else {
                        sz_xw_zero_row(frag, t, lane);
                    }
                }
            }
            prev_g = g; prev_kb = kb; prev_st = st;
            __syncwarp();
            if (lane == 0) sz_mbar_arrive(&R.full[st]);
        }
    } else {
        sz_pdl_wait();
        sz_pdl_trigger();
        const SzXWLane<K> LS = sz_xw_lane<K>(lane);
        int g = u0 / (KB * NC), kb, cc;   // (divided out once, then stepped, as in the gate / up kernel)
        { const int rem = u0 - g * KB * NC; kb = rem / NC; cc = rem - kb * NC; }
        for (int i = 0; i < count; i++) {
            const int st = i % S;
            if (i > 0) {
                if (++cc == NC) { cc = 0; if (++kb == KB) { kb = 0; g++; } }
            }
            if (!sz_mbar_wait(&R.full[st], (i / S) & 1)) { failed = 1; break; }
            float c[TW][4];
            sz_xw_compute<K, TW>(R.stages + (size_t)st * X::STAGE_BYTES, R.frags + st * 256, warp, lane, LS, c);
            __syncwarp();
            if (lane == 0) sz_mbar_arrive(&R.empty[st]);
            sz_xw_flush<TW>(plan, g, D, m, top_k, out, (size_t)H, (cc * 8 * TW + warp * TW) * 16, lane, c);
        }
    }
    if (failed && lane == 0) atomicExch(&ctrl[1], 1u);
}
