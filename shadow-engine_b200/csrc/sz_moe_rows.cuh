// The MoE sublayer over MANY rows (a prompt chunk, or the verify rows of many sequences): what sz_moe_verify computes for up to 8
// rows, for up to SZ_ROWS_MAX, with every expert's matrices decoded ONCE for all the rows that chose it.  The role of the reference's
// grouped experts of a long prompt (device planner plan_scan_w / plan_fill_w, kernels/forward.cu:3234-3319; mma_grouped*,
// kernels/matvec.cu:1190-1260; EXL3 exl3_mma, kernels/exl3.cu:500-590) with this library's exact kernels: the expert kernels are
// the verify pass's own (sz_xw_gateup_kernel, sz_xw_down_kernel), a window a block row of their grids.
//
//   route     sz_route_kernel with a second grid dimension: 8 rows a block row, same arithmetic as a verify pass
//   plan      sz_rows_plan_kernel: every expert's rows (ascending), cut into groups of up to 8 rows, groups packed into WINDOWS of at
//             most 80 groups and 256 (row, rank) pairs - the sizes one SzPlan holds.  A pair's place is (window, slot).
//   gather    sz_rows_gather_kernel: xg[window][slot] = the pair's input row (a window's rows are then indexed by a byte)
//   experts   one gate/up and one down launch, block row w over window w's plan, input and accumulators
//   shared    the shared expert as windows of their own: groups of 8 consecutive rows, expert 0 of a one-matrix "layer"
//   combine   sz_rows_combine_kernel: per (row, 128 outputs) the ranks' terms in rank order, as sz_x3_combine_kernel adds them
// A pair's numbers do not depend on which rows share its group (every row of a group is a column of its own in the tensor-core
// product, the sums over column blocks are integer): a row's output is bit for bit what sz_moe_verify gives for it.
#pragma once
#include "sz_moe.cuh"

#define SZ_ROWS_MAX 256           // rows a call (a multiple of 8): an expert's rows then always fit one window
#define SZ_ROWS_WIN 20            // windows of routed experts a call can need (2,560 pairs = 10 full windows; cuts waste some room)
#define SZ_ROWS_SHWIN 1           // windows of the shared expert (256 rows = 32 groups of 8)
#define SZ_ROWS_SLOTS 256         // pairs a window

struct SzRowsPlan {
    int32_t n_windows, n_sh_windows, overflow, pad;
    SzPlan win[SZ_ROWS_WIN + SZ_ROWS_SHWIN];                     // routed windows, then the shared expert's
    int32_t src[SZ_ROWS_WIN + SZ_ROWS_SHWIN][SZ_ROWS_SLOTS];     // slot -> input row (-1: unused)
    int32_t pair_loc[SZ_ROWS_MAX * SZ_MAX_TOPK];                 // pair (row * top_k + rank) -> window * 256 + slot
};

// ---- one block of 1024 threads -------------------------------------------------------------------------------------------------------
// Every (row, rank) pair marks its row in its expert's row mask (256 bits); an expert's pairs in ascending row order are then the
// set bits of its mask, and a pair's place among them the number of set bits below its row: no sorting, no order of arrival.
__global__ void __launch_bounds__(1024)
sz_rows_plan_kernel(const int32_t* __restrict__ ridx, int R, int k, int ne, int has_shared, SzRowsPlan* __restrict__ P) {
    __shared__ u32 mask[SZ_MAX_EXPERTS][SZ_ROWS_MAX / 32];
    __shared__ short win_of[SZ_MAX_EXPERTS], grp_of[SZ_MAX_EXPERTS], slot_of[SZ_MAX_EXPERTS], cnt[SZ_MAX_EXPERTS];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int t = threadIdx.x, pairs = R * k;
    for (int i = t; i < ne * (SZ_ROWS_MAX / 32); i += 1024) (&mask[0][0])[i] = 0u;
    for (int i = t; i < (SZ_ROWS_WIN + SZ_ROWS_SHWIN) * SZ_ROWS_SLOTS; i += 1024) P->src[i / SZ_ROWS_SLOTS][i % SZ_ROWS_SLOTS] = -1;
    __syncthreads();
    for (int p = t; p < pairs; p += 1024) {
        const int e = __ldcg(ridx + p), row = p / k;
        if ((unsigned)e >= (unsigned)ne) continue;     // (a routing that was never written: caught below, nothing is touched)
        atomicOr(&mask[e][row >> 5], 1u << (row & 31));
    }
    __syncthreads();
    for (int e = t; e < ne; e += 1024) {
        int c = 0;
#pragma unroll
        for (int q = 0; q < SZ_ROWS_MAX / 32; q++) c += __popc(mask[e][q]);
        cnt[e] = (short)c;
    }
    __syncthreads();
    if (t == 0) {
        // experts in ascending order into windows: an expert's rows (at most R <= 256) stay in one window, as groups of up to 8
        int w = 0, g = 0, s = 0, over = 0;
        for (int e = 0; e < ne; e++) {
            const int c = cnt[e];
            if (c == 0) { win_of[e] = -1; continue; }
            const int ng = (c + 7) / 8;
            if (g + ng > SZ_MAXG || s + c > SZ_ROWS_SLOTS) {
                if (w < SZ_ROWS_WIN) P->win[w].n_groups = g;
                w++; g = 0; s = 0;
            }
            if (w >= SZ_ROWS_WIN) { over = 1; win_of[e] = -1; continue; }
            win_of[e] = (short)w; grp_of[e] = (short)g; slot_of[e] = (short)s;
            g += ng; s += c;
        }
        if (w < SZ_ROWS_WIN) { P->win[w].n_groups = g; w++; }
        P->n_windows = w < SZ_ROWS_WIN ? w : SZ_ROWS_WIN;
        for (int q = P->n_windows; q < SZ_ROWS_WIN; q++) P->win[q].n_groups = 0;
        P->win[SZ_ROWS_WIN].n_groups = has_shared ? (R + 7) / 8 : 0;
        P->n_sh_windows = has_shared ? 1 : 0;
        P->overflow = over;
    }
    __syncthreads();
    for (int p = t; p < pairs; p += 1024) {
        const int e = __ldcg(ridx + p), row = p / k;
        if ((unsigned)e >= (unsigned)ne) { P->pair_loc[p] = 0; P->overflow = 4; continue; }   // an expert id out of range: the call is reported as failed
        const int w = win_of[e];
        if (w < 0) { P->pair_loc[p] = 0; continue; }
        int n = __popc(mask[e][row >> 5] & ((1u << (row & 31)) - 1u));
        for (int q = 0; q < (row >> 5); q++) n += __popc(mask[e][q]);
        const int c = cnt[e];
        const int slot = slot_of[e] + n, grp = grp_of[e] + n / 8, in = n % 8;
        SzPlan& W = P->win[w];
        W.rows[grp][in] = (uint8_t)slot;
        W.pairs[grp][in] = (uint8_t)slot;
        if (in == 0) { W.expert[grp] = (int16_t)e; W.count[grp] = (uint8_t)(c - n < 8 ? c - n : 8); }
        P->src[w][slot] = row;
        P->pair_loc[p] = w * SZ_ROWS_SLOTS + slot;
    }
    if (has_shared)   // the shared expert: the rows in order, 8 a group; its pair of row r is slot r of the last window
        for (int r = t; r < R; r += 1024) {
            SzPlan& W = P->win[SZ_ROWS_WIN];
            W.rows[r / 8][r % 8] = (uint8_t)r;
            W.pairs[r / 8][r % 8] = (uint8_t)r;
            if (r % 8 == 0) { W.expert[r / 8] = 0; W.count[r / 8] = (uint8_t)(R - r < 8 ? R - r : 8); }
            P->src[SZ_ROWS_WIN][r] = r;
        }
}

// ---- grid (slots, windows), block 256: xg[window][slot][:] = x[src] (nothing for an unused slot) ---------------------------------
__global__ void __launch_bounds__(256)
sz_rows_gather_kernel(const float* __restrict__ x, int H, const SzRowsPlan* __restrict__ P, float* __restrict__ xg) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int s = blockIdx.x, w = blockIdx.y;
    const int r = P->src[w][s];
    if (r < 0) return;
    const float4* src = (const float4*)(x + (size_t)r * H);
    float4* dst = (float4*)(xg + ((size_t)w * SZ_ROWS_SLOTS + s) * H);
    for (int i = threadIdx.x; i < H / 4; i += 256) dst[i] = __ldcg(src + i);
}

// ---- combine: grid (rows * H / 128), block (top_k + 1) warps ---------------------------------------------------------------------------
// y[j] = sum over ranks of w * (H eo * svh) + sigmoid(shared gate logit) * (H so * svh_shared), term by term as sz_x3_combine_kernel:
// warp t finishes rank t's term (warp top_k: the shared expert's), warp 0 adds them in rank order in f64.  out: the windows' down
// accumulators, i64 [window][slot][H].
__global__ void __launch_bounds__((SZ_MAX_TOPK + 1) * 32)
sz_rows_combine_kernel(const long long* __restrict__ out, const SzRowsPlan* __restrict__ P, const int32_t* __restrict__ ridx, const double* __restrict__ rw,
                       const u8* __restrict__ down, u64 dstride, const u8* __restrict__ sh_down, const float* __restrict__ logits, int ne, int top_k,
                       int H, int FF, int SF, int has_shared, float* __restrict__ y) {
    __shared__ float part[SZ_MAX_TOPK + 1][128];
    __shared__ double rws[SZ_MAX_TOPK];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = H / 128;
    const int j = blockIdx.x / nb, b = blockIdx.x % nb;
    if (warp < top_k) {
        const int pair = j * top_k + warp;
        int e = __ldcg(ridx + pair);
        e = (unsigned)e < (unsigned)ne ? e : 0;
        const u16* svh = (const u16*)(down + (u64)e * dstride + 2 * (size_t)FF) + b * 128;
        const int loc = P->pair_loc[pair];
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) v[q] = (float)((double)__ldcg(out + (size_t)loc * H + b * 128 + lane + 32 * q) * SZ_FIX_INV);
        sz_wht128_warp(v, lane);
#pragma unroll
        for (int q = 0; q < 4; q++) part[warp][lane + 32 * q] = (v[q] * SZ_RSQRT128) * sz_f16_to_f32(svh[lane + 32 * q]);
        if (lane == 0) rws[warp] = __ldcg(rw + pair);
    } else if (warp == top_k && has_shared) {
        const float sg = sz_sigmoid(__ldcg(logits + (size_t)j * (ne + 1) + ne));
        const u16* svh = (const u16*)(sh_down + 2 * (size_t)SF) + b * 128;
        const size_t loc = (size_t)SZ_ROWS_WIN * SZ_ROWS_SLOTS + j;
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) v[q] = (float)((double)__ldcg(out + loc * H + b * 128 + lane + 32 * q) * SZ_FIX_INV);
        sz_wht128_warp(v, lane);
#pragma unroll
        for (int q = 0; q < 4; q++) part[top_k][lane + 32 * q] = sg * ((v[q] * SZ_RSQRT128) * sz_f16_to_f32(svh[lane + 32 * q]));
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int i = lane + 32 * e;
            double a = 0.0;
            for (int t = 0; t < top_k; t++) a += rws[t] * (double)part[t][i];
            if (has_shared) a += (double)part[top_k][i];
            y[(size_t)j * H + b * 128 + i] = (float)a;
        }
    }
}
