// The MoE sublayer of a verify pass for 1..8 rows: router + plan, grouped expert FFN, weighted combine.
// Arithmetic follows Session::moe of the CPU reference (crates/shadowzero-model/src/forward.rs:1009-1034): router logits and
// the softmax in f64, expert dot products accumulated in f32, the weighted sum over experts in f64 in rank order.
#include "sz_moe.cuh"
#include "sz_moe_exl3w.cuh"
#include "sz_moe_blk.cuh"
#include "sz_moe_rows.cuh"

#include <float.h>
#include <stdlib.h>

// ---------------------------------------------------------------------------------------------------------------------------------
// router: logits (a warp a router row, f64 accumulate), then the last block to finish does softmax, top-k and the plan

#define SZ_ROUTE_RB 4        // router rows a block
#define SZ_ROUTE_THREADS 256

// orderable 32-bit image of a float: a > b  <=>  key(a) > key(b) for every pair of non-NaN values (-0 sorts below +0, which cannot
// matter here: the values are logit - max, and a tie in value is decided by the index)
__device__ __forceinline__ u32 sz_fkey(float v) {
    const u32 u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float sz_fkey_inv(u32 k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

// Sums N = 2^h values a lane over the 32 lanes of a warp.  While more than one value is left, a step at offset o halves them: the
// lanes with bit o set keep the upper half and send the lower, the others the reverse, so N + N/2 + .. shuffles do the work of
// 5 N.  Afterwards every lane holds the total of value number lane >> (5 - h) in v[0].
template <int N>
__device__ __forceinline__ void sz_warp_sum_many(double* v, int lane) {
    int n = N;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        if (n > 1) {
            const int half = n >> 1;
            const bool up = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < N / 2; i++) {
                if (i < half) {
                    const double send = up ? v[i] : v[i + half];
                    const double keep = up ? v[i + half] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            n = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
        }
    }
}

// grid: ceil(rows / 4) blocks of 256 threads.  A block takes 4 router rows (row ne: the shared expert's gate); its threads split the
// hidden dimension: thread t holds the float4 pieces t, t + 256, .. of every one of the 4 rows (fetched before the dependency
// wait) and of the M rows of the pass, so nothing is staged in shared memory and every product is formed and added in f64 with one
// conversion a weight.  The 4 x M partial sums a thread ends with are summed over the warp (sz_warp_sum_many), then over the 8 warps
// in warp order.  M: rows of the pass; MP: M rounded up to a power of two; NCH: float4 pieces a thread holds per row.
template <int M, int MP, int NCH>
__global__ void __launch_bounds__(SZ_ROUTE_THREADS)
sz_route_kernel(const float* __restrict__ x, int H, const float* __restrict__ router, const float* __restrict__ shared_router,
                int ne, int k, float* __restrict__ logits, int32_t* __restrict__ ridx, double* __restrict__ rw, SzPlan* __restrict__ plan,
                SzPlan* __restrict__ plan_sh, u32* __restrict__ ctrl, int32_t* __restrict__ out_idx, double* __restrict__ out_w,
                uint4* __restrict__ zero, int zero_n, int ep_first, int ep_count) {
    constexpr int RB = SZ_ROUTE_RB, N = RB * MP;
    __shared__ double part[SZ_ROUTE_THREADS / 32][N];
    __shared__ u32 rowmask[SZ_MAX_EXPERTS];     // which rows of the pass chose expert e
    __shared__ u32 bitmap[SZ_MAX_EXPERTS / 32]; // experts chosen at all (and held here)
    __shared__ int sel[SZ_MAX_VERIFY * SZ_MAX_TOPK];
    __shared__ int s_last;
    __shared__ float tk_red[SZ_ROUTE_THREADS / 32];
    __shared__ u64 tk_max[SZ_ROUTE_THREADS];
    __shared__ u64 tk_floor[SZ_MAX_VERIFY];
    __shared__ int tk_cnt[SZ_MAX_VERIFY];
    __shared__ u64 tk_cand[MP][SZ_MAX_TOPK * (SZ_MAX_EXPERTS / (SZ_ROUTE_THREADS / MP))];
    __shared__ double tk_ex[SZ_MAX_VERIFY][SZ_MAX_TOPK];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int ld = ne + 1;
    const int nrows = ne + (shared_router != nullptr ? 1 : 0);
    const int row0 = blockIdx.x * RB;
    // grid.y > 1 (sz_moe_rows): block row y routes rows y * M .. of a longer batch, with tables and a ticket of its own
    if (gridDim.y > 1) {
        const size_t cy = blockIdx.y;
        x += cy * M * H; logits += cy * M * ld; ridx += cy * M * k; rw += cy * M * k; plan += cy; plan_sh += cy; ctrl += cy * 16;
        if (out_idx) out_idx += cy * M * k;
        if (out_w) out_w += cy * M * k;
    }
    SZ_PH_DECL;
    SZ_PH();  // 0 start
    // the router rows do not depend on the previous kernel: fetched before waiting for it
    float4 w[RB][NCH];
#pragma unroll
    for (int r = 0; r < RB; r++) {
        const int row = row0 + r;
        const float4* wrow = (const float4*)(row < ne ? router + (size_t)row * H : shared_router);
#pragma unroll
        for (int u = 0; u < NCH; u++) {
            w[r][u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < nrows && t + 256 * u < H / 4) {
                const uint4 q = sz_ldg16_here(wrow + t + 256 * u);
                w[r][u] = make_float4(__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w));
            }
        }
    }
    for (int i = t; i < SZ_MAX_EXPERTS; i += SZ_ROUTE_THREADS) rowmask[i] = 0u;
    if (t < SZ_MAX_EXPERTS / 32) bitmap[t] = 0u;
    sz_pdl_wait();
    sz_pdl_trigger();
    SZ_PH();  // 1 after wait
    float4 xv[M][NCH];
#pragma unroll
    for (int j = 0; j < M; j++)
#pragma unroll
        for (int u = 0; u < NCH; u++)
            xv[j][u] = t + 256 * u < H / 4 ? __ldcg((const float4*)(x + (size_t)j * H) + t + 256 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
    // the streaming kernels' fixed-point accumulators start every call at zero
    for (int i = blockIdx.x * blockDim.x + t; i < zero_n; i += gridDim.x * blockDim.x) zero[i] = make_uint4(0, 0, 0, 0);

    // ---- logits: f64 products, f64 sums
    double acc[N];
#pragma unroll
    for (int i = 0; i < N; i++) acc[i] = 0.0;
#pragma unroll
    for (int u = 0; u < NCH; u++) {
        double xd[M][4];
#pragma unroll
        for (int j = 0; j < M; j++) { xd[j][0] = (double)xv[j][u].x; xd[j][1] = (double)xv[j][u].y; xd[j][2] = (double)xv[j][u].z; xd[j][3] = (double)xv[j][u].w; }
#pragma unroll
        for (int r = 0; r < RB; r++) {
            const double w0 = (double)w[r][u].x, w1 = (double)w[r][u].y, w2 = (double)w[r][u].z, w3 = (double)w[r][u].w;
#pragma unroll
            for (int j = 0; j < M; j++) {
                double a = acc[r * MP + j];
                a = fma(w0, xd[j][0], a);
                a = fma(w1, xd[j][1], a);
                a = fma(w2, xd[j][2], a);
                a = fma(w3, xd[j][3], a);
                acc[r * MP + j] = a;
            }
        }
    }
    SZ_PH();  // 2 products
    constexpr int HB = N == 1 ? 0 : (N == 2 ? 1 : (N == 4 ? 2 : (N == 8 ? 3 : (N == 16 ? 4 : 5))));  // log2(N), N <= 32
    sz_warp_sum_many<N>(acc, lane);
    if ((lane & ((32 >> HB) - 1)) == 0) part[warp][lane >> (5 - HB)] = acc[0];
    __syncthreads();
    if (t < N) {
        double s = 0.0;
#pragma unroll
        for (int q = 0; q < SZ_ROUTE_THREADS / 32; q++) s += part[q][t];
        const int r = t / MP, j = t % MP;
        if (j < M && row0 + r < nrows) logits[(size_t)j * ld + row0 + r] = (float)s;
    }

    // ---- the last block to arrive routes every row
    SZ_PH();  // 3 logits done
    __threadfence();
    __syncthreads();
    if (t == 0) s_last = (atomicAdd(&ctrl[0], 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    SZ_PH();  // 4 ticket taken

    // ---- top-k of every row, all rows at once: G = 256 / MP threads a row, a thread owns the experts g, g + G, ..  The k-th best of
    // the G per-thread maxima is a floor under the k-th best logit, so only values at or above it (at most k threads' worth, typically
    // a dozen) can be chosen; those are ranked by counting.  Keys are (orderable f32 image of logit - max, ~index): one unsigned
    // comparison orders by value descending, then index ascending.  Every loop is a short rolled loop.
    {
        constexpr int G = SZ_ROUTE_THREADS / MP;          // threads a row
        constexpr int NK = SZ_MAX_EXPERTS / G;            // most keys a thread owns
        const int j = t / G, g = t % G;
        const bool live_row = j < M;
        float lv[NK];
        float mxv = -FLT_MAX;  // f32::MIN, forward.rs:1093
#pragma unroll
        for (int q = 0; q < NK; q++) {
            const int e = g + G * q;
            lv[q] = (live_row && e < ne) ? __ldcg(logits + (size_t)j * ld + e) : -INFINITY;
            if (live_row && e < ne) mxv = fmaxf(mxv, lv[q]);
        }
        // the row's maximum: over the thread's values, the warp, then the warps of the row
        for (int o = 16; o > 0; o >>= 1) mxv = fmaxf(mxv, __shfl_xor_sync(0xffffffffu, mxv, o));
        if (lane == 0) tk_red[warp] = mxv;
        __syncthreads();
        constexpr int WPR = G / 32 > 0 ? G / 32 : 1;      // warps a row
        mxv = tk_red[(t / 32 / WPR) * WPR];
        for (int q = 1; q < WPR; q++) mxv = fmaxf(mxv, tk_red[(t / 32 / WPR) * WPR + q]);
        u64 key[NK];
        u64 best = 0ull;
#pragma unroll
        for (int q = 0; q < NK; q++) {
            const int e = g + G * q;
            key[q] = (live_row && e < ne) ? (((u64)sz_fkey(lv[q] - mxv) << 32) | (u64)(0xffffffffu - (u32)e)) : 0ull;  // in f32, as the reference
            best = key[q] > best ? key[q] : best;
        }
        tk_max[t] = best;
        if (g == 0) tk_cnt[j] = 0;
        __syncthreads();
        int rank = 0;
#pragma unroll 4
        for (int i = 0; i < G; i++) rank += tk_max[j * G + i] > best;
        if (live_row && rank == k - 1) tk_floor[j] = best;   // keys are distinct, so exactly one thread has this rank
        __syncthreads();
        const u64 fl = live_row ? tk_floor[j] : ~0ull;
#pragma unroll
        for (int q = 0; q < NK; q++)
            if (key[q] >= fl && key[q] != 0ull) tk_cand[j][atomicAdd(&tk_cnt[j], 1)] = key[q];
        __syncthreads();
        const int C = live_row ? tk_cnt[j] : 0;              // k <= C <= k * NK
        for (int i = g; i < C; i += G) {
            const u64 mine = tk_cand[j][i];
            int r = 0;
#pragma unroll 4
            for (int q = 0; q < C; q++) r += tk_cand[j][q] > mine;
            if (r < k) {
                const int e = (int)(0xffffffffu - (u32)mine);
                sel[j * SZ_MAX_TOPK + r] = e;
                ridx[j * k + r] = e;
                if (out_idx) out_idx[j * k + r] = e;
                tk_ex[j][r] = exp((double)sz_fkey_inv((u32)(mine >> 32)));
            }
        }
        __syncthreads();
        // weights: softmax over all experts, then the chosen ones renormalised - the full sum cancels, so only the k chosen
        // exponentials are needed: w_r = exp(d_r) / sum over ranks (in rank order) of exp(d_r')
        if (live_row && g < k) {
            double tz = 0.0;
            for (int r = 0; r < k; r++) tz += tk_ex[j][r];
            const double wv = tk_ex[j][g] / tz;
            rw[j * k + g] = wv;
            if (out_w) out_w[j * k + g] = wv;
        }
    }
    __syncthreads();
    SZ_PH();  // 5 rows routed

    // ---- plan: groups in ascending expert order, rows ascending inside a group.  Each (row, rank) pair marks its expert in a bitmap
    // and its row in the expert's row mask; a group's index is then the number of marked experts below it and a pair's place in the
    // group the number of lower rows in the mask.  With expert parallelism only the experts this rank holds enter the plan; routing
    // itself is the same on every rank.
    const int pairs = M * k;
    const int e_lo = ep_count > 0 ? ep_first : 0, e_hi = ep_count > 0 ? ep_first + ep_count : ne;
    int e = -1, j = 0;
    if (t < pairs) {
        j = t / k;
        e = sel[j * SZ_MAX_TOPK + t % k];
        if (e < e_lo || e >= e_hi) e = -1;
        if (e >= 0) { atomicOr(&rowmask[e], 1u << j); atomicOr(&bitmap[e >> 5], 1u << (e & 31)); }
    }
    __syncthreads();
    if (e >= 0) {
        int g = __popc(bitmap[e >> 5] & ((1u << (e & 31)) - 1u));
        for (int q = 0; q < (e >> 5); q++) g += __popc(bitmap[q]);
        const u32 rm = rowmask[e];
        const int pos = __popc(rm & ((1u << j) - 1u));
        plan->rows[g][pos] = j;
        plan->pairs[g][pos] = t;
        if (pos == 0) { plan->expert[g] = e; plan->count[g] = __popc(rm); }
    }
    if (t == 0) {
        int n = 0;
        for (int q = 0; q < SZ_MAX_EXPERTS / 32; q++) n += __popc(bitmap[q]);
        plan->n_groups = n;
    }
    // the shared expert: one group holding every row; its per-pair buffers are indexed by row
    if (t < SZ_MAX_VERIFY) {
        plan_sh->rows[0][t] = t;
        plan_sh->pairs[0][t] = t;
    }
    if (t == 0) {
        plan_sh->n_groups = 1;
        plan_sh->expert[0] = 0;
        plan_sh->count[0] = M;
        ctrl[0] = 0;  // ready for the next call
        ctrl[2] = 0;  // the unit counters of the streaming expert kernels
        ctrl[3] = 0;
    }
    SZ_PH();  // 6 plan written
    SZ_PH_FLUSH(0, true);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// block formats (Q8_0, IQ3_S): a warp a matrix row, a lane four consecutive weights of every 128

// Adds to acc[j] the lane's share of row . xs[j] for j < N.  `row`: the matrix row's bytes (2-byte aligned); xs: shared, [N][cols].
template <int TYPE, int N>
__device__ __forceinline__ void sz_row_dot(const u8* __restrict__ row, int cols, const float* xs, const u32* grid, int lane, float* acc) {
    for (int e = 4 * lane; e < cols; e += 128) {
        float w0, w1, w2, w3, scale;
        if (TYPE == SZ_TYPE_Q8_0) {
            const u8* blk = row + (e >> 5) * 34;
            const int i = e & 31;
            scale = sz_f16_to_f32(sz_ld16(blk));
            const u32 q01 = sz_ld16(blk + 2 + i), q23 = sz_ld16(blk + 4 + i);
            w0 = (float)(int8_t)(q01 & 0xff); w1 = (float)(int8_t)(q01 >> 8);
            w2 = (float)(int8_t)(q23 & 0xff); w3 = (float)(int8_t)(q23 >> 8);
        } else {
            const u8* blk = row + (e >> 8) * 110;
            const int jj = (e & 255) >> 2;  // group of four inside the superblock
            const int idx = blk[2 + jj] | (((blk[66 + (jj >> 3)] >> (jj & 7)) & 1) << 8);
            const int g = jj >> 3;
            const int s = (blk[106 + (g >> 1)] >> (4 * (g & 1))) & 15;
            scale = sz_f16_to_f32(sz_ld16(blk)) * (float)(1 + 2 * s);
            const u32 mags = grid[idx];
            const u32 sg = blk[74 + (jj >> 1)] >> (4 * (jj & 1));
            w0 = (float)(mags & 0xff); w1 = (float)((mags >> 8) & 0xff); w2 = (float)((mags >> 16) & 0xff); w3 = (float)(mags >> 24);
            w0 = (sg & 1) ? -w0 : w0; w1 = (sg & 2) ? -w1 : w1; w2 = (sg & 4) ? -w2 : w2; w3 = (sg & 8) ? -w3 : w3;
        }
#pragma unroll
        for (int j = 0; j < N; j++) {
            const float4 v = *(const float4*)(xs + (size_t)j * cols + e);
            float p = w0 * v.x;
            p = fmaf(w1, v.y, p);
            p = fmaf(w2, v.z, p);
            p = fmaf(w3, v.w, p);
            acc[j] = fmaf(scale, p, acc[j]);
        }
    }
}

template <int TYPE>
__device__ __forceinline__ int64_t sz_row_bytes(int cols) { return TYPE == SZ_TYPE_Q8_0 ? (int64_t)(cols / 32) * 34 : (int64_t)(cols / 256) * 110; }

// gate and up rows of one group, SwiGLU fused: act[pair][r] = silu(gate_r . x) * (up_r . x)
template <int TYPE, int N>
__device__ __forceinline__ void sz_gateup_body(const u8* gate, const u8* up, int H, int FF, const float* xs, const u32* grid,
                                               const u8* pairs, float* act, int r0, int r1) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t rb = sz_row_bytes<TYPE>(H);
    for (int r = r0 + warp; r < r1; r += 8) {
        float ag[N], au[N];
#pragma unroll
        for (int j = 0; j < N; j++) { ag[j] = 0.f; au[j] = 0.f; }
        sz_row_dot<TYPE, N>(gate + r * rb, H, xs, grid, lane, ag);
        sz_row_dot<TYPE, N>(up + r * rb, H, xs, grid, lane, au);
#pragma unroll
        for (int j = 0; j < N; j++) {
            const float g = sz_warp_sum(ag[j]), u = sz_warp_sum(au[j]);
            if (lane == 0) act[(size_t)pairs[j] * FF + r] = sz_silu(g) * u;
        }
    }
}

template <int TYPE, int N>
__device__ __forceinline__ void sz_down_body(const u8* down, int FF, int H, const float* xs, const u32* grid, const u8* pairs,
                                             float* eo, int r0, int r1) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t rb = sz_row_bytes<TYPE>(FF);
    for (int r = r0 + warp; r < r1; r += 8) {
        float a[N];
#pragma unroll
        for (int j = 0; j < N; j++) a[j] = 0.f;
        sz_row_dot<TYPE, N>(down + r * rb, FF, xs, grid, lane, a);
#pragma unroll
        for (int j = 0; j < N; j++) {
            const float v = sz_warp_sum(a[j]);
            if (lane == 0) eo[(size_t)pairs[j] * H + r] = v;
        }
    }
}

#define SZ_ROWS_PER_CTA 32

// grid: (ceil(out_rows / SZ_ROWS_PER_CTA), max groups).  DOWN = false: gate/up + SwiGLU from x rows; true: down from act rows.
template <int TYPE, bool DOWN>
__global__ void __launch_bounds__(256)
sz_rows_kernel(const SzPlan* __restrict__ plan, const u8* __restrict__ w0, u64 stride0, const u8* __restrict__ w1, u64 stride1,
               const float* __restrict__ in, int n_in, int n_out, float* __restrict__ out) {
    extern __shared__ __align__(128) u8 smem[];
    u32* grid = (u32*)smem;                // 512 words
    float* xs = (float*)(smem + 2048);     // [n][n_in]
    sz_pdl_wait();
    sz_pdl_trigger();
    const int g = blockIdx.y;
    if (g >= plan->n_groups) return;
    const int n = plan->count[g];
    const int64_t e = plan->expert[g];
    const u8* src_rows = DOWN ? plan->pairs[g] : plan->rows[g];
    for (int i = threadIdx.x; i < 512; i += 256) grid[i] = c_iq3s_grid[i];
    for (int j = 0; j < n; j++) {
        const float4* src = (const float4*)(in + (size_t)src_rows[j] * n_in);
        float4* dst = (float4*)(xs + (size_t)j * n_in);
        for (int i = threadIdx.x; i < n_in / 4; i += 256) dst[i] = __ldcg(src + i);
    }
    __syncthreads();
    const int r0 = blockIdx.x * SZ_ROWS_PER_CTA;
    const int r1 = min(r0 + SZ_ROWS_PER_CTA, n_out);
    const u8* a = w0 + e * stride0;
    const u8* pairs = plan->pairs[g];
    if (!DOWN) {
        const u8* b = w1 + e * stride1;
        switch (n) {
            case 1: sz_gateup_body<TYPE, 1>(a, b, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 2: sz_gateup_body<TYPE, 2>(a, b, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 3: sz_gateup_body<TYPE, 3>(a, b, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 4: sz_gateup_body<TYPE, 4>(a, b, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 5: sz_gateup_body<TYPE, 5>(a, b, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 6: sz_gateup_body<TYPE, 6>(a, b, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 7: sz_gateup_body<TYPE, 7>(a, b, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            default: sz_gateup_body<TYPE, 8>(a, b, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
        }
    } else {
        switch (n) {
            case 1: sz_down_body<TYPE, 1>(a, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 2: sz_down_body<TYPE, 2>(a, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 3: sz_down_body<TYPE, 3>(a, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 4: sz_down_body<TYPE, 4>(a, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 5: sz_down_body<TYPE, 5>(a, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 6: sz_down_body<TYPE, 6>(a, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            case 7: sz_down_body<TYPE, 7>(a, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
            default: sz_down_body<TYPE, 8>(a, n_in, n_out, xs, grid, pairs, out, r0, r1); break;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// EXL3: a block a 128-output slice of one matrix for one group; warp w owns tile column w of the slice

template <int K, int N>
__device__ __forceinline__ void sz_exl3_body(const u8* __restrict__ blob, int n_in, int n_out, int ob, const float* xr, float* so,
                                             const u8* pairs, float* out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const u32* tr = (const u32*)(blob + 2 * (size_t)n_in + 2 * (size_t)n_out + 4);
    const int nt = n_out / 16, kt = n_in / 16;
    float acc[N][2];
#pragma unroll
    for (int j = 0; j < N; j++) { acc[j][0] = 0.f; acc[j][1] = 0.f; }
    for (int k = 0; k < kt; k++) {
        u32 st[8];
        SzExl3Tile<K>::states(tr + ((size_t)k * nt + ob * 8 + warp) * (8 * K), lane, st);
#pragma unroll
        for (int jj = 0; jj < 8; jj++) {
            const float v = sz_exl3_cb2(st[jj]);
            const int row = k * 16 + sz_exl3_row(lane, jj);
#pragma unroll
            for (int j = 0; j < N; j++) acc[j][jj >> 2] = fmaf(xr[(size_t)j * n_in + row], v, acc[j][jj >> 2]);
        }
    }
    // the four lanes that share lane >> 2 hold the four input-row classes of the same two output columns
#pragma unroll
    for (int j = 0; j < N; j++) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float v = acc[j][h];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if ((lane & 3) == 0) so[j * 128 + warp * 16 + (lane >> 2) + 8 * h] = v;
        }
    }
    __syncthreads();
    // rotate the 128 outputs back and scale: y = H so * svh (exl3.rs:556-562); warp j takes row j
    const u16* svh = (const u16*)(blob + 2 * (size_t)n_in);
    for (int j = warp; j < N; j += 8) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = so[j * 128 + lane + 32 * e];
        sz_wht128_warp(v, lane);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int c = ob * 128 + lane + 32 * e;
            out[(size_t)pairs[j] * n_out + c] = (v[e] * SZ_RSQRT128) * sz_f16_to_f32(svh[c]);
        }
    }
}

// grid: (blocks of 128 outputs x matrices, max groups).  in1 != null: the input row is silu(in0) * in1 (the SwiGLU product).
template <int K>
__global__ void __launch_bounds__(256)
sz_exl3_kernel(const SzPlan* __restrict__ plan, const u8* __restrict__ w0, u64 stride0, const u8* __restrict__ w1, u64 stride1,
               const float* __restrict__ in0, const float* __restrict__ in1, int in_by_pair, int n_in, int n_out,
               float* __restrict__ out0, float* __restrict__ out1) {
    extern __shared__ __align__(128) u8 smem[];
    float* so = (float*)smem;              // [8][128]
    float* xr = (float*)(smem + 4096);     // [n][n_in]
    sz_pdl_wait();
    sz_pdl_trigger();
    const int g = blockIdx.y;
    if (g >= plan->n_groups) return;
    const int n = plan->count[g];
    const int64_t e = plan->expert[g];
    const int nblk = n_out / 128;
    const int mat = blockIdx.x / nblk, ob = blockIdx.x % nblk;
    const u8* blob = mat == 0 ? w0 + e * stride0 : w1 + e * stride1;
    float* out = mat == 0 ? out0 : out1;
    const u8* src_rows = in_by_pair ? plan->pairs[g] : plan->rows[g];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the input in the trellis' basis: (x * suh) H on every 128-block (exl3.rs:414-421), a warp a (row, block) item
    const u16* suh = (const u16*)blob;
    const int nb = n_in / 128;
    for (int item = warp; item < n * nb; item += 8) {
        const int j = item / nb, b = item % nb;
        const size_t src = (size_t)src_rows[j] * n_in + b * 128;
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int i = lane + 32 * q;
            float a = __ldcg(in0 + src + i);
            if (in1) a = sz_silu(a) * __ldcg(in1 + src + i);
            v[q] = a * sz_f16_to_f32(suh[b * 128 + i]);
        }
        sz_wht128_warp(v, lane);
#pragma unroll
        for (int q = 0; q < 4; q++) xr[(size_t)j * n_in + b * 128 + lane + 32 * q] = v[q] * SZ_RSQRT128;
    }
    __syncthreads();
    const u8* pairs = plan->pairs[g];
    switch (n) {
        case 1: sz_exl3_body<K, 1>(blob, n_in, n_out, ob, xr, so, pairs, out); break;
        case 2: sz_exl3_body<K, 2>(blob, n_in, n_out, ob, xr, so, pairs, out); break;
        case 3: sz_exl3_body<K, 3>(blob, n_in, n_out, ob, xr, so, pairs, out); break;
        case 4: sz_exl3_body<K, 4>(blob, n_in, n_out, ob, xr, so, pairs, out); break;
        case 5: sz_exl3_body<K, 5>(blob, n_in, n_out, ob, xr, so, pairs, out); break;
        case 6: sz_exl3_body<K, 6>(blob, n_in, n_out, ob, xr, so, pairs, out); break;
        case 7: sz_exl3_body<K, 7>(blob, n_in, n_out, ob, xr, so, pairs, out); break;
        default: sz_exl3_body<K, 8>(blob, n_in, n_out, ob, xr, so, pairs, out); break;
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// y[j] = sum over ranks of w * eo (f64, rank order) + sigmoid(shared gate logit) * shared output (forward.rs:1020-1033)

// With expert parallelism (e_lo..e_hi the experts this rank holds, y_fix != null) only the local pairs count and every term is
// added as 64-bit fixed point (scale 2^40), so that the all-reduce over ranks - integer addition - gives the same bits for any
// number of ranks.
#define SZ_YFIX_SCALE 1099511627776.0          // 2^40
#define SZ_YFIX_INV (1.0 / 1099511627776.0)

__global__ void __launch_bounds__(256)
sz_combine_kernel(const float* __restrict__ eo, const int32_t* __restrict__ ridx, const double* __restrict__ rw, const float* __restrict__ so,
                  const float* __restrict__ logits, int ne, int k, int H, int has_shared, float* __restrict__ y, long long* __restrict__ y_fix,
                  int e_lo, int e_hi, const SzEpPush push) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int j = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const bool on = i < H;
    const int slot = y_fix && push.world > 0 ? (int)(__ldcg(&((const SzEpHeader*)push.buf[push.me])->epoch) & 1ull) : 0;
    double acc = 0.0;
    long long fix = 0;
    for (int t = 0; t < (on ? k : 0); t++) {
        if (y_fix) {
            const int e = __ldcg(ridx + j * k + t);
            if (e < e_lo || e >= e_hi) continue;
            fix += __double2ll_rn(__ldcg(rw + j * k + t) * (double)__ldcg(eo + (size_t)(j * k + t) * H + i) * SZ_YFIX_SCALE);
        } else {
            acc += __ldcg(rw + j * k + t) * (double)__ldcg(eo + (size_t)(j * k + t) * H + i);
        }
    }
    if (has_shared && on) {
        const float sg = sz_sigmoid(__ldcg(logits + (size_t)j * (ne + 1) + ne));
        const double sv = (double)(sg * __ldcg(so + (size_t)j * H + i));
        if (y_fix) fix += __double2ll_rn(sv * SZ_YFIX_SCALE); else acc += sv;
    }
    if (!y_fix) { if (on) y[(size_t)j * H + i] = (float)acc; return; }
    if (push.world == 0) { if (on) y_fix[(size_t)j * H + i] = fix; return; }
    if (on) {
        for (int r = 0; r < push.world; r++) sz_ep_slot(push.buf[r], push.world, push.row_elems, slot, push.me)[(size_t)j * H + i] = fix;
    }
    __threadfence_system();
    __syncthreads();   // every thread of the block reaches this: the returns above depend on kernel arguments only
    if (threadIdx.x < push.world) atomicAdd_system(sz_ep_arrive(push.buf[threadIdx.x], push.me), 1ull);
}

// the summed fixed-point output back to f32
__global__ void __launch_bounds__(256) sz_yfix_finish_kernel(const long long* __restrict__ y_fix, int n, float* __restrict__ y) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = (float)((double)__ldcg(y_fix + i) * SZ_YFIX_INV);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// host side

static bool sz_is_exl3(int t) { return t > 1020 && t <= 1028; }

// Which kernels a layer takes.  The streaming EXL3 kernels cover K = 2..4, expert widths 128 / 256 / 512 and hidden sizes that are
// multiples of 512; everything else runs on the generic kernels above.
struct SzFast { bool exl3; bool shared_fused; };

static SzFast sz_fast_path(const sz_moe_layer* L) {
    SzFast f = {false, false};
    static const bool off = getenv("SZ_GENERIC_KERNELS") && atoi(getenv("SZ_GENERIC_KERNELS")) != 0;  // A/B switch: 1 = generic kernels only
    if (off) return f;
    const int K = L->expert_type - 1020;
    const int FF = L->expert_ff;
    if (sz_is_exl3(L->expert_type) && K >= 2 && K <= 4 && (FF == 128 || FF == 256 || FF == 512) && L->hidden % 512 == 0) {
        f.exl3 = true;
        f.shared_fused = L->shared_ff == FF && L->shared_type == L->expert_type;
    }
    return f;
}


static int sz_check_matrix(const char* what, int type, int n_in, int n_out) {
    if (sz_is_exl3(type)) {
        if (n_in % 128 || n_out % 128) return sz_fail(SZ_E_ARG, "%s: EXL3 needs whole 128-blocks, got %d -> %d", what, n_in, n_out);
    } else if (type == SZ_TYPE_Q8_0) {
        if (n_in % 128) return sz_fail(SZ_E_ARG, "%s: Q8_0 rows of %d weights are not a multiple of 128", what, n_in);
    } else if (type == SZ_TYPE_IQ3_S) {
        if (n_in % 256) return sz_fail(SZ_E_ARG, "%s: IQ3_S rows of %d weights are not whole superblocks", what, n_in);
    } else {
        return sz_fail(SZ_E_TYPE, "%s: no kernel for tensor type %d", what, type);
    }
    return SZ_OK;
}

// Block types start on a 16-byte boundary; an EXL3 blob is placed so that its trellis (after suh, svh and the marker) does.
static int sz_check_align(const char* what, int type, u64 base, int n_in, int n_out) {
    const u64 start = sz_is_exl3(type) ? base + 2 * (u64)n_in + 2 * (u64)n_out + 4 : base;
    if (start & 15) return sz_fail(SZ_E_ARG, "%s: %s must start on a 16-byte boundary", what, sz_is_exl3(type) ? "the trellis of an EXL3 blob" : "the tensor");
    return SZ_OK;
}

static int sz_moe_check(const sz_moe_layer* L, int m) {
    if (!L) return sz_fail(SZ_E_ARG, "null layer");
    if (m < 1 || m > SZ_MAX_VERIFY) return sz_fail(SZ_E_ARG, "a verify pass has 1..%d rows, got %d", SZ_MAX_VERIFY, m);
    if (L->hidden <= 0 || L->hidden % 128 || L->hidden > 4096) return sz_fail(SZ_E_ARG, "hidden = %d is not a multiple of 128 in 128..4096", L->hidden);
    if (L->n_expert < 1 || L->n_expert > SZ_MAX_EXPERTS) return sz_fail(SZ_E_ARG, "n_expert = %d (1..%d)", L->n_expert, SZ_MAX_EXPERTS);
    if (L->top_k < 1 || L->top_k > SZ_MAX_TOPK || L->top_k > L->n_expert)
        return sz_fail(SZ_E_ARG, "top_k = %d (1..%d, at most n_expert)", L->top_k, SZ_MAX_TOPK);
    if (L->expert_ff <= 0 || L->shared_ff < 0) return sz_fail(SZ_E_ARG, "expert_ff = %d, shared_ff = %d", L->expert_ff, L->shared_ff);
    if (L->ep_count < 0 || L->ep_first < 0 || (L->ep_count > 0 && L->ep_first + L->ep_count > L->n_expert))
        return sz_fail(SZ_E_ARG, "expert shard [%d, %d) of %d experts", L->ep_first, L->ep_first + L->ep_count, L->n_expert);
    int rc;
    if ((rc = sz_check_matrix("expert gate/up", L->expert_type, L->hidden, L->expert_ff))) return rc;
    if ((rc = sz_check_matrix("expert down", L->expert_type, L->expert_ff, L->hidden))) return rc;
    if (!L->router || !L->gate || !L->up || !L->down) return sz_fail(SZ_E_ARG, "null router or expert tensor");
    if (!sz_aligned16(L->router) || (L->gate_stride & 15) || (L->up_stride & 15) || (L->down_stride & 15))
        return sz_fail(SZ_E_ARG, "the router must be 16-byte aligned and expert strides multiples of 16");
    if ((rc = sz_check_align("expert gate", L->expert_type, L->gate, L->hidden, L->expert_ff))) return rc;
    if ((rc = sz_check_align("expert up", L->expert_type, L->up, L->hidden, L->expert_ff))) return rc;
    if ((rc = sz_check_align("expert down", L->expert_type, L->down, L->expert_ff, L->hidden))) return rc;
    if (L->shared_ff > 0 && (L->ep_count == 0 || L->ep_shared)) {  // a shard that does not add the shared term holds none of it
        if ((rc = sz_check_matrix("shared gate/up", L->shared_type, L->hidden, L->shared_ff))) return rc;
        if ((rc = sz_check_matrix("shared down", L->shared_type, L->shared_ff, L->hidden))) return rc;
        if (!L->shared_router || !L->sh_gate || !L->sh_up || !L->sh_down) return sz_fail(SZ_E_ARG, "null shared-expert tensor");
        if (!sz_aligned16(L->shared_router)) return sz_fail(SZ_E_ARG, "the shared router row must be 16-byte aligned");
        if ((rc = sz_check_align("shared gate", L->shared_type, L->sh_gate, L->hidden, L->shared_ff))) return rc;
        if ((rc = sz_check_align("shared up", L->shared_type, L->sh_up, L->hidden, L->shared_ff))) return rc;
        if ((rc = sz_check_align("shared down", L->shared_type, L->sh_down, L->shared_ff, L->hidden))) return rc;
    }
    return SZ_OK;
}

extern "C" int sz_moe_scratch_bytes(const sz_moe_layer* L, int m, int64_t* bytes) {
    int rc = sz_moe_check(L, m);
    if (rc) return rc;
    if (!bytes) return sz_fail(SZ_E_ARG, "null result pointer");
    *bytes = sz_moe_layout(L, m).total;
    return SZ_OK;
}

extern "C" int sz_moe_scratch_init(uint64_t scratch, int64_t scratch_bytes, uint64_t stream) {
    if (!scratch || scratch_bytes < 256 || (scratch & 255)) return sz_fail(SZ_E_ARG, "scratch must be 256-byte aligned and non-empty");
    SZ_CUDA(cudaMemsetAsync((void*)scratch, 0, 256, (cudaStream_t)stream));
    return SZ_OK;
}

extern "C" int sz_moe_launches(const sz_moe_layer* L) {
    if (!L) return 0;
    const SzFast f = sz_fast_path(L);
    const int ep = L->ep_count > 0 ? 1 : 0;  // the fixed-point finish (the all-reduce is NCCL's kernel, not counted)
    if (f.exl3) return 4 + (L->shared_ff > 0 && !f.shared_fused ? 2 : 0) + ep;
    return (L->shared_ff > 0 ? 6 : 4) + ep;
}

static int sz_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// The streaming block-format kernels.  Returns SZ_E_TYPE (without setting an error text) when the shape is not one they take.
template <int TYPE, bool DOWN>
static int sz_launch_blk(cudaStream_t st, const SzPlan* plan, int groups, const u8* w0, u64 s0, const u8* w1, u64 s1, const float* in, int n_in,
                         int n_out, float* out, u32* ctrl) {
    constexpr int RT = DOWN ? 4 : 1;
    if (n_in % 256 || n_out % (16 * RT) || groups < 1) return SZ_E_TYPE;
    const size_t rb = TYPE == SZ_TYPE_Q8_0 ? (size_t)(n_in / 32) * 34 : (size_t)(n_in / 256) * 110;
    SzBlkCfg c = {};
    c.by_row = rb % 16 == 0 && rb >= 1024;   // short rows go in one copy a unit: a copy a row would cost more to issue than the bank conflicts it avoids
    int rbp = (int)rb;
    if (c.by_row) while (((rbp / 4) % 32) % 8 != 4) rbp += 16;   // consecutive rows 4 (mod 8) words apart in bank space
    c.rbp = rbp;
    c.unit_bytes = (DOWN ? 1 : 2) * 16 * RT * rbp;
    int xsp = n_in;
    while (((xsp / 2) % 32) != 16) xsp += 8;
    c.xsp = xsp;
    c.slices = n_out / (16 * RT);
    const size_t fixed = 64 + 2048 + 4096 + (size_t)(DOWN ? 1 : 2) * RT * 4096 + (size_t)2 * SZ_MAX_VERIFY * xsp * 2;
    const size_t budget = 222 * 1024;   // dynamic + the kernel's static shared memory stay under the 227 KB a block may have
    if (fixed + 2 * (size_t)c.unit_bytes > budget) return SZ_E_TYPE;
    int NS = (int)((budget - fixed) / c.unit_bytes);
    c.NS = NS > 4 ? 4 : NS;
    const size_t smem = fixed + (size_t)c.NS * c.unit_bytes;
    static bool set = false;
    if (!set) { SZ_CUDA(cudaFuncSetAttribute(sz_blk_ffn_kernel<TYPE, DOWN, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024)); set = true; }
    const int per_sm = smem + 4096 <= 110 * 1024 ? 2 : 1;
    int blocks = sz_sm_count() * per_sm;
    const long long units = (long long)groups * c.slices;
    if (blocks > units) blocks = (int)units;
    SZ_CUDA(sz_launch(DOWN ? "down_blk" : "gateup_blk", sz_blk_ffn_kernel<TYPE, DOWN, RT>, dim3(blocks), dim3(256), smem, st, true, plan, w0, s0, w1, s1,
                      in, n_in, n_out, out, c, ctrl));
    return SZ_OK;
}

template <int TYPE>
static int sz_launch_rows(cudaStream_t st, const SzPlan* plan, int groups, const u8* gate, u64 gs, const u8* up, u64 us, const u8* down,
                          u64 ds, const float* x, int H, int FF, float* act, float* eo, bool down_pass, u32* ctrl) {
    static const bool generic_only = getenv("SZ_GENERIC_KERNELS") && atoi(getenv("SZ_GENERIC_KERNELS")) != 0;
    if (!generic_only) {  // the streaming tensor-pipe kernels, where the shapes fit them
        int rc = down_pass ? sz_launch_blk<TYPE, true>(st, plan, groups, down, ds, nullptr, 0, act, FF, H, eo, ctrl)
                           : sz_launch_blk<TYPE, false>(st, plan, groups, gate, gs, up, us, x, H, FF, act, ctrl);
        if (rc != SZ_E_TYPE) return rc;  // SZ_E_TYPE: not a shape for them
    }
    const size_t smem = 2048 + (size_t)SZ_MAX_VERIFY * (down_pass ? FF : H) * 4;
    if (!down_pass) {
        static bool set = false;
        if (!set) { SZ_CUDA(cudaFuncSetAttribute(sz_rows_kernel<TYPE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); set = true; }
        dim3 grid((FF + SZ_ROWS_PER_CTA - 1) / SZ_ROWS_PER_CTA, groups);
        SZ_CUDA(sz_launch("gateup_rows", sz_rows_kernel<TYPE, false>, grid, dim3(256), smem, st, true, plan, gate, gs, up, us, x, H, FF, act));
    } else {
        static bool set = false;
        if (!set) { SZ_CUDA(cudaFuncSetAttribute(sz_rows_kernel<TYPE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); set = true; }
        dim3 grid((H + SZ_ROWS_PER_CTA - 1) / SZ_ROWS_PER_CTA, groups);
        SZ_CUDA(sz_launch("down_rows", sz_rows_kernel<TYPE, true>, grid, dim3(256), smem, st, true, plan, down, ds, (const u8*)nullptr, (u64)0, act, FF, H, eo));
    }
    return SZ_OK;
}

template <int K>
static int sz_launch_exl3(cudaStream_t st, const SzPlan* plan, int groups, const u8* w0, u64 s0, const u8* w1, u64 s1, const float* in0,
                          const float* in1, int by_pair, int n_in, int n_out, float* out0, float* out1) {
    static bool set = false;
    if (!set) { SZ_CUDA(cudaFuncSetAttribute(sz_exl3_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); set = true; }
    const size_t smem = 4096 + (size_t)SZ_MAX_VERIFY * n_in * 4;
    dim3 grid((n_out / 128) * (w1 ? 2 : 1), groups);
    SZ_CUDA(sz_launch(w1 ? "gateup_exl3" : "down_exl3", sz_exl3_kernel<K>, grid, dim3(256), smem, st, true, plan, w0, s0, w1, s1, in0, in1, by_pair, n_in, n_out, out0, out1));
    return SZ_OK;
}

// One expert FFN pass (gate/up then down) for the groups of `plan`.
static int sz_ffn(cudaStream_t st, int type, const SzPlan* plan, int groups, u64 gate, u64 gs, u64 up, u64 us, u64 down, u64 ds,
                  const float* x, int H, int FF, float* g, float* u, float* eo, bool down_pass, u32* ctrl) {
    const u8 *pg = (const u8*)gate, *pu = (const u8*)up, *pd = (const u8*)down;
    if (type == SZ_TYPE_Q8_0) return sz_launch_rows<SZ_TYPE_Q8_0>(st, plan, groups, pg, gs, pu, us, pd, ds, x, H, FF, g, eo, down_pass, ctrl);
    if (type == SZ_TYPE_IQ3_S) return sz_launch_rows<SZ_TYPE_IQ3_S>(st, plan, groups, pg, gs, pu, us, pd, ds, x, H, FF, g, eo, down_pass, ctrl);
#define SZ_EXL3_CASE(KK)                                                                                                        \
    case KK:                                                                                                                    \
        return down_pass ? sz_launch_exl3<KK>(st, plan, groups, pd, ds, nullptr, 0, g, u, 1, FF, H, eo, nullptr)               \
                         : sz_launch_exl3<KK>(st, plan, groups, pg, gs, pu, us, x, nullptr, 0, H, FF, g, u);
    switch (type - 1020) {
        SZ_EXL3_CASE(1) SZ_EXL3_CASE(2) SZ_EXL3_CASE(3) SZ_EXL3_CASE(4) SZ_EXL3_CASE(5) SZ_EXL3_CASE(6) SZ_EXL3_CASE(7) SZ_EXL3_CASE(8)
    }
#undef SZ_EXL3_CASE
    return sz_fail(SZ_E_TYPE, "no kernel for tensor type %d", type);
}


struct SzXWindows { int n = 1; long long x = 0, gu = 0, d = 0; };   // plans in a row, one block row each: elements between the windows' inputs and sums
template <int K, int NTC>
static int sz_x3_launch_k(cudaStream_t st, const sz_moe_layer* L, int m, const SzPlan* plan, const float* x, long long* acc_gu, long long* acc_d,
                          u32* ctrl, bool sh, bool only_xw = false, SzXWindows win = SzXWindows()) {
    static bool set = false;
    if (!set) {
        SZ_CUDA(cudaFuncSetAttribute(sz_x3_gateup_kernel<K, NTC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SzX3<K, NTC>::SMEM_BYTES));
        SZ_CUDA(cudaFuncSetAttribute(sz_x3_down_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, SzX3<K, 4>::SMEM_BYTES));
        set = true;
    }
    // SZ_X3_CLASSIC=1: the block-synchronous kernels of sz_moe_exl3.cuh (the second implementation; same bits) instead of the
    // warp-specialised ones
    const char* cl = getenv("SZ_X3_CLASSIC");   // (read at every call: a test switches it inside one process)
    const bool classic = !only_xw && cl && atoi(cl) != 0;
    if (!classic) {
        // Shape of the launch: OCC blocks a multiprocessor (2 or 3), a unit 8 TW tile columns a consumer warp wide (TW = 4, 2 or 1: 24, 12
        // or 6 KB of trellis at 3 bits).  Narrower units and a third block spread the units evenly: gate / up of 40 experts of the
        // benchmark's shape are 1,280 units 4 wide - 4.3 a block at 296 blocks, so some take 5 - and the down matrices only 640.
        // SZ_XW_OCC / SZ_XW_TW / SZ_XW_TWD override the choice (experiments).
        const dim3 block(SZ_XW_THREADS);
        const char *eo = getenv("SZ_XW_OCC"), *et = getenv("SZ_XW_TW"), *ed = getenv("SZ_XW_TWD");
        // few rows mean few units (a 1-row pass of the benchmark's shape: 11 groups, 352 units 4 wide for 296 blocks): narrower units
        // and a third block a multiprocessor spread them better (4.30 -> 4.19 ms a 1-row pass of the 48-layer model); with 4 rows the
        // wide units win (6.18 against 6.35 ms)
        const bool few = m * (int)L->top_k <= 24;
        const int occ = eo && atoi(eo) == 2 ? 2 : (eo && atoi(eo) == 3 ? 3 : (few ? 3 : 2));
        int tw = et ? atoi(et) : (few ? 2 : 4), twd = ed ? atoi(ed) : (few ? 2 : 4);
        if (!(tw == 1 || tw == 2 || tw == 4) || tw > NTC || NTC % tw) tw = NTC < 4 ? NTC : 4;
        if (tw == 3) tw = 1;
        if (!(twd == 1 || twd == 2 || twd == 4)) twd = 4;
        const dim3 grid(occ * sz_sm_count(), win.n);
        int rc = SZ_E_TYPE;
#define SZ_XW_GU(TT, OO)                                                                                                                    \
    if (tw == TT && occ == OO) {                                                                                                            \
        static bool setv = false;                                                                                                           \
        if (!setv) { SZ_CUDA(cudaFuncSetAttribute(sz_xw_gateup_kernel<K, NTC, TT, OO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SzXW<K, TT, OO>::SMEM_BYTES)); setv = true; } \
        SZ_CUDA(sz_launch("gateup_exl3s", sz_xw_gateup_kernel<K, NTC, TT, OO>, grid, block, SzXW<K, TT, OO>::SMEM_BYTES, st, true, plan, (const u8*)L->gate, \
                          (u64)L->gate_stride, (const u8*)L->up, (u64)L->up_stride, (const u8*)(sh ? L->sh_gate : 0), (const u8*)(sh ? L->sh_up : 0), x, m, \
                          (int)L->hidden, (int)L->top_k, acc_gu, ctrl, win.x, win.gu));                                                     \
        rc = SZ_OK;                                                                                                                         \
    }
#define SZ_XW_DN(TT, OO)                                                                                                                    \
    if (twd == TT && occ == OO) {                                                                                                           \
        static bool setv = false;                                                                                                           \
        if (!setv) { SZ_CUDA(cudaFuncSetAttribute(sz_xw_down_kernel<K, TT, OO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SzXW<K, TT, OO>::SMEM_BYTES)); setv = true; } \
        SZ_CUDA(sz_launch("down_exl3s", sz_xw_down_kernel<K, TT, OO>, grid, block, SzXW<K, TT, OO>::SMEM_BYTES, st, true, plan, (const u8*)L->gate, (u64)L->gate_stride, \
                          (const u8*)L->up, (u64)L->up_stride, (const u8*)L->down, (u64)L->down_stride, (const u8*)(sh ? L->sh_gate : 0),   \
                          (const u8*)(sh ? L->sh_up : 0), (const u8*)(sh ? L->sh_down : 0), m, (int)L->hidden, (int)L->expert_ff, (int)L->top_k, \
                          (const long long*)acc_gu, acc_d, ctrl, win.gu, win.d));                                                           \
        rc = SZ_OK;                                                                                                                         \
    }
        if constexpr (NTC % 4 == 0) { SZ_XW_GU(4, 2) SZ_XW_GU(4, 3) }
        if constexpr (NTC % 2 == 0) { SZ_XW_GU(2, 2) SZ_XW_GU(2, 3) }
        SZ_XW_GU(1, 2) SZ_XW_GU(1, 3)
        if (rc) return sz_fail(SZ_E_TYPE, "no gate/up kernel for this unit shape");
        rc = SZ_E_TYPE;
        SZ_XW_DN(4, 2) SZ_XW_DN(4, 3) SZ_XW_DN(2, 2) SZ_XW_DN(2, 3) SZ_XW_DN(1, 2) SZ_XW_DN(1, 3)
        if (rc) return sz_fail(SZ_E_TYPE, "no down kernel for this unit shape");
        return SZ_OK;
#undef SZ_XW_GU
#undef SZ_XW_DN
    }
    const dim3 grid(2 * sz_sm_count());
    const dim3 block(SZ_X3_THREADS);
    SZ_CUDA(sz_launch("gateup_exl3s", sz_x3_gateup_kernel<K, NTC>, grid, block, SzX3<K, NTC>::SMEM_BYTES, st, true, plan, (const u8*)L->gate,
                      (u64)L->gate_stride, (const u8*)L->up, (u64)L->up_stride, (const u8*)(sh ? L->sh_gate : 0), (const u8*)(sh ? L->sh_up : 0), x, m,
                      (int)L->hidden, (int)L->top_k, acc_gu, ctrl));
    SZ_CUDA(sz_launch("down_exl3s", sz_x3_down_kernel<K>, grid, block, SzX3<K, 4>::SMEM_BYTES, st, true, plan, (const u8*)L->gate, (u64)L->gate_stride,
                      (const u8*)L->up, (u64)L->up_stride, (const u8*)L->down, (u64)L->down_stride, (const u8*)(sh ? L->sh_gate : 0),
                      (const u8*)(sh ? L->sh_up : 0), (const u8*)(sh ? L->sh_down : 0), m, (int)L->hidden, (int)L->expert_ff, (int)L->top_k,
                      (const long long*)acc_gu, acc_d, ctrl));
    return SZ_OK;
}

static int sz_x3_launch(cudaStream_t st, const sz_moe_layer* L, int m, const SzPlan* plan, const float* x, long long* acc_gu, long long* acc_d,
                        u32* ctrl, bool sh, bool only_xw = false, SzXWindows win = SzXWindows()) {
    const int K = L->expert_type - 1020, NTC = L->expert_ff / 128;
#define SZ_X3_CASE(KK, NN) if (K == KK && NTC == NN) return sz_x3_launch_k<KK, NN>(st, L, m, plan, x, acc_gu, acc_d, ctrl, sh, only_xw, win);
    SZ_X3_CASE(2, 1) SZ_X3_CASE(2, 2) SZ_X3_CASE(2, 4) SZ_X3_CASE(3, 1) SZ_X3_CASE(3, 2) SZ_X3_CASE(3, 4) SZ_X3_CASE(4, 1) SZ_X3_CASE(4, 2) SZ_X3_CASE(4, 4)
#undef SZ_X3_CASE
    return sz_fail(SZ_E_TYPE, "no streaming EXL3 kernel for K = %d, FF = %d", K, L->expert_ff);
}

int sz_ep_allreduce_i64(long long* buf, size_t count, cudaStream_t st);  // sz_ep.cu
int sz_ep_p2p_push(int hidden, SzEpPush* p);
int sz_ep_p2p_finish(int m, int hidden, unsigned long long combine_blocks, float* y, cudaStream_t st);
extern "C" int sz_ep_p2p_world(void);
extern "C" int sz_ep_world(void);

// The pass itself.  y_fix == null: the whole layer into y (f32).  y_fix != null: expert-parallel share - only the experts this rank
// holds (and the shared expert where ep_shared says so) - as 64-bit fixed point into y_fix; y is not touched.
static int sz_moe_run(const sz_moe_layer* L0, uint64_t x, int m, float* y, long long* y_fix, uint64_t route_idx, uint64_t route_w, uint64_t scratch,
                      int64_t scratch_bytes, uint64_t stream, const SzEpPush& push, unsigned long long* combine_blocks) {
    int rc = sz_moe_check(L0, m);
    if (rc) return rc;
    if (!x || !sz_aligned16(x)) return sz_fail(SZ_E_ARG, "x must be non-null and 16-byte aligned");
    if ((route_idx & 3) || (route_w & 7)) return sz_fail(SZ_E_ARG, "misaligned routing output");
    const SzMoeScratch S = sz_moe_layout(L0, m);
    if (!scratch || (scratch & 255)) return sz_fail(SZ_E_ARG, "scratch must be 256-byte aligned");
    if (scratch_bytes < S.total) return sz_fail(SZ_E_SCRATCH, "scratch of %lld bytes, %lld needed", (long long)scratch_bytes, (long long)S.total);
    // kernels index an expert's matrix as base + e * stride with the global expert id: shift the bases of a local shard accordingly
    sz_moe_layer Lc = *L0;
    const bool ep = y_fix != nullptr;
    int e_lo = 0, e_hi = Lc.n_expert;
    if (Lc.ep_count > 0) {
        e_lo = Lc.ep_first; e_hi = Lc.ep_first + Lc.ep_count;
        Lc.gate -= (u64)e_lo * Lc.gate_stride; Lc.up -= (u64)e_lo * Lc.up_stride; Lc.down -= (u64)e_lo * Lc.down_stride;
    }
    const sz_moe_layer* L = &Lc;
    cudaStream_t st = (cudaStream_t)stream;
    u8* base = (u8*)scratch;
    u32* ctrl = (u32*)(base + S.ctrl);
    float* logits = (float*)(base + S.logits);
    int32_t* ridx = (int32_t*)(base + S.ridx);
    double* rw = (double*)(base + S.rw);
    SzPlan* plan = (SzPlan*)(base + S.plan);
    SzPlan* plan_sh = (SzPlan*)(base + S.plan_sh);
    float *g = (float*)(base + S.g), *u = (float*)(base + S.u), *sg = (float*)(base + S.sg), *su = (float*)(base + S.su);
    float *eo = (float*)(base + S.eo), *so = (float*)(base + S.so);
    const float* xp = (const float*)x;
    const int H = L->hidden, FF = L->expert_ff, SF = L->shared_ff;
    const bool shared = SF > 0 && (!ep || L->ep_count == 0 || L->ep_shared);

    const int route_rows = L->n_expert + (shared ? 1 : 0);
    const SzFast fast = sz_fast_path(L);
    {
        const dim3 grid((route_rows + SZ_ROUTE_RB - 1) / SZ_ROUTE_RB), block(SZ_ROUTE_THREADS);
        const int nch = (H / 4 + SZ_ROUTE_THREADS - 1) / SZ_ROUTE_THREADS;
        cudaError_t e = cudaErrorInvalidValue;
#define SZ_ROUTE_GO(MM, MPP, NC)                                                                                                         \
    e = sz_launch("route", sz_route_kernel<MM, MPP, NC>, grid, block, 0, st, true, xp, H, (const float*)L->router,                       \
                  (const float*)(shared ? L->shared_router : 0), (int)L->n_expert, (int)L->top_k, logits, ridx, rw, plan, plan_sh, ctrl, \
                  (int32_t*)route_idx, (double*)route_w, (uint4*)(base + S.acc_gu), fast.exl3 ? (int)(S.acc_bytes / 16) : 0,             \
                  (int)L->ep_first, (int)L->ep_count)
#define SZ_ROUTE_M(MM, MPP)                                                                    \
    case MM:                                                                                   \
        if (nch <= 1) SZ_ROUTE_GO(MM, MPP, 1); else if (nch == 2) SZ_ROUTE_GO(MM, MPP, 2); else SZ_ROUTE_GO(MM, MPP, 4); \
        break;
        switch (m) {
            SZ_ROUTE_M(1, 1) SZ_ROUTE_M(2, 2) SZ_ROUTE_M(3, 4) SZ_ROUTE_M(4, 4) SZ_ROUTE_M(5, 8) SZ_ROUTE_M(6, 8) SZ_ROUTE_M(7, 8) SZ_ROUTE_M(8, 8)
        }
#undef SZ_ROUTE_M
#undef SZ_ROUTE_GO
        SZ_CUDA(e);
    }
    const int groups = m * L->top_k;
    if (fast.exl3) {
        // streaming EXL3 kernels for the routed experts (and the shared expert when it has the same type and width)
        long long *acc_gu = (long long*)(base + S.acc_gu), *acc_d = (long long*)(base + S.acc_d);
        const bool sh_fused = fast.shared_fused && shared;
        if (shared && !sh_fused) {
            if ((rc = sz_ffn(st, L->shared_type, plan_sh, 1, L->sh_gate, 0, L->sh_up, 0, L->sh_down, 0, xp, H, SF, sg, su, so, false, ctrl))) return rc;
            if ((rc = sz_ffn(st, L->shared_type, plan_sh, 1, L->sh_gate, 0, L->sh_up, 0, L->sh_down, 0, xp, H, SF, sg, su, so, true, ctrl))) return rc;
        }
        if ((rc = sz_x3_launch(st, L, m, plan, xp, acc_gu, acc_d, ctrl, sh_fused))) return rc;
        SZ_CUDA(sz_launch("combine_exl3", sz_x3_combine_kernel, dim3(m * (H / 128)), dim3((L->top_k + 1) * 32), 0, st, true, (const long long*)acc_d,
                          (const int32_t*)ridx, (const double*)rw, (const u8*)L->down, (u64)L->down_stride,
                          (const u8*)(sh_fused ? L->sh_down : 0), (const float*)(shared && !sh_fused ? so : nullptr), (const float*)logits,
                          (int)L->n_expert, (int)L->top_k, m, H, FF, shared ? 1 : 0, y, y_fix, e_lo, e_hi, push));
        if (combine_blocks) *combine_blocks = (unsigned long long)m * (H / 128);
        return SZ_OK;
    }
    if ((rc = sz_ffn(st, L->expert_type, plan, groups, L->gate, L->gate_stride, L->up, L->up_stride, L->down, L->down_stride, xp, H, FF, g, u,
                     eo, false, ctrl)))
        return rc;
    if (shared && (rc = sz_ffn(st, L->shared_type, plan_sh, 1, L->sh_gate, 0, L->sh_up, 0, L->sh_down, 0, xp, H, SF, sg, su, so, false, ctrl))) return rc;
    if ((rc = sz_ffn(st, L->expert_type, plan, groups, L->gate, L->gate_stride, L->up, L->up_stride, L->down, L->down_stride, xp, H, FF, g, u,
                     eo, true, ctrl)))
        return rc;
    if (shared && (rc = sz_ffn(st, L->shared_type, plan_sh, 1, L->sh_gate, 0, L->sh_up, 0, L->sh_down, 0, xp, H, SF, sg, su, so, true, ctrl))) return rc;
    SZ_CUDA(sz_launch("combine", sz_combine_kernel, dim3((H + 255) / 256, m), dim3(256), 0, st, true, (const float*)eo, (const int32_t*)ridx,
                      (const double*)rw, (const float*)so, (const float*)logits, (int)L->n_expert, (int)L->top_k, H, shared ? 1 : 0, y, y_fix, e_lo, e_hi, push));
    if (combine_blocks) *combine_blocks = (unsigned long long)((H + 255) / 256) * m;
    return SZ_OK;
}

// pdl: whether the launch may overlap the tail of the kernel before it.  After a collective it may not: a library's kernel is no
// party to the programmatic-dependency protocol, so the finish follows it in plain stream order.
static int sz_moe_finish_launch(uint64_t y_fix, int m, int hidden, uint64_t y, uint64_t stream, bool pdl) {
    if (!y_fix || !y || m < 1 || m > SZ_MAX_VERIFY || hidden < 1 || (y_fix & 7) || (y & 3)) return sz_fail(SZ_E_ARG, "sz_moe_finish: bad argument");
    const int n = m * hidden;
    SZ_CUDA(sz_launch("moe_finish", sz_yfix_finish_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, pdl, (const long long*)y_fix, n, (float*)y));
    return SZ_OK;
}

// blocks of the combine kernel a pass of m rows launches for this layer (what one exchange adds to the arrival counters)
int sz_moe_combine_blocks(const sz_moe_layer* L, int m) {
    return sz_fast_path(L).exl3 ? m * (L->hidden / 128) : ((L->hidden + 255) / 256) * m;
}

extern "C" int sz_moe_finish(uint64_t y_fix, int m, int hidden, uint64_t y, uint64_t stream) {
    return sz_moe_finish_launch(y_fix, m, hidden, y, stream, false);  // the caller's own exchange came before it
}

extern "C" int sz_moe_verify_partial(const sz_moe_layer* L, uint64_t x, int m, uint64_t y_fix, uint64_t scratch, int64_t scratch_bytes,
                                     uint64_t stream) {
    if (sz_ep_p2p_world() > 0 && !y_fix) {  // exchange attached and no local destination: the partial goes to every rank's buffer
        int rc = sz_moe_check(L, m);
        if (rc) return rc;
        SzEpPush push;
        if ((rc = sz_ep_p2p_push(L->hidden, &push))) return rc;
        const SzMoeScratch S0 = sz_moe_layout(L, m);
        return sz_moe_run(L, x, m, nullptr, (long long*)((u8*)scratch + S0.y_fix), 0, 0, scratch, scratch_bytes, stream, push, nullptr);
    }
    if (!y_fix || (y_fix & 15)) return sz_fail(SZ_E_ARG, "sz_moe_verify_partial: y_fix must be non-null and 16-byte aligned");
    SzEpPush none = {};
    return sz_moe_run(L, x, m, nullptr, (long long*)y_fix, 0, 0, scratch, scratch_bytes, stream, none, nullptr);
}

extern "C" int sz_moe_verify(const sz_moe_layer* L, uint64_t x, int m, uint64_t y, uint64_t route_idx, uint64_t route_w,
                             uint64_t scratch, int64_t scratch_bytes, uint64_t stream) {
    if (!y || !sz_aligned16(y)) return sz_fail(SZ_E_ARG, "y must be non-null and 16-byte aligned");
    SzEpPush none = {};
    if (!L || L->ep_count <= 0) return sz_moe_run(L, x, m, (float*)y, nullptr, route_idx, route_w, scratch, scratch_bytes, stream, none, nullptr);
    // expert-parallel layer: this rank's share in fixed point, summed over the ranks (exactly: integers), then back to f32
    int rc = sz_moe_check(L, m);
    if (rc) return rc;
    if (sz_ep_p2p_world() > 0) {
        // over peer memory: the combine kernel stores its share into every rank's exchange buffer and the finish kernel adds the shares
        SzEpPush push;
        if ((rc = sz_ep_p2p_push(L->hidden, &push))) return rc;
        const SzMoeScratch S0 = sz_moe_layout(L, m);
        unsigned long long nb = 0;
        if ((rc = sz_moe_run(L, x, m, nullptr, (long long*)((u8*)scratch + S0.y_fix), route_idx, route_w, scratch, scratch_bytes, stream, push, &nb))) return rc;
        return sz_ep_p2p_finish(m, L->hidden, nb, (float*)y, (cudaStream_t)stream);
    }
    if (sz_ep_world() < 1) return sz_fail(SZ_E_ARG, "the layer is sharded (ep_count = %d) but neither sz_ep_init nor sz_ep_p2p_attach has run", L->ep_count);
    const SzMoeScratch S = sz_moe_layout(L, m);
    long long* y_fix = (long long*)((u8*)scratch + S.y_fix);
    if ((rc = sz_moe_run(L, x, m, nullptr, y_fix, route_idx, route_w, scratch, scratch_bytes, stream, none, nullptr))) return rc;
    const bool exchange = sz_ep_world() > 1;
    if (exchange && (rc = sz_ep_allreduce_i64(y_fix, (size_t)m * L->hidden, (cudaStream_t)stream))) return rc;
    return sz_moe_finish_launch((uint64_t)y_fix, m, L->hidden, y, stream, !exchange);
}

// ---- many rows at once (sz_moe_rows.cuh) ---------------------------------------------------------------------------------------------
struct SzRowsScratch {
    int64_t ctrl, logits, ridx, rw, cplan, cplan_sh, plan, xg, acc_gu, acc_d, total;
    int64_t gu_row, d_row;   // i64 elements a slot
};
// One layout whatever the rows of a call (sized for SZ_ROWS_MAX): a scratch serves calls of any row count, and the tickets and the
// error word stay where they were cleared - a layout that moved with the row count would put one call's tickets on another's data.
static SzRowsScratch sz_rows_layout(const sz_moe_layer* L) {
    SzRowsScratch s;
    int64_t o = 0;
    const int R = SZ_ROWS_MAX;
    const int chunks = R / 8, W = SZ_ROWS_WIN + SZ_ROWS_SHWIN;
    const int64_t ffm = L->expert_ff > L->shared_ff ? L->expert_ff : L->shared_ff;
    s.ctrl = o; o = sz_up256(o + 64 * (int64_t)(chunks + 1));            // one block of 16 words a chunk (the router's ticket), then the expert kernels'
    s.logits = o; o = sz_up256(o + 4 * (int64_t)R * (L->n_expert + 1));
    s.ridx = o; o = sz_up256(o + 4 * (int64_t)R * L->top_k);
    s.rw = o; o = sz_up256(o + 8 * (int64_t)R * L->top_k);
    s.cplan = o; o = sz_up256(o + (int64_t)sizeof(SzPlan) * chunks);
    s.cplan_sh = o; o = sz_up256(o + (int64_t)sizeof(SzPlan) * chunks);
    s.plan = o; o = sz_up256(o + (int64_t)sizeof(SzRowsPlan));
    s.xg = o; o = sz_up256(o + 4 * (int64_t)W * SZ_ROWS_SLOTS * L->hidden);
    s.gu_row = 2 * ffm; s.d_row = L->hidden;
    s.acc_gu = o; o = sz_up256(o + 8 * (int64_t)W * SZ_ROWS_SLOTS * s.gu_row);
    s.acc_d = o; o = sz_up256(o + 8 * (int64_t)W * SZ_ROWS_SLOTS * s.d_row);
    s.total = o;
    return s;
}

// zeroes the accumulators of the slots a window uses (grid (slots, windows), block 256)
static __global__ void __launch_bounds__(256)
sz_rows_zero_kernel(const SzRowsPlan* __restrict__ P, long long* __restrict__ acc_gu, long long gu_row, long long* __restrict__ acc_d, long long d_row) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int s = blockIdx.x, w = blockIdx.y;
    if (P->src[w][s] < 0) return;
    uint4* a = (uint4*)(acc_gu + ((size_t)w * SZ_ROWS_SLOTS + s) * gu_row);
    uint4* b = (uint4*)(acc_d + ((size_t)w * SZ_ROWS_SLOTS + s) * d_row);
    for (long long i = threadIdx.x; i < gu_row / 2; i += 256) a[i] = make_uint4(0, 0, 0, 0);
    for (long long i = threadIdx.x; i < d_row / 2; i += 256) b[i] = make_uint4(0, 0, 0, 0);
}

extern "C" int sz_moe_rows_scratch_bytes(const sz_moe_layer* L, int rows, int64_t* bytes) {
    if (!L || !bytes) return sz_fail(SZ_E_ARG, "sz_moe_rows_scratch_bytes: null argument");
    if (rows < 8 || rows > SZ_ROWS_MAX || rows % 8) return sz_fail(SZ_E_ARG, "sz_moe_rows: rows = %d (a multiple of 8 up to %d)", rows, SZ_ROWS_MAX);
    *bytes = sz_rows_layout(L).total;
    return SZ_OK;
}

// y[j] = moe(x[j]) for j < rows; x, y: f32 [rows][hidden].  EXL3 experts (routed and shared); every distinct expert is decoded once.
// route_idx / route_w: as sz_moe_verify's, [rows][top_k], or 0.
extern "C" int sz_moe_rows(const sz_moe_layer* L, uint64_t x, int rows, uint64_t y, uint64_t route_idx, uint64_t route_w, uint64_t scratch,
                           int64_t scratch_bytes, uint64_t stream) {
    int rc = sz_moe_check(L, 8);
    if (rc) return rc;
    if (rows < 8 || rows > SZ_ROWS_MAX || rows % 8) return sz_fail(SZ_E_ARG, "sz_moe_rows: rows = %d (a multiple of 8 up to %d)", rows, SZ_ROWS_MAX);
    const SzFast fast = sz_fast_path(L);
    if (!fast.exl3 || L->ep_count > 0 || (L->shared_ff > 0 && !fast.shared_fused))
        return sz_fail(SZ_E_TYPE, "sz_moe_rows: EXL3 experts of the streaming kernels' shapes, a shared expert of the same width and type, no expert sharding");
    if (!x || !y || !sz_aligned16(x) || !sz_aligned16(y)) return sz_fail(SZ_E_ARG, "sz_moe_rows: x and y must be non-null and 16-byte aligned");
    const SzRowsScratch S = sz_rows_layout(L);
    if (!scratch || (scratch & 255)) return sz_fail(SZ_E_ARG, "scratch must be 256-byte aligned");
    if (scratch_bytes < S.total) return sz_fail(SZ_E_SCRATCH, "scratch of %lld bytes, %lld needed", (long long)scratch_bytes, (long long)S.total);
    cudaStream_t st = (cudaStream_t)stream;
    u8* base = (u8*)scratch;
    const int H = L->hidden, chunks = rows / 8, W = SZ_ROWS_WIN + SZ_ROWS_SHWIN;
    const bool shared = L->shared_ff > 0;
    u32* ctrl = (u32*)(base + S.ctrl);
    u32* ctrl_x = ctrl + 16 * (SZ_ROWS_MAX / 8);   // the expert kernels' error word lives in word 1 of the block after the chunks'
    float* logits = (float*)(base + S.logits);
    int32_t* ridx = (int32_t*)(base + S.ridx);
    double* rw = (double*)(base + S.rw);
    SzRowsPlan* P = (SzRowsPlan*)(base + S.plan);
    float* xg = (float*)(base + S.xg);
    long long *acc_gu = (long long*)(base + S.acc_gu), *acc_d = (long long*)(base + S.acc_d);
    {   // routing: 8 rows a block row of the verify pass's router kernel (the chunks' own plans are written and not used)
        const int route_rows = L->n_expert + (shared ? 1 : 0);
        const dim3 grid((route_rows + SZ_ROUTE_RB - 1) / SZ_ROUTE_RB, chunks), block(SZ_ROUTE_THREADS);
        const int nch = (H / 4 + SZ_ROUTE_THREADS - 1) / SZ_ROUTE_THREADS;
        cudaError_t e = cudaErrorInvalidValue;
#define SZ_ROWS_ROUTE(NC)                                                                                                                  \
    e = sz_launch("route_rows", sz_route_kernel<8, 8, NC>, grid, block, 0, st, true, (const float*)x, H, (const float*)L->router,           \
                  (const float*)(shared ? L->shared_router : 0), (int)L->n_expert, (int)L->top_k, logits, ridx, rw, (SzPlan*)(base + S.cplan), \
                  (SzPlan*)(base + S.cplan_sh), ctrl, (int32_t*)route_idx, (double*)route_w, (uint4*)nullptr, 0, 0, 0)
        if (nch <= 1) SZ_ROWS_ROUTE(1); else if (nch == 2) SZ_ROWS_ROUTE(2); else SZ_ROWS_ROUTE(4);
#undef SZ_ROWS_ROUTE
        SZ_CUDA(e);
    }
    SZ_CUDA(sz_launch("rows_plan", sz_rows_plan_kernel, dim3(1), dim3(1024), 0, st, true, (const int32_t*)ridx, rows, (int)L->top_k, (int)L->n_expert,
                      shared ? 1 : 0, P));
    SZ_CUDA(sz_launch("rows_zero", sz_rows_zero_kernel, dim3(SZ_ROWS_SLOTS, W), dim3(256), 0, st, true, (const SzRowsPlan*)P, acc_gu, (long long)S.gu_row, acc_d,
                      (long long)S.d_row));
    SZ_CUDA(sz_launch("rows_gather", sz_rows_gather_kernel, dim3(SZ_ROWS_SLOTS, W), dim3(256), 0, st, true, (const float*)x, H, (const SzRowsPlan*)P, xg));
    // the experts: every window a block row of one gate/up and one down launch (how many windows the routing needs is known on the
    // device only: the blocks of a window without groups return at once).  SZ_ROWS_SERIAL=1: a launch pair a window, one after the
    // other (the second form; same bits).
    const size_t win_plan = offsetof(SzRowsPlan, win);
    const char* ser = getenv("SZ_ROWS_SERIAL");   // (read at every call: a test switches it inside one process)
    if (ser && atoi(ser) != 0) {
        for (int w = 0; w < SZ_ROWS_WIN; w++) {
            const SzPlan* pw = (const SzPlan*)((u8*)P + win_plan + (size_t)w * sizeof(SzPlan));
            if ((rc = sz_x3_launch(st, L, 8, pw, xg + (size_t)w * SZ_ROWS_SLOTS * H, acc_gu + (size_t)w * SZ_ROWS_SLOTS * S.gu_row,
                                   acc_d + (size_t)w * SZ_ROWS_SLOTS * S.d_row, ctrl_x, false, true)))
                return rc;
        }
    } else {
        SzXWindows win;
        win.n = SZ_ROWS_WIN; win.x = (long long)SZ_ROWS_SLOTS * H; win.gu = (long long)SZ_ROWS_SLOTS * S.gu_row; win.d = (long long)SZ_ROWS_SLOTS * S.d_row;
        if ((rc = sz_x3_launch(st, L, 8, (const SzPlan*)((u8*)P + win_plan), xg, acc_gu, acc_d, ctrl_x, false, true, win))) return rc;
    }
    if (shared) {   // the shared expert as expert 0 of a layer of one
        sz_moe_layer Ls = *L;
        Ls.gate = L->sh_gate; Ls.up = L->sh_up; Ls.down = L->sh_down;
        Ls.gate_stride = Ls.up_stride = Ls.down_stride = 0;
        Ls.expert_ff = L->shared_ff; Ls.expert_type = L->shared_type;
        const int w = SZ_ROWS_WIN;
        const SzPlan* pw = (const SzPlan*)((u8*)P + win_plan + (size_t)w * sizeof(SzPlan));
        if ((rc = sz_x3_launch(st, &Ls, 8, pw, xg + (size_t)w * SZ_ROWS_SLOTS * H, acc_gu + (size_t)w * SZ_ROWS_SLOTS * S.gu_row,
                               acc_d + (size_t)w * SZ_ROWS_SLOTS * S.d_row, ctrl_x, false, true)))
            return rc;
    }
    SZ_CUDA(sz_launch("rows_combine", sz_rows_combine_kernel, dim3(rows * (H / 128)), dim3((L->top_k + 1) * 32), 0, st, true, (const long long*)acc_d,
                      (const SzRowsPlan*)P, (const int32_t*)ridx, (const double*)rw, (const u8*)L->down, (u64)L->down_stride, (const u8*)L->sh_down,
                      (const float*)logits, (int)L->n_expert, (int)L->top_k, H, (int)L->expert_ff, (int)L->shared_ff, shared ? 1 : 0, (float*)y));
    return SZ_OK;
}

// Clears the scratch's counters (once after allocation, and after a failed call); code != null: reads the expert kernels' error
// word and the plan's overflow flag instead (synchronises).
extern "C" int sz_moe_rows_status(const sz_moe_layer* L, int rows, uint64_t scratch, int* code, uint64_t stream) {
    if (!L || !scratch || rows < 8 || rows > SZ_ROWS_MAX || rows % 8) return sz_fail(SZ_E_ARG, "sz_moe_rows_status: bad argument");
    const SzRowsScratch S = sz_rows_layout(L);
    cudaStream_t st = (cudaStream_t)stream;
    u8* base = (u8*)scratch;
    if (!code) { SZ_CUDA(cudaMemsetAsync(base + S.ctrl, 0, (size_t)(S.logits - S.ctrl), st)); return SZ_OK; }
    u32 err = 0;
    int32_t over = 0;
    SZ_CUDA(cudaMemcpyAsync(&err, base + S.ctrl + 64 * (SZ_ROWS_MAX / 8) + 4, 4, cudaMemcpyDeviceToHost, st));
    SZ_CUDA(cudaMemcpyAsync(&over, base + S.plan + offsetof(SzRowsPlan, overflow), 4, cudaMemcpyDeviceToHost, st));
    SZ_CUDA(cudaStreamSynchronize(st));
    *code = (int)(err ? 1 : 0) | (over & 1 ? 2 : 0) | (over & 4);
    return SZ_OK;
}

extern "C" int sz_moe_verify_host(const sz_moe_layer* L, const float* x_host, int m, float* y_host, int32_t* route_idx_host,
                                  double* route_w_host, uint64_t x_dev, uint64_t y_dev, uint64_t scratch, int64_t scratch_bytes,
                                  uint64_t stream) {
    int rc = sz_moe_check(L, m);
    if (rc) return rc;
    if (!x_host || !y_host || !x_dev || !y_dev) return sz_fail(SZ_E_ARG, "null host or device buffer");
    cudaStream_t st = (cudaStream_t)stream;
    const SzMoeScratch S = sz_moe_layout(L, m);
    const size_t bytes = (size_t)m * L->hidden * sizeof(float);
    SZ_CUDA(cudaMemcpyAsync((void*)x_dev, x_host, bytes, cudaMemcpyHostToDevice, st));
    rc = sz_moe_verify(L, x_dev, m, y_dev, 0, 0, scratch, scratch_bytes, stream);
    if (rc) return rc;
    SZ_CUDA(cudaMemcpyAsync(y_host, (const void*)y_dev, bytes, cudaMemcpyDeviceToHost, st));
    if (route_idx_host)
        SZ_CUDA(cudaMemcpyAsync(route_idx_host, (const u8*)scratch + S.ridx, (size_t)m * L->top_k * 4, cudaMemcpyDeviceToHost, st));
    if (route_w_host)
        SZ_CUDA(cudaMemcpyAsync(route_w_host, (const u8*)scratch + S.rw, (size_t)m * L->top_k * 8, cudaMemcpyDeviceToHost, st));
    u32 err = 0;  // (pageable: this copy is the call's last and the call synchronises anyway)
    SZ_CUDA(cudaMemcpyAsync(&err, (const u8*)scratch + S.ctrl + 4, 4, cudaMemcpyDeviceToHost, st));
    SZ_CUDA(cudaStreamSynchronize(st));
    if (err) return sz_fail(SZ_E_DEVICE, "a bounded wait on an asynchronous copy ran out in a MoE kernel: the results of this call are not valid");
    return SZ_OK;
}

#ifdef SZ_PHASES
extern "C" int sz_phase_read_moe(long long* out) { return cudaMemcpyFromSymbol(out, sz_phase_t, sizeof(long long) * 16 * 16) == cudaSuccess ? 0 : 1; }
#endif

SZ_TIMELINE_READER(moe)
