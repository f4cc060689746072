// Kernels of the verify pass other than the MoE sublayer and the dense projections: embedding rows, hyper-connection glue,
// the DeltaNet front end and state scan, the attention front end (norm, RoPE, Q8_KV write) and the masked attention itself, the
// top-64 of the logits and the greedy acceptance.  Arithmetic follows the CPU reference (crates/shadowzero-model/src/forward.rs);
// sums the reference widens to f64 are f64 here too (FP64 is half rate on this part).
#pragma once

#include "sz_dense.cuh"
#include "sz_topk.cuh"

// A draft tree's tables, as the kernels read them (device memory, written from the pass's staging block).  Row 0 is the root (the
// pass's own token); parents[j] < j.  No counterpart in the reference, whose verify pass is a chain
// (crates/shadowzero-cuda/src/session.rs:7698-7723).
struct SzTree {
    int32_t parents[SZ_MAX_VERIFY];   // parent row, -1 for the root
    int32_t depth[SZ_MAX_VERIFY];     // distance from the root: the row's position is committed + depth
    u32 mask[SZ_MAX_VERIFY];          // bit a: row a is the row itself or one of its ancestors (what it may attend to among the pass's rows)
    u32 save;                         // bit j: a later row branches off row j, so the recurrent state after it is kept
    u32 pad[7];
};
static_assert(sizeof(SzTree) == 128, "the tree tables are 32 words of the staging block");

#ifdef __CUDACC__

// the row `dist` steps up the tree from row j; -1, -2, .. are the committed rows before the pass (most recent first)
__device__ __forceinline__ int sz_tree_up(const SzTree* tr, int j, int dist) {
    if (!tr) return j - dist;
    int a = j;
    for (int s = 0; s < dist; s++) a = a >= 0 ? tr->parents[a] : a - 1;
    return a;
}

__device__ __forceinline__ double sz_block_sum(double v, double* red) {
    v = sz_warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}

// ---- embedding: r[j][s][:] = row ids[j] of token_embd for every stream s (forward.rs:759-767) -----------------------------------
__global__ void __launch_bounds__(256)
sz_embed_kernel(const int32_t* __restrict__ ids, const u8* __restrict__ embd, int type, int H, int C, int vocab, float* __restrict__ r) {
    __shared__ u32 grid[512];
    sz_pdl_wait();
    sz_pdl_trigger();
    for (int i = threadIdx.x; i < 512; i += 256) grid[i] = c_iq3s_grid[i];
    __syncthreads();
    const int j = blockIdx.x;
    int tok = ids[j];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const u8* row = embd + (size_t)tok * sz_dense_row_bytes(type, H);
    for (int e = 4 * threadIdx.x; e < H; e += 1024) {
        float w[4], sc;
        sz_dense_w4(type, row, e, grid, w, sc);
        const float4 v = make_float4(sc * w[0], sc * w[1], sc * w[2], sc * w[3]);
        for (int s = 0; s < C; s++) *(float4*)(r + ((size_t)j * C + s) * H + e) = v;
    }
}

// ---- hyper-connection: (pending write) r[s] += g[s] * y, then rn[s] = rmsnorm(r[s]) * w[s] (forward.rs:801,1078-1084) ----------
// grid (C, m)
__global__ void __launch_bounds__(256)
sz_hc_norm_kernel(float* __restrict__ r, const float* __restrict__ g, const float* __restrict__ y, const float* __restrict__ w, int H,
                  int C, float eps, float* __restrict__ rn) {
    __shared__ double red[8];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int s = blockIdx.x, j = blockIdx.y;
    float* rs = r + ((size_t)j * C + s) * H;
    const float gs = g ? g[j * C + s] : 0.f;
    double ss = 0.0;
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = rs[i];
        if (y) { v = v + gs * y[(size_t)j * H + i]; rs[i] = v; }
        ss += (double)v * (double)v;
    }
    ss = sz_block_sum(ss, red);
    const double rr = sz_rsqrt64(ss / (double)H + (double)eps);
    for (int i = threadIdx.x; i < H; i += 256) rn[((size_t)j * C + s) * H + i] = (float)((double)rs[i] * rr) * w[s * H + i];
}

// u[i] = (sum over streams of mix[s][i] * rn[s][i]) / C in f32, stream order (forward.rs:805-811).  grid (ceil(H / 256), m)
__global__ void __launch_bounds__(256)
sz_hc_mix_kernel(const float* __restrict__ mix, const float* __restrict__ rn, int H, int C, float* __restrict__ u) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int i = blockIdx.x * 256 + threadIdx.x, j = blockIdx.y;
    if (i >= H) return;
    float a = 0.f;
    for (int s = 0; s < C; s++) a += mix[((size_t)j * C + s) * H + i] * rn[((size_t)j * C + s) * H + i];
    u[(size_t)j * H + i] = a / (float)C;
}

// ---- hyper-connection read, fused form ---------------------------------------------------------------------------------------------
// Two launches a read instead of four.  The work is split so that every weight byte is requested at once and the activation rows a
// block stages are small:
//   down kernel: block b owns columns [64 b, 64 b + 64) of the C*H-wide input (all inside one stream s).  Each thread keeps one row
//   slice of the down (or inject) matrix - 128 contiguous bytes - in registers, fetched before the dependency wait.  The block
//   applies the pending residual write to stream s of every row, takes the stream's RMS (every block of a stream computes the same
//   sum in the same order), writes its 64 columns of the new residual and of rn, and adds its partial dot products to a fixed-point
//   accumulator (64-bit integer atomics: the total does not depend on the order the blocks arrive in).
//   up kernel: block b owns 16 positions h of the hidden dimension and the C rows s*H + h of the up matrix for each (512-byte rows
//   at rank 256, one 16-byte piece a lane, all in flight before the wait), turns the accumulator into silu(down / C), and finishes
//   u[h] = mean over streams of sigmoid(up row) * rn in the same block.
// Residual streams ping-pong between two buffers (a block reads the whole stream while its neighbours write their columns); the
// accumulator rotates over three (this read's, the previous read's - it holds the inject gates the pending write needs - and the
// next read's, which block 0 clears).
#define SZ_HC_ACC_ROWS 272                    // rank + streams, padded
#define SZ_HC_FIX 1099511627776.0             // 2^40
#define SZ_HC_FIX_INV (1.0 / 1099511627776.0)

// grid C*H / 64; block: a multiple of 32 threads, at least rank + C (one thread a matrix row) and at most 320
// this thread's 64 weights of the down (or inject) matrix: constant data, requested before the dependency wait
__device__ __forceinline__ const u8* sz_hc_down_fetch(const u8* __restrict__ down, const u8* __restrict__ inject, int H, int C, int rank, uint4* w) {
    const int t = threadIdx.x, CH = C * H, c0 = blockIdx.x * 64;
    const u8* wrow = nullptr;
    if (c0 < CH) {
        if (t < rank) wrow = down + ((size_t)t * CH + c0) * 2;
        else if (inject != nullptr && t < rank + C) wrow = inject + ((size_t)(t - rank) * CH + c0) * 2;
    }
#pragma unroll
    for (int i = 0; i < 8; i++) w[i] = wrow ? sz_ldg16_here((const uint4*)wrow + i) : make_uint4(0, 0, 0, 0);
    return wrow;
}

// everything after the wait; every thread of the block returns from it together (no early exits: a grid-wide barrier may follow)
template <int M>  // rows of the pass: a compile-time count keeps every per-row loop free of branches
__device__ __forceinline__ void
sz_hc_down_body(const float* __restrict__ r_in, float* __restrict__ r_out, const long long* __restrict__ g_acc, const float* __restrict__ y,
                const float* __restrict__ normw, int H, int C, int rank, float eps, float* __restrict__ rn, long long* __restrict__ acc,
                long long* __restrict__ acc_next, const u8* wrow, const uint4* w) {
    __shared__ double red[10][SZ_MAX_VERIFY];
    __shared__ float rinv[SZ_MAX_VERIFY];
    __shared__ float gs[SZ_MAX_VERIFY];
    __shared__ __align__(16) float xs[SZ_MAX_VERIFY][64];
    __shared__ float nws[64];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31, nt = blockDim.x;
    const int CH = C * H;
    const int c0 = blockIdx.x * 64;
    SZ_PH_DECL;
    const int s = c0 / H;
    SZ_PH();  // 1 after wait
    // every load of the prologue is issued before anything waits on one: the gates, the stream's rows, the mixer output
    if (t < 64) nws[t] = __ldg(normw + c0 + t);
    long long graw = 0;
    if (g_acc && t < M) graw = __ldcg(g_acc + t * SZ_HC_ACC_ROWS + rank + s);
    constexpr int NV = 2;  // float4 pieces of a stream row a thread holds: covers H <= 8 * blockDim
    float4 rv[M][NV], yv[M][NV];
#pragma unroll
    for (int j = 0; j < M; j++) {
#pragma unroll
        for (int q = 0; q < NV; q++) {
            const int i = t + q * nt;
            const bool on = i < H / 4;
            rv[j][q] = on ? __ldcg((const float4*)(r_in + ((size_t)j * C + s) * H) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            yv[j][q] = on && g_acc ? __ldcg((const float4*)(y + (size_t)j * H) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (blockIdx.x == 0) {   // (a block row of a grid over many rows clears its own rows only: its neighbours clear theirs)
        const int clr = (gridDim.y > 1 ? M : SZ_MAX_VERIFY) * SZ_HC_ACC_ROWS;
        for (int i = t; i < clr; i += nt) acc_next[i] = 0;
    }
    if (t < M) gs[t] = g_acc ? 2.0f * sz_sigmoid((float)((double)graw * SZ_HC_FIX_INV) / (float)C) : 0.f;
    __syncthreads();
    SZ_PH();  // 2 gates
    // the pending write, the stream's sum of squares for every row, and this block's 64 columns of the new residual
    const int lo4 = (c0 - s * H) / 4;  // first float4 of the block's columns inside the stream
#pragma unroll
    for (int j = 0; j < M; j++) {
        double ss = 0.0;
        if (j < M) {
            const float g = gs[j];
#pragma unroll
            for (int q = 0; q < NV; q++) {
                const int i = t + q * nt;
                float4 v = rv[j][q];
                const float4 w4 = yv[j][q];
                v.x = v.x + g * w4.x; v.y = v.y + g * w4.y; v.z = v.z + g * w4.z; v.w = v.w + g * w4.w;
                ss += (double)v.x * (double)v.x;
                ss += (double)v.y * (double)v.y;
                ss += (double)v.z * (double)v.z;
                ss += (double)v.w * (double)v.w;
                if (i >= lo4 && i < lo4 + 16) *(float4*)&xs[j][4 * (i - lo4)] = v;
            }
            ss = sz_warp_sum(ss);
            if (lane == 0) red[warp][j] = ss;
        }
    }
    __syncthreads();
    SZ_PH();  // 3 sums
    if (t < M) {
        double v = 0.0;
        for (int q = 0; q < (nt >> 5); q++) v += red[q][t];
        rinv[t] = (float)sz_rsqrt64(v / (double)H + (double)eps);
    }
    __syncthreads();
    SZ_PH();  // 4 rinv
    // this block's 64 columns: the new residual and rn (to memory for the up kernel, to shared memory for the dot products)
    for (int idx = t; idx < M * 64; idx += nt) {
        const int j = idx >> 6, c = idx & 63;
        const size_t at = (size_t)j * CH + c0 + c;
        const float v = xs[j][c];
        r_out[at] = v;
        const float x = (float)((double)v * (double)rinv[j]) * nws[c];
        rn[at] = x;
        xs[j][c] = x;
    }
    __syncthreads();
    SZ_PH();  // 5 columns
    if (wrow != nullptr) {
        float a[M];
#pragma unroll
        for (int j = 0; j < M; j++) a[j] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const u32 ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float w0 = __uint_as_float(ww[q] << 16), w1 = __uint_as_float(ww[q] & 0xffff0000u);
#pragma unroll
                for (int j = 0; j < M; j++) {
                    if (j < M) {
                        const float2 xv = *(const float2*)&xs[j][8 * i + 2 * q];
                        a[j] = fmaf(w0, xv.x, a[j]);
                        a[j] = fmaf(w1, xv.y, a[j]);
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < M; j++)
            if (j < M) atomicAdd((unsigned long long*)(acc + j * SZ_HC_ACC_ROWS + t), (unsigned long long)__double2ll_rn((double)a[j] * SZ_HC_FIX));
    }
    SZ_PH();  // 6 dots + atomics issued
    SZ_PH_FLUSH(1, blockIdx.x == 5);
}

template <int M>
__global__ void __launch_bounds__(320)
sz_hc_down_kernel(const float* __restrict__ r_in, float* __restrict__ r_out, const long long* __restrict__ g_acc, const float* __restrict__ y,
                  const float* __restrict__ normw, const u8* __restrict__ down, const u8* __restrict__ inject, int H, int C, int rank,
                  float eps, float* __restrict__ rn, long long* __restrict__ acc, long long* __restrict__ acc_next) {
    uint4 w[8];
    const u8* wrow = sz_hc_down_fetch(down, inject, H, C, rank, w);
    sz_pdl_wait();
    sz_pdl_trigger();
    // grid.y > 1: block row g serves rows [g M, g M + M) of buffers that hold the rows of several sequences one after the other
    const size_t g = (size_t)blockIdx.y * M;
    sz_hc_down_body<M>(r_in + g * C * H, r_out + g * C * H, g_acc ? g_acc + g * SZ_HC_ACC_ROWS : nullptr, y + g * H, normw, H, C, rank, eps,
                       rn + g * C * H, acc + g * SZ_HC_ACC_ROWS, acc_next + g * SZ_HC_ACC_ROWS, wrow, w);
}

// ---- the first half of the read over MANY rows (a batch of sequences) ------------------------------------------------------------------
// sz_hc_down_kernel makes every one of a stream's H / 64 blocks load the whole stream of its rows and sum its squares - nothing
// for the few rows of a pass, 32 times the work when a launch carries the rows of many sequences.  Here that part runs once a
// (row, stream) - sz_hc_rows_norm_kernel: the pending write, the sum of squares in the very order of the kernel above (the same
// block size, the same float4 a thread, warp sums, then the warps in order), the new residual and rn - and sz_hc_rows_down_kernel
// only multiplies: a block's 64 columns of rn for 8 rows, the thread's 64 weights, the same chain of multiply-adds, the same
// fixed-point sums.  Bit for bit the kernel above's results.
// grid (streams, rows); block: as sz_hc_down_kernel's (the order of the sum of squares depends on it)
__global__ void __launch_bounds__(320)
sz_hc_rows_norm_kernel(const float* __restrict__ r_in, float* __restrict__ r_out, const long long* __restrict__ g_acc, const float* __restrict__ y,
                       const float* __restrict__ normw, int H, int C, int rank, float eps, float* __restrict__ rn, long long* __restrict__ acc_next) {
    __shared__ double red[10];
    __shared__ float rinv_s, gs_s;
    sz_pdl_wait();
    sz_pdl_trigger();
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31, nt = blockDim.x;
    const int s = blockIdx.x, row = blockIdx.y;
    constexpr int NV = 2;
    float4 rv[NV], yv[NV];
#pragma unroll
    for (int q = 0; q < NV; q++) {
        const int i = t + q * nt;
        const bool on = i < H / 4;
        rv[q] = on ? __ldcg((const float4*)(r_in + ((size_t)row * C + s) * H) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        yv[q] = on && g_acc ? __ldcg((const float4*)(y + (size_t)row * H) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (s == 0)
        for (int i = t; i < SZ_HC_ACC_ROWS; i += nt) acc_next[(size_t)row * SZ_HC_ACC_ROWS + i] = 0;
    if (t == 0) {
        const long long graw = g_acc ? __ldcg(g_acc + (size_t)row * SZ_HC_ACC_ROWS + rank + s) : 0;
        gs_s = g_acc ? 2.0f * sz_sigmoid((float)((double)graw * SZ_HC_FIX_INV) / (float)C) : 0.f;
    }
    __syncthreads();
    const float g = gs_s;
    double ss = 0.0;
#pragma unroll
    for (int q = 0; q < NV; q++) {
        float4 v = rv[q];
        const float4 w4 = yv[q];
        v.x = v.x + g * w4.x; v.y = v.y + g * w4.y; v.z = v.z + g * w4.z; v.w = v.w + g * w4.w;
        ss += (double)v.x * (double)v.x;
        ss += (double)v.y * (double)v.y;
        ss += (double)v.z * (double)v.z;
        ss += (double)v.w * (double)v.w;
        rv[q] = v;
    }
    ss = sz_warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (t == 0) {
        double v = 0.0;
        for (int q = 0; q < (nt >> 5); q++) v += red[q];
        rinv_s = (float)sz_rsqrt64(v / (double)H + (double)eps);
    }
    __syncthreads();
    const float rinv = rinv_s;
#pragma unroll
    for (int q = 0; q < NV; q++) {
        const int i = t + q * nt;
        if (i < H / 4) {
            const size_t at = ((size_t)row * C + s) * H + 4 * (size_t)i;
            const float4 v = rv[q];
            const float4 nw = __ldg((const float4*)(normw + (size_t)s * H) + i);
            float4 x;
            x.x = (float)((double)v.x * (double)rinv) * nw.x;
            x.y = (float)((double)v.y * (double)rinv) * nw.y;
            x.z = (float)((double)v.z * (double)rinv) * nw.z;
            x.w = (float)((double)v.w * (double)rinv) * nw.w;
            *(float4*)(r_out + at) = v;
            *(float4*)(rn + at) = x;
        }
    }
}

// grid (C * H / 64, rows / M); block: as sz_hc_down_kernel's (one thread a row of the down / inject matrices)
template <int M>
__global__ void __launch_bounds__(320)
sz_hc_rows_down_kernel(const float* __restrict__ rn, const u8* __restrict__ down, const u8* __restrict__ inject, int H, int C, int rank,
                       long long* __restrict__ acc) {
    __shared__ __align__(16) float xs[M][64];
    uint4 w[8];
    const u8* wrow = sz_hc_down_fetch(down, inject, H, C, rank, w);
    sz_pdl_wait();
    sz_pdl_trigger();
    const int t = threadIdx.x, nt = blockDim.x, CH = C * H, c0 = blockIdx.x * 64;
    const size_t g = (size_t)blockIdx.y * M;
    for (int idx = t; idx < M * 64; idx += nt) {
        const int j = idx >> 6, c = idx & 63;
        xs[j][c] = __ldcg(rn + (g + j) * CH + c0 + c);
    }
    __syncthreads();
    if (wrow != nullptr) {
        float a[M];
#pragma unroll
        for (int j = 0; j < M; j++) a[j] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const u32 ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float w0 = __uint_as_float(ww[q] << 16), w1 = __uint_as_float(ww[q] & 0xffff0000u);
#pragma unroll
                for (int j = 0; j < M; j++) {
                    const float2 xv = *(const float2*)&xs[j][8 * i + 2 * q];
                    a[j] = fmaf(w0, xv.x, a[j]);
                    a[j] = fmaf(w1, xv.y, a[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < M; j++)
            atomicAdd((unsigned long long*)(acc + (g + j) * SZ_HC_ACC_ROWS + t), (unsigned long long)__double2ll_rn((double)a[j] * SZ_HC_FIX));
    }
}

// grid H / 16, block 256.  CPR = rank / 8: 16-byte pieces a row of the up matrix.
// the block's rows of the up matrix, one 16-byte piece a thread and slot: constant data, requested before the dependency wait
// (threads 256 and up of a wider block hold none)
__device__ __forceinline__ void sz_hc_up_fetch(const u8* __restrict__ up, int H, int C, int rank, uint4* w) {
    const int t = threadIdx.x, cpr = rank >> 3, h0 = blockIdx.x * 16;
    // piece t + 256 i of the block's rows: cpr divides 256, so the thread's place c in a row is the same for every i and the row
    // advances by 256 / cpr (one division here instead of one a slot)
    const int lr0 = t / cpr, c = t - lr0 * cpr, step = 256 / cpr;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int lr = lr0 + step * i;                        // local row s * 16 + hl
        w[i] = make_uint4(0, 0, 0, 0);
        if (t < 256 && lr < 16 * C && h0 < H) {
            const int row = (lr >> 4) * H + h0 + (lr & 15);
            w[i] = sz_ldg16_here((const uint4*)(up + (size_t)row * rank * 2) + c);
        }
    }
}

// One level of the reduce-scatter over the lanes of a row (see sz_hc_up_body).  Before level LVL a lane holds sz_hc_up_held(N, LVL)
// values: an even count is halved - the lane keeps the half its bit `o` of the lane's place selects, adds the partner's partial of
// those, and hands over the other half - an odd count (a pass of 3, 5, 6 or 7 rows gets there) stays whole and both sides add, as
// a butterfly level does.  o == 0: the row has fewer lanes than that, nothing to do.
__host__ __device__ constexpr int sz_hc_up_held(int n, int levels) {
    for (int l = 0; l < levels; l++)
        if (n % 2 == 0) n /= 2;
    return n;
}
template <int N, int LVL>
__device__ __forceinline__ void sz_hc_up_level(float* v, int o, int place, int& base) {
    if (o <= 0) return;
    constexpr int n = sz_hc_up_held(N, LVL);
    if constexpr (n % 2 == 0) {
        constexpr int h = n / 2;
        const bool up = (place & o) != 0;
#pragma unroll
        for (int k = 0; k < h; k++) {
            const float lo = v[k], hi = v[k + h];
            const float send = up ? lo : hi, keep = up ? hi : lo;
            v[k] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
        if (up) base += h;
    } else {
#pragma unroll
        for (int k = 0; k < n; k++) v[k] += __shfl_xor_sync(0xffffffffu, v[k], o);
    }
}

// everything after the wait, for the first 256 threads of the block (all of them reach every barrier inside)
template <int M>
__device__ __forceinline__ void
sz_hc_up_body(const long long* __restrict__ acc, const float* __restrict__ rn, int H, int C, int rank, float* __restrict__ u, const uint4* w) {
    __shared__ __align__(16) float hd[SZ_MAX_VERIFY][256];
    __shared__ float mixs[64][SZ_MAX_VERIFY];
    const int t = threadIdx.x;
    const int cpr = rank >> 3;
    const int h0 = blockIdx.x * 16;
    const int lr0 = t / cpr, c = t - lr0 * cpr, step = 256 / cpr;   // (as sz_hc_up_fetch: the thread's place in a row, its first row)
    SZ_PH_DECL;
    SZ_PH();  // 1
    const bool on = t < 256;   // a wider block's extra warps only keep the barriers company
    if (on) {
#pragma unroll
        for (int j = 0; j < M; j++)
            for (int q = t; q < rank; q += 256) {
                const float v = (float)((double)__ldcg(acc + j * SZ_HC_ACC_ROWS + q) * SZ_HC_FIX_INV);
                hd[j][q] = sz_silu(v / (float)C);
            }
    }
    __syncthreads();
    SZ_PH();  // 2 hd
    // all partial dot products first, then the butterflies over the cpr lanes of a row interleaved (independent chains).  A thread's
    // pieces all sit at the same place c of their rows (256 is a multiple of cpr), so its 8 inputs per row are read once.
    if (on) {
        float p[8][M];
        {
            float4 x0[M], x1[M];
#pragma unroll
            for (int j = 0; j < M; j++) { x0[j] = *(const float4*)&hd[j][8 * c]; x1[j] = *(const float4*)&hd[j][8 * c + 4]; }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const u32 ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
                float wf[8];
#pragma unroll
                for (int q = 0; q < 4; q++) { wf[2 * q] = __uint_as_float(ww[q] << 16); wf[2 * q + 1] = __uint_as_float(ww[q] & 0xffff0000u); }
#pragma unroll
                for (int j = 0; j < M; j++) {
                    float v = wf[0] * x0[j].x;
                    v = fmaf(wf[1], x0[j].y, v); v = fmaf(wf[2], x0[j].z, v); v = fmaf(wf[3], x0[j].w, v);
                    v = fmaf(wf[4], x1[j].x, v); v = fmaf(wf[5], x1[j].y, v); v = fmaf(wf[6], x1[j].z, v); v = fmaf(wf[7], x1[j].w, v);
                    p[i][j] = v;
                }
            }
        }
        // The sums over the cpr lanes of a row: a butterfly's additions (lane with lane ^ 16, then ^ 8, .. ^ 1: every sum the same
        // tree), but each level hands half of the lane's values to the partner instead of summing all of them on both sides - a
        // reduce-scatter: about 8 M shuffles a thread instead of 8 M log2(cpr) - and every lane ends with its share of the finished
        // sums (a + b on one side is b + a on the other: the bits are the butterfly's).
        float* v = &p[0][0];          // value i * M + j
        int base = 0;                 // the first of the values this lane still holds
        sz_hc_up_level<8 * M, 0>(v, cpr >> 1, c, base);
        sz_hc_up_level<8 * M, 1>(v, cpr >> 2, c, base);
        sz_hc_up_level<8 * M, 2>(v, cpr >> 3, c, base);
        sz_hc_up_level<8 * M, 3>(v, cpr >> 4, c, base);
        sz_hc_up_level<8 * M, 4>(v, cpr >> 5, c, base);
        int held = 8 * M;             // values a lane ends with
        for (int o = cpr >> 1; o > 0; o >>= 1)
            if (!(held & 1)) held >>= 1;
#pragma unroll
        for (int k = 0; k < 8 * M; k++) {
            if (k < held) {
                const int idx = base + k, i = idx / M, j = idx - i * M;
                const int lr = lr0 + step * i;
                if (lr < 16 * C) mixs[lr][j] = v[k];
            }
        }
    }
    __syncthreads();
    SZ_PH();  // 3 dots
    // mix * rn for each (stream, position, row), one a thread; then the mean over the streams
    if (on)
        for (int idx = t; idx < 16 * C * M; idx += 256) {
            const int lr = idx / M, j = idx - lr * M;
            mixs[lr][j] = sz_sigmoid(mixs[lr][j]) * __ldcg(rn + ((size_t)j * C + (lr >> 4)) * H + h0 + (lr & 15));
        }
    __syncthreads();
    if (on)
        for (int idx = t; idx < M * 16; idx += 256) {
            const int j = idx >> 4, hl = idx & 15;
            float a = 0.f;
            for (int s = 0; s < C; s++) a += mixs[s * 16 + hl][j];
            u[(size_t)j * H + h0 + hl] = a / (float)C;
        }
    SZ_PH();  // 4 u
    SZ_PH_FLUSH(2, blockIdx.x == 5);
}

template <int M>
__global__ void __launch_bounds__(256)
sz_hc_up_kernel(const long long* __restrict__ acc, const u8* __restrict__ up, const float* __restrict__ rn, int H, int C, int rank,
                float* __restrict__ u) {
    uint4 w[8];
    sz_hc_up_fetch(up, H, C, rank, w);
    sz_pdl_wait();
    sz_pdl_trigger();
    const size_t g = (size_t)blockIdx.y * M;   // (as the down kernel)
    sz_hc_up_body<M>(acc + g * SZ_HC_ACC_ROWS, rn + g * C * H, H, C, rank, u + g * H, w);
}

// A barrier over all blocks of a grid whose blocks are all resident (no more blocks than the GPU holds at once: the caller sizes
// the grid so).  sync[0] counts arrivals, sync[1] is the generation: the last block to arrive clears the count and bumps the
// generation, the others poll it - a bounded number of times, after which the block raises *err and goes on (its results are then
// wrong and flagged; nothing ever spins for good).  Writes before the barrier are visible to every block after it.
__device__ __forceinline__ void sz_grid_barrier(u32* sync, u32 blocks, u32* err) {
    __syncthreads();
    if (threadIdx.x == 0) {
        u32 gen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(sync + 1));
        __threadfence();
        const u32 arrived = atomicAdd(sync, 1u);
        if (arrived == blocks - 1) {
            atomicExch(sync, 0u);
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(sync + 1), "r"(gen + 1) : "memory");
        } else {
            u32 now = gen;
            int polls = 0;
            while (now == gen && polls < 2000000) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(now) : "l"(sync + 1));
                polls++;
                if (polls > 64) __nanosleep(40);
            }
            if (now == gen && err) atomicExch(err, 1u);
        }
        __threadfence();
    }
    __syncthreads();
}

// The whole read in one launch: the down half, a grid-wide barrier, the up half.  grid = max(C H / 64, H / 16) blocks (one a
// multiprocessor at most: the barrier needs them all resident), block = the down half's.  Both halves' weights are requested ahead
// of the dependency wait, so the up matrix arrives while the down half runs.
template <int M>
__global__ void __launch_bounds__(320)
sz_hc_read_kernel(const float* __restrict__ r_in, float* __restrict__ r_out, const long long* __restrict__ g_acc, const float* __restrict__ y,
                  const float* __restrict__ normw, const u8* __restrict__ down, const u8* __restrict__ inject, const u8* __restrict__ up, int H,
                  int C, int rank, float eps, float* __restrict__ rn, long long* __restrict__ acc, long long* __restrict__ acc_next,
                  float* __restrict__ u, u32* __restrict__ sync, u32* __restrict__ err) {
    uint4 wd[8], wu[8];
    const u8* wrow = sz_hc_down_fetch(down, inject, H, C, rank, wd);
    sz_hc_up_fetch(up, H, C, rank, wu);
    sz_pdl_wait();
    sz_pdl_trigger();
    if ((int)blockIdx.x * 64 < C * H) sz_hc_down_body<M>(r_in, r_out, g_acc, y, normw, H, C, rank, eps, rn, acc, acc_next, wrow, wd);
    sz_grid_barrier(sync, gridDim.x, err);
    if ((int)blockIdx.x * 16 < H) sz_hc_up_body<M>(acc, rn, H, C, rank, u, wu);
}

// ---- DeltaNet front end (forward.rs:829-861): causal conv (k taps) + SiLU over the rows of the pass, L2 norm of q and k heads,
// beta and decay.  grid (ch / 256, m), block 256: a block takes 256 channels - whole heads, since the head width divides 256 - of
// one row.  conv0 / conv1: (k-1) x ch, oldest first: the state BEFORE the pass (state[1] says which).  xin: [m][ch] raw projections.
__global__ void __launch_bounds__(256)
sz_delta_prep_kernel(const float* __restrict__ xin, const float* __restrict__ conv0, const float* __restrict__ conv1, const int32_t* __restrict__ state,
                     const float* __restrict__ cw, const float* __restrict__ b,
                     const float* __restrict__ a, const float* __restrict__ a_log, const float* __restrict__ dt, int kh, int vh, int d, int k,
                     float* __restrict__ xc, float* __restrict__ beta, float* __restrict__ decay) {
    __shared__ double sred[8];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int j = blockIdx.y;
    const int kd = kh * d, ch = 2 * kd + vh * d;
    const float* conv = state[1] ? conv1 : conv0;  // the carried rows of the current state buffer
    const int i = blockIdx.x * 256 + threadIdx.x;
    float v = 0.f;
    if (i < ch) {
        double acc = (double)cw[i * k + (k - 1)] * (double)xin[(size_t)j * ch + i];
        for (int t = 0; t < k - 1; t++) {
            const int tau = j - (k - 1) + t;  // row of this pass, or (negative) a row of the carried state
            const float prev = tau >= 0 ? xin[(size_t)tau * ch + i] : conv[(size_t)((k - 1) + tau) * ch + i];
            acc += (double)cw[i * k + t] * (double)prev;
        }
        v = sz_silu((float)acc);
    }
    // L2 norm of the q and k heads (q also / sqrt(d)): squares summed per warp, then over the warps of the head
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const double sq = sz_warp_sum((double)v * (double)v);
    if (lane == 0) sred[warp] = sq;
    __syncthreads();
    if (i < ch) {
        if (i < 2 * kd) {
            double ss;
            if (d >= 32) {
                const int w0 = (threadIdx.x / d) * (d / 32);
                ss = 0.0;
                for (int t = 0; t < d / 32; t++) ss += sred[w0 + t];
            } else {  // heads narrower than a warp: sum inside the warp's head segment
                ss = (double)v * (double)v;
                for (int o = d >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            }
            const double n = sz_rsqrt64(ss + 1e-6);
            float t = (float)((double)v * n);
            if (i < kd) t = t / sqrtf((float)d);
            v = t;
        }
        xc[(size_t)j * ch + i] = v;
    }
    if (blockIdx.x == 0) {
        for (int h = threadIdx.x; h < vh; h += 256) {
            beta[j * vh + h] = sz_sigmoid(b[j * vh + h]);
            const float sp_in = a[j * vh + h] + dt[h];
            const float sp = sp_in > 20.0f ? sp_in : log1pf(expf(sp_in));
            decay[j * vh + h] = expf(a_log[h] * sp);
        }
    }
}

// The carried conv rows after the kept rows of the pass: the last k-1 of [state rows ; xin rows 0..keep-1], for every DeltaNet layer.
// grid (k-1, n_delta), block 256.  res[0] = rows kept; nothing is written when it is 0.
__global__ void __launch_bounds__(256)
sz_conv_commit_kernel(const float* __restrict__ conv0, const float* __restrict__ conv1, const int32_t* __restrict__ state,
                      const int32_t* __restrict__ res, const float* __restrict__ xin_all, int ch, int k, float* __restrict__ out0,
                      float* __restrict__ out1, int tree) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int keep = res[0];
    if (keep <= 0) return;
    const int cur = state[1];
    const int t = blockIdx.x, di = blockIdx.y;  // row of the new state, oldest first
    const size_t cl = (size_t)(k - 1) * ch;
    const float* conv = (cur ? conv1 : conv0) + di * cl;
    float* dst = (cur ? out0 : out1) + di * cl;   // the other buffer
    const float* xin = xin_all + (size_t)di * SZ_MAX_VERIFY * ch;
    const int tau = keep - (k - 1) + t;    // index into the kept rows, negative: into the old state
    // (the kept rows of a tree pass are the path res[2 ..]; of a chain, rows 0 .. keep - 1)
    const float* src = tau >= 0 ? xin + (size_t)(tree ? res[2 + tau] : tau) * ch : conv + (size_t)((k - 1) + tau) * ch;
    for (int i = threadIdx.x; i < ch; i += 256) dst[(size_t)t * ch + i] = src[i];
}

// After the commit kernels: positions += kept rows, and the state buffers swap.
__global__ void sz_state_update_kernel(int32_t* __restrict__ state, const int32_t* __restrict__ res) {
    sz_pdl_wait();
    sz_pdl_trigger();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const int keep = res[0];
        if (keep > 0) { state[0] += keep; state[1] ^= 1; }
    }
}

// ---- DeltaNet state scan (forward.rs:859-894): per value head, the d x d state column-resident in registers.
// Thread (col = tid % D, part = tid / D) holds S[i][col] for the i of its part.  grid (vh, layers), block D * PARTS.
// Reads the state of the current buffer (state[1]) and writes the other one.  With `og` != null it applies all m rows and writes
// the gated, normalised outputs (the pass itself, one layer: blockIdx.y = 0 and the pointers are that layer's).  With og == null it
// is the replay of a commit: layer blockIdx.y of every per-layer array, only the res[0] kept rows, and nothing at all when every
// row was kept (the pass already wrote that state) or none was.
// In the pass itself (og != null) the block also does the front end for the channels it needs - q and k of its key head, v of its
// own head: causal conv + SiLU, L2 norms, beta and decay (what sz_delta_prep_kernel does for a whole row) - so the layer needs no
// launch between the projections and the scan.  It leaves the conv outputs, beta and decay where the replay of a commit reads them.
struct SzDeltaPrep {
    const float* xin;     // [m][ch] raw projections of this layer (null: the front end already ran as a kernel of its own)
    const float* conv0;   // (k - 1) x ch carried rows, two buffers
    const float* conv1;
    const float* cw;      // [ch][k] conv taps
    const float* b;       // [m][vh]
    const float* a;       // [m][vh]
    const float* a_log;   // [vh]
    const float* dt;      // [vh]
    float* xc;            // [m][ch] out
    float* beta;          // [m][vh] out
    float* decay;         // [m][vh] out
    int k;
};

// (the kernel's body: block (hd, di) of the grid described above)
template <int D, int PARTS>
__device__ __forceinline__ void
sz_delta_scan_body(const float* __restrict__ xc_all, const float* __restrict__ beta_all, const float* __restrict__ decay_all,
                   const float* __restrict__ z, const float* __restrict__ norm_w, const float* __restrict__ S0, const float* __restrict__ S1,
                   float* __restrict__ O0, float* __restrict__ O1, const int32_t* __restrict__ state, const int32_t* __restrict__ res, int kh,
                   int vh, int m, float eps, float* __restrict__ og, const SzDeltaPrep& pp, const SzTree* __restrict__ tr,
                   float* __restrict__ fork, const int hd, const int di) {
    constexpr int NI = D / PARTS;
    constexpr int RUN = NI < 16 ? NI : 16;  // sums run in f32 over 16 terms and the runs are added in f64, as the reference's exact
                                            // GPU scan does (kernels/forward.cu:991-1013): a conversion to f64 per term would
                                            // keep the conversion unit busy for longer than the state takes to arrive
    __shared__ float sk[D], sq[D];
    __shared__ double part[PARTS][D];
    __shared__ float ofs[SZ_MAX_VERIFY][D];
    __shared__ double rrs[SZ_MAX_VERIFY];
    __shared__ float pbuf[SZ_MAX_VERIFY][3][D];   // the rows' q, k, v after the front end
    __shared__ float sbeta[SZ_MAX_VERIFY], sdecay[SZ_MAX_VERIFY];
    const int col = threadIdx.x % D, pt = threadIdx.x / D;
    const int kx = hd % kh;  // value heads are tiled over the key heads (forward.rs:862-864)
    const int kd = kh * D, ch = 2 * kd + vh * D;
    const size_t Sl = (size_t)vh * D * D;
    float S[NI];
    // the state belongs to the previous pass (and the buffer index with it): in the pass itself it is fetched ahead of the wait
    if (og) {
        const int cur0 = state[1];
        const float* Sg = (cur0 ? S1 : S0) + di * Sl + (size_t)hd * D * D;
#pragma unroll
        for (int i = 0; i < NI; i++) S[i] = sz_ld32_here(Sg + (size_t)(pt * NI + i) * D + col);
    }
    sz_pdl_wait();
    sz_pdl_trigger();
    // A tree pass (tr != null): a row continues from the state after its PARENT.  Rows come parents first, so the state after a row
    // that a later row branches off (tr->save) is kept in `fork` ([value head][row][D * D]) and fetched when a row's parent is not the
    // row just before it.  The state the pass leaves in the other buffer is then that of no one path: the commit of a tree pass
    // always replays, along the kept path res[2 ..] (row indices), where a chain's kept rows are simply 0 .. res[0] - 1.
    int rows = m;
    if (!og) {
        rows = res[0];
        if (rows <= 0 || (!tr && rows >= m)) return;
    }
    const int cur = state[1];
    const float* S_in = (cur ? S1 : S0) + di * Sl;
    float* S_out = (cur ? O0 : O1) + di * Sl;
    const float* xc = xc_all + (size_t)di * SZ_MAX_VERIFY * ch;
    const float* beta = beta_all + (size_t)di * SZ_MAX_VERIFY * vh;
    const float* decay = decay_all + (size_t)di * SZ_MAX_VERIFY * vh;
    if (!og) {
        const float* Sg = S_in + (size_t)hd * D * D;
#pragma unroll
        for (int i = 0; i < NI; i++) S[i] = Sg[(size_t)(pt * NI + i) * D + col];
    }
    const bool fused = og != nullptr && pp.xin != nullptr;
    if (fused) {
        // ---- front end for this block's channels (forward.rs:829-861)
        const float* conv = cur ? pp.conv1 : pp.conv0;
        const int k = pp.k;
        for (int idx = threadIdx.x; idx < rows * 3 * D; idx += D * PARTS) {
            const int j = idx / (3 * D), c = idx - j * 3 * D, part3 = c / D, i = c - part3 * D;
            const int chn = part3 == 0 ? kx * D + i : (part3 == 1 ? kd + kx * D + i : 2 * kd + hd * D + i);
            double acc = (double)pp.cw[chn * k + (k - 1)] * (double)pp.xin[(size_t)j * ch + chn];
            for (int t = 0; t < k - 1; t++) {
                const int tau = sz_tree_up(tr, j, (k - 1) - t);  // the row (k - 1) - t steps back: of this pass, or (negative) of the carried state
                const float prev = tau >= 0 ? pp.xin[(size_t)tau * ch + chn] : conv[(size_t)((k - 1) + tau) * ch + chn];
                acc += (double)pp.cw[chn * k + t] * (double)prev;
            }
            pbuf[j][part3][i] = sz_silu((float)acc);
        }
        if (threadIdx.x < rows) {
            const int j = threadIdx.x;
            const float bt = sz_sigmoid(pp.b[j * vh + hd]);
            const float sp_in = pp.a[j * vh + hd] + pp.dt[hd];
            const float sp = sp_in > 20.0f ? sp_in : log1pf(expf(sp_in));
            const float dc = expf(pp.a_log[hd] * sp);
            sbeta[j] = bt; sdecay[j] = dc;
            pp.beta[j * vh + hd] = bt; pp.decay[j * vh + hd] = dc;
        }
        __syncthreads();
        // L2 norm of q and k (q also / sqrt(d)): a warp an item (row, q or k)
        {
            const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            for (int it = warp; it < rows * 2; it += (D * PARTS) / 32) {
                const int j = it >> 1, part3 = it & 1;
                double ss = 0.0;
                for (int i = lane; i < D; i += 32) ss += (double)pbuf[j][part3][i] * (double)pbuf[j][part3][i];
                ss = sz_warp_sum(ss);
                const double nn = sz_rsqrt64(ss + 1e-6);
                for (int i = lane; i < D; i += 32) {
                    float t = (float)((double)pbuf[j][part3][i] * nn);
                    if (part3 == 0) t = t / sqrtf((float)D);
                    pbuf[j][part3][i] = t;
                }
            }
        }
        __syncthreads();
        // what the replay of a commit reads: q and k once a key head (its first value head writes them), v by every head
        for (int idx = threadIdx.x; idx < rows * 3 * D; idx += D * PARTS) {
            const int j = idx / (3 * D), c = idx - j * 3 * D, part3 = c / D, i = c - part3 * D;
            if (part3 == 2) pp.xc[(size_t)j * ch + 2 * kd + hd * D + i] = pbuf[j][2][i];
            else if (hd < kh) pp.xc[(size_t)j * ch + part3 * kd + kx * D + i] = pbuf[j][part3][i];
        }
    }
    float* fk = fork ? fork + ((size_t)di * vh + hd) * SZ_MAX_VERIFY * D * D : nullptr;
    int prev_row = -1;
    for (int jj = 0; jj < rows; jj++) {
        const int j = (!og && tr) ? res[2 + jj] : jj;   // replay of a tree pass: the kept path
        if (tr && og) {
            const int par = tr->parents[j];
            if (par != prev_row && par >= 0) {          // another branch: back to the state after the parent
#pragma unroll
                for (int i = 0; i < NI; i++) S[i] = fk[((size_t)par * D + pt * NI + i) * D + col];
            }
        }
        prev_row = j;
        const float* x = xc + (size_t)j * ch;
        __syncthreads();
        float vj, dc, bt;
        if (fused) {
            if (threadIdx.x < D) { sq[threadIdx.x] = pbuf[j][0][threadIdx.x]; sk[threadIdx.x] = pbuf[j][1][threadIdx.x]; }
            vj = pbuf[j][2][col]; dc = sdecay[j]; bt = sbeta[j];
        } else {
            if (threadIdx.x < D) { sq[threadIdx.x] = x[kx * D + threadIdx.x]; sk[threadIdx.x] = x[kd + kx * D + threadIdx.x]; }
            vj = x[2 * kd + hd * D + col];
            dc = decay[j * vh + hd]; bt = beta[j * vh + hd];
        }
        __syncthreads();
        double mem = 0.0;
#pragma unroll
        for (int i0 = 0; i0 < NI; i0 += RUN) {
            float run = 0.f;
#pragma unroll
            for (int i = i0; i < i0 + RUN; i++) {
                S[i] = S[i] * dc;
                run = fmaf(S[i], sk[pt * NI + i], run);
            }
            mem += (double)run;
        }
        part[pt][col] = mem;
        __syncthreads();
        double tot = 0.0;
#pragma unroll
        for (int p = 0; p < PARTS; p++) tot += part[p][col];
        const float dl = (float)(((double)vj - tot) * (double)bt);
        double o = 0.0;
#pragma unroll
        for (int i0 = 0; i0 < NI; i0 += RUN) {
            float run = 0.f;
#pragma unroll
            for (int i = i0; i < i0 + RUN; i++) {
                S[i] = __fadd_rn(S[i], __fmul_rn(sk[pt * NI + i], dl));  // unfused, as the CPU reference
                run = fmaf(S[i], sq[pt * NI + i], run);
            }
            o += (double)run;
        }
        if (og) {
            __syncthreads();
            part[pt][col] = o;
            __syncthreads();
            if (pt == 0) {
                double ot = 0.0;
#pragma unroll
                for (int p = 0; p < PARTS; p++) ot += part[p][col];
                ofs[j][col] = (float)ot;
            }
            if (tr && ((tr->save >> j) & 1u)) {
#pragma unroll
                for (int i = 0; i < NI; i++) fk[((size_t)j * D + pt * NI + i) * D + col] = S[i];
            }
        }
    }
    if (og) {
        // gated RMS norm of every row's output at once: warp w sums the squares of row w, one thread a row takes the root, then
        // every thread scales its share
        __syncthreads();
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int j = warp; j < rows; j += (D * PARTS) / 32) {
            double ss = 0.0;
            for (int i = lane; i < D; i += 32) ss += (double)ofs[j][i] * (double)ofs[j][i];
            ss = sz_warp_sum(ss);
            if (lane == 0) rrs[j] = sz_rsqrt64(ss / (double)D + (double)eps);
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < rows * D; idx += D * PARTS) {
            const int j = idx / D, c = idx - j * D;
            const float normed = (float)((double)ofs[j][c] * rrs[j]) * norm_w[c];
            og[(size_t)j * vh * D + hd * D + c] = normed * sz_sigmoid(z[(size_t)j * vh * D + hd * D + c]);
        }
    }
    float* So = S_out + (size_t)hd * D * D;
#pragma unroll
    for (int i = 0; i < NI; i++) So[(size_t)(pt * NI + i) * D + col] = S[i];
}

template <int D, int PARTS>
__global__ void __launch_bounds__(D * PARTS)
sz_delta_scan_kernel(const float* __restrict__ xc_all, const float* __restrict__ beta_all, const float* __restrict__ decay_all,
                     const float* __restrict__ z, const float* __restrict__ norm_w, const float* __restrict__ S0, const float* __restrict__ S1,
                     float* __restrict__ O0, float* __restrict__ O1, const int32_t* __restrict__ state, const int32_t* __restrict__ res, int kh,
                     int vh, int m, float eps, float* __restrict__ og, const SzDeltaPrep pp, const SzTree* __restrict__ tr,
                     float* __restrict__ fork) {
    sz_delta_scan_body<D, PARTS>(xc_all, beta_all, decay_all, z, norm_w, S0, S1, O0, O1, state, res, kh, vh, m, eps, og, pp, tr, fork,
                                 (int)blockIdx.x, (int)blockIdx.y);
}

// The pass of one layer for SEVERAL sequences in one launch (a batched step): block row b is sequence b's scan, its pointers and
// row count from a table.  grid (vh, sequences); the arithmetic is the kernel above's.
struct SzScanSeq {
    const float *xc, *beta, *decay, *z, *S0, *S1;
    float *O0, *O1;
    const int32_t *state, *res;
    float* og;
    SzDeltaPrep pp;
    int m, pad;
};
template <int D, int PARTS>
__global__ void __launch_bounds__(D * PARTS, 512 / (D * PARTS))   // (128 registers a thread, as the kernel above happens to need)
sz_delta_scan_seqs_kernel(const SzScanSeq* __restrict__ tab, const float* __restrict__ norm_w, int kh, int vh, float eps) {
    __shared__ SzScanSeq q;   // (the entry in shared memory: two dozen pointers in registers would cost the kernel its second block)
    static_assert(sizeof(SzScanSeq) % 8 == 0, "copied in 8-byte words");
    if (threadIdx.x < sizeof(SzScanSeq) / 8) ((u64*)&q)[threadIdx.x] = ((const u64*)(tab + blockIdx.y))[threadIdx.x];
    __syncthreads();
    sz_delta_scan_body<D, PARTS>(q.xc, q.beta, q.decay, q.z, norm_w, q.S0, q.S1, q.O0, q.O1, q.state, q.res, kh, vh, q.m, eps, q.og, q.pp,
                                 (const SzTree*)nullptr, (float*)nullptr, (int)blockIdx.x, 0);
}

// ---- attention front end (forward.rs:908-927): per head RMSNorm + NeoX RoPE of q and k, the gate halves, K and V into the cache.
// grid (nh + 2 nkv, m), block 128.  Q8 cache: [kv head][pos][hd i8 | hd/32 f16 scales, zero-padded to 16 bytes] - the reference's packed
// Q8_KV head (kernels/forward.cu:3652-3687), stored per head so that a range of positions of one head is contiguous; f32 cache:
// [kv head][pos][hd].
__device__ __forceinline__ int sz_kv_head_bytes(int hd) { return hd + (((hd >> 5) * 2 + 15) & ~15); }

__device__ __forceinline__ void sz_kv_store(const float* src, int hd, int q8, u8* dst_q8, float* dst_f32) {
    if (!q8) {
        for (int i = threadIdx.x; i < hd; i += blockDim.x) dst_f32[i] = src[i];
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, ng = hd >> 5;
    u16* sc = (u16*)(dst_q8 + hd);
    for (int grp = warp; grp < ng; grp += nw) {
        const float v0 = src[grp * 32 + lane];
        float amax = fabsf(v0);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const __half sh = __float2half_rn(amax > 0.0f ? amax * (1.0f / 127.0f) : 0.0f);
        const float sr = __half2float(sh);
        const float inv = sr > 0.0f ? (1.0f / sr) : 0.0f;
        int q0 = __float2int_rn(v0 * inv);
        q0 = q0 < -127 ? -127 : (q0 > 127 ? 127 : q0);
        ((int8_t*)dst_q8)[grp * 32 + lane] = (int8_t)q0;
        if (lane == 0) sc[grp] = __half_as_ushort(sh);
    }
    const int total = (sz_kv_head_bytes(hd) - hd) >> 1;
    for (int u = ng + threadIdx.x; u < total; u += blockDim.x) sc[u] = 0;
}

__global__ void __launch_bounds__(128)
sz_attn_prep_kernel(const float* __restrict__ qg, const float* __restrict__ kk, const float* __restrict__ vv, const float* __restrict__ wq,
                    const float* __restrict__ wk, int nh, int nkv, int hd, int ctx, float eps, const int32_t* __restrict__ state, int rope_dims,
                    const double* __restrict__ rope_den, int q8, u8* __restrict__ kc, u8* __restrict__ vc, float* __restrict__ q, float* __restrict__ gate,
                    const SzTree* __restrict__ tr) {
    __shared__ float tmp[512];
    __shared__ double red[8];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int b = blockIdx.x, j = blockIdx.y;
    const int pos = state[0] + j;                              // the row's cache slot
    const int rpos = state[0] + (tr ? tr->depth[j] : j);      // its position in the sequence (a tree: rows of one depth share it)
    const size_t hbytes = q8 ? (size_t)sz_kv_head_bytes(hd) : (size_t)hd * 4;  // the cache is [kv head][position][head bytes]
    if (b >= nh + nkv) {  // V head: raw into the cache
        const int h = b - nh - nkv;
        u8* dst = vc + ((size_t)h * ctx + pos) * hbytes;
        sz_kv_store(vv + ((size_t)j * nkv + h) * hd, hd, q8, dst, (float*)dst);
        return;
    }
    const bool isq = b < nh;
    const float* x = isq ? qg + ((size_t)j * nh + b) * 2 * hd : kk + ((size_t)j * nkv + (b - nh)) * hd;
    const float* w = isq ? wq : wk;
    double ss = 0.0;
    for (int i = threadIdx.x; i < hd; i += 128) ss += (double)x[i] * (double)x[i];
    ss = sz_block_sum(ss, red);
    const double rr = sz_rsqrt64(ss / (double)hd + (double)eps);
    for (int i = threadIdx.x; i < hd; i += 128) tmp[i] = (float)((double)x[i] * rr) * w[i];
    __syncthreads();
    const int half = rope_dims / 2;
    for (int i = threadIdx.x; i < half; i += 128) {  // forward.rs:290-299
        // angle = pos / theta^(2i / rope_dims) in f64 (the table holds the denominators), reduced to [-pi, pi] in f64; sine and cosine
        // of the reduced angle in f32
        const double f = (double)rpos / __ldg(rope_den + i);
        const double kq = rint(f * 0.15915494309189535);
        double rd = fma(-kq, 6.283185307179586, f);
        rd = fma(-kq, 2.4492935982947064e-16, rd);
        float sn, cs;
        sincosf((float)rd, &sn, &cs);
        const float a0 = tmp[i], b0 = tmp[i + half];
        tmp[i] = a0 * cs - b0 * sn;
        tmp[i + half] = b0 * cs + a0 * sn;
    }
    __syncthreads();
    if (isq) {
        for (int i = threadIdx.x; i < hd; i += 128) {
            q[((size_t)j * nh + b) * hd + i] = tmp[i];
            gate[((size_t)j * nh + b) * hd + i] = x[hd + i];
        }
    } else {
        const int h = b - nh;
        u8* dst = kc + ((size_t)h * ctx + pos) * hbytes;
        sz_kv_store(tmp, hd, q8, dst, (float*)dst);
    }
}

// ---- masked attention over the cache (forward.rs:978-997): row j of the pass attends to positions 0 .. pos0 + j.
// grid (nh, m, splits), block 256: a warp a position at a time, lane owns hd / 32 consecutive dimensions; online softmax per warp,
// merged per block; partial (max, sum, acc[hd]) per split.  part: [m][nh][splits][hd + 2].
template <int EPL>  // elements per lane = hd / 32
__global__ void __launch_bounds__(256)
sz_attn_kernel(const float* __restrict__ q, const u8* __restrict__ kc, const u8* __restrict__ vc, int nh, int nkv, int ctx,
               const int32_t* __restrict__ state, int q8, int splits, float* __restrict__ part, const SzTree* __restrict__ tr) {
    constexpr int HD = EPL * 32;
    __shared__ float sm_m[8], sm_s[8];
    __shared__ float sm_acc[8][HD];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int h = blockIdx.x, j = blockIdx.y, sp = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = h / (nh / nkv);
    const int pos0 = state[0];
    const u32 mk = tr ? tr->mask[j] : (2u << j) - 1u;          // which of the pass's rows this row sees (a chain: rows 0 .. j)
    const int n = pos0 + 32 - __clz(mk);                        // one past the last slot it may see
    const int per = (n + splits - 1) / splits;
    const int t0 = sp * per, t1 = min(n, t0 + per);
    const int hb = sz_kv_head_bytes(HD);
    const size_t rowb = (size_t)(q8 ? hb : HD * 4), headb = (size_t)g * ctx * rowb;
    float qv[EPL];
#pragma unroll
    for (int e = 0; e < EPL; e++) qv[e] = q[((size_t)j * nh + h) * HD + lane * EPL + e];
    const float scale = rsqrtf((float)HD);
    float mx = -INFINITY, sum = 0.f, acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; e++) acc[e] = 0.f;
    for (int t = t0 + warp; t < t1; t += 8) {
        if (t >= pos0 && !((mk >> (t - pos0)) & 1u)) continue;  // a row of another branch
        const u8* kb = kc + (size_t)t * rowb + headb;
        const u8* vb = vc + (size_t)t * rowb + headb;
        float kvv[EPL], vvv[EPL];
        if (q8) {
            const float ks = sz_f16_to_f32(*(const u16*)(kb + HD + 2 * ((lane * EPL) >> 5)));
            const float vs = sz_f16_to_f32(*(const u16*)(vb + HD + 2 * ((lane * EPL) >> 5)));
#pragma unroll
            for (int e = 0; e < EPL; e++) {
                kvv[e] = (float)((const int8_t*)kb)[lane * EPL + e] * ks;
                vvv[e] = (float)((const int8_t*)vb)[lane * EPL + e] * vs;
            }
        } else {
#pragma unroll
            for (int e = 0; e < EPL; e++) { kvv[e] = ((const float*)kb)[lane * EPL + e]; vvv[e] = ((const float*)vb)[lane * EPL + e]; }
        }
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; e++) s = fmaf(qv[e], kvv[e], s);
        s = sz_warp_sum(s) * scale;
        const float nm = fmaxf(mx, s);
        const float c = __expf(mx - nm), p = __expf(s - nm);
        sum = sum * c + p;
#pragma unroll
        for (int e = 0; e < EPL; e++) acc[e] = fmaf(p, vvv[e], acc[e] * c);
        mx = nm;
    }
    if (lane == 0) { sm_m[warp] = mx; sm_s[warp] = sum; }
#pragma unroll
    for (int e = 0; e < EPL; e++) sm_acc[warp][lane * EPL + e] = acc[e];
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < 8; w++) M = fmaxf(M, sm_m[w]);
    float* out = part + (((size_t)j * nh + h) * splits + sp) * (HD + 2);
    if (threadIdx.x < HD) {
        float a = 0.f, ssum = 0.f;
        for (int w = 0; w < 8; w++) {
            const float c = sm_m[w] == -INFINITY ? 0.f : __expf(sm_m[w] - M);
            a += sm_acc[w][threadIdx.x] * c;
            ssum += sm_s[w] * c;
        }
        out[threadIdx.x] = a;
        if (threadIdx.x == 0) { out[HD] = M; out[HD + 1] = ssum; }
    }
}

// ---- masked attention, grouped form --------------------------------------------------------------------------------------------------
// A block takes one KV head and one range of positions and serves every query that shares the head: the G = nh / nkv heads of the
// group times the m rows of the pass (up to 64 query vectors), so each key and value byte leaves HBM once per layer instead of once
// per query.  Both contractions run on mma.sync: scores = Q K^T with the int8 keys turned into f16 exactly and the per-32 scales
// applied to 32-dimension partial sums; out += P V with the value scales folded into P.  Chunks of 64 positions are staged by the
// TMA engine (the cache is laid out per head, so a chunk is one contiguous copy), double-buffered.  Online softmax per query; the
// partial (out, max, sum) of the block goes to the same merge kernel as the simple form.
// Query vector qv = j * G + hh (row j of the pass, head hh of the group); row j attends to positions < pos0 + j + 1.
#define SZ_AT_T 64
template <int HD>
struct SzAttn2 {
    static constexpr int HB = HD + (((HD >> 5) * 2 + 15) & ~15);
    static constexpr int KS = HD / 16;            // k-steps of the score contraction
    static constexpr int DW = HD / 8;             // output dimensions of a warp
    static constexpr int NT = DW / 8;             // its n-tiles
    static constexpr int SST = SZ_AT_T + 2;       // row stride of the score / probability tile (floats)
    static constexpr int STAGE = 2 * SZ_AT_T * HB;  // K chunk then V chunk
    static int smem_bytes(int nqt) { return 64 + 2 * STAGE + nqt * KS * 32 * 16 * 2 + 64 * SST * 4 + 64 * 3 * 4; }
};

template <int HD, int NQT>
__global__ void __launch_bounds__(256)
sz_attn2_kernel(const float* __restrict__ qin, const u8* __restrict__ kc, const u8* __restrict__ vc, int nh, int nkv, int m, int ctx,
                const int32_t* __restrict__ state, int splits, float* __restrict__ part, u32* __restrict__ err, const SzTree* __restrict__ tr,
                const int32_t* __restrict__ glist, const int32_t* __restrict__ gcount, int gstride, int ratio) {
    // glist != null: the sparse form, grid (kv heads, splits, rows).  The block serves ONE row (blockIdx.z) and walks that row's list
    // of position groups (`ratio` positions each; row j's list at glist + j * gstride, gcount[j] long) instead of the positions
    // themselves.  A chunk of 64 list positions is then 64 / ratio copies of a group each for K and for V.
    using A = SzAttn2<HD>;
    extern __shared__ __align__(128) u8 smem[];
    u64* bars = (u64*)smem;
    u8* stage = smem + 64;
    uint4* qhi = (uint4*)(smem + 64 + 2 * A::STAGE);
    uint4* qlo = qhi + NQT * A::KS * 32;
    float* S = (float*)(qlo + NQT * A::KS * 32);          // [64][SST]
    float* rmax = S + 64 * A::SST;                           // running max, sum, and this chunk's rescale factor per query
    float* rsum = rmax + 64;
    float* ralpha = rsum + 64;
    __shared__ int32_t cgrp[2][SZ_AT_T];     // sparse form: the groups of the chunk in each stage
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, q4 = lane & 3;
    const int kvh = blockIdx.x, sp = blockIdx.y;
    const bool sparse = glist != nullptr;
    const int jz = sparse ? (int)blockIdx.z : 0;   // sparse: the one row of this block
    if (sparse) { glist += (size_t)jz * gstride; m = 1; }
    const int G = nh / nkv, QV = G * m;
    // The committed length belongs to the previous pass, and so does every cache position below it: the block's first chunk is
    // requested ahead of the dependency wait when it lies wholly there (the rows of this pass are written by the kernel before).
    int pos0;
    asm volatile("ld.global.s32 %0, [%1];" : "=r"(pos0) : "l"(state));
    // (sparse: the list is written by the kernel before, so its length is read after the dependency wait, below)
    int nmax = pos0 + m;
    if (sparse) { sz_pdl_wait(); nmax = __ldcg(gcount + jz) * ratio; }
    const int per = ((nmax + splits - 1) / splits + SZ_AT_T - 1) / SZ_AT_T * SZ_AT_T;
    const int t0 = sp * per, t1 = min(nmax, t0 + per);
    const int nchunk = t1 > t0 ? (t1 - t0 + SZ_AT_T - 1) / SZ_AT_T : 0;
    const u8* kbase = kc + (size_t)kvh * ctx * A::HB;
    const u8* vbase = vc + (size_t)kvh * ctx * A::HB;
    const bool early = !sparse && nchunk > 0 && t0 + SZ_AT_T <= pos0;
    if (threadIdx.x == 0) {
        sz_mbar_init(&bars[0], 1);
        sz_mbar_init(&bars[1], 1);
        sz_mbar_fence_init();
        if (early) {
            const u32 bytes = (u32)(SZ_AT_T * A::HB);
            sz_mbar_expect_tx(&bars[0], 2 * bytes);
            sz_bulk_g2s(stage, kbase + (size_t)t0 * A::HB, bytes, &bars[0]);
            sz_bulk_g2s(stage + SZ_AT_T * A::HB, vbase + (size_t)t0 * A::HB, bytes, &bars[0]);
        }
    }
    sz_pdl_wait();
    sz_pdl_trigger();
    // the queries as A fragments (f16 high and low parts), scaled by 1 / sqrt(HD)
    const float scale = rsqrtf((float)HD);
    for (int e = threadIdx.x; e < NQT * A::KS * 32; e += 256) {
        const int ln = e & 31, ks = (e >> 5) % A::KS, qt = e / (32 * A::KS);
        const int gg = ln >> 2, qq = ln & 3;
        u32 hi[4], lo[4];
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int qv = qt * 16 + gg + 8 * (r & 1);
            const int dim = ks * 16 + 2 * qq + 8 * (r >> 1);
            float v0 = 0.f, v1 = 0.f;
            if (qv < QV) {
                const int j = jz + qv / G, h = kvh * G + qv % G;
                const float* src = qin + ((size_t)j * nh + h) * HD + dim;
                v0 = src[0] * scale; v1 = src[1] * scale;
            }
            const __half h0 = __float2half_rn(v0), h1 = __float2half_rn(v1);
            const __half l0 = __float2half_rn(v0 - __half2float(h0)), l1 = __float2half_rn(v1 - __half2float(h1));
            hi[r] = (u32)__half_as_ushort(h0) | ((u32)__half_as_ushort(h1) << 16);
            lo[r] = (u32)__half_as_ushort(l0) | ((u32)__half_as_ushort(l1) << 16);
        }
        qhi[e] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        qlo[e] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
    if (threadIdx.x < 64) { rmax[threadIdx.x] = -INFINITY; rsum[threadIdx.x] = 0.f; }
    auto issue = [&](int ci) {  // thread 0: chunk ci of this block into stage ci & 1
        const int t = t0 + ci * SZ_AT_T;
        const u32 bytes = (u32)(min(SZ_AT_T, t1 - t) * A::HB);
        u64* bar = &bars[ci & 1];
        u8* dst = stage + (size_t)(ci & 1) * A::STAGE;
        sz_mbar_expect_tx(bar, 2 * bytes);
        sz_bulk_g2s(dst, kbase + (size_t)t * A::HB, bytes, bar);
        sz_bulk_g2s(dst + SZ_AT_T * A::HB, vbase + (size_t)t * A::HB, bytes, bar);
    };
    auto issue_sparse = [&](int ci) {  // warp 0: lane i copies group i of chunk ci (K and V) and notes the group for the masks
        const int t = t0 + ci * SZ_AT_T;
        const int np = min(SZ_AT_T, t1 - t), ng = np / ratio;        // list positions come in whole groups
        u64* bar = &bars[ci & 1];
        u8* dst = stage + (size_t)(ci & 1) * A::STAGE;
        if (lane == 0) sz_mbar_expect_tx(bar, 2u * (u32)np * A::HB);
        __syncwarp();
        for (int i = lane; i < ng; i += 32) {
            const int gi = __ldcg(glist + t / ratio + i);
            cgrp[ci & 1][i] = gi;
            const u32 bytes = (u32)ratio * A::HB;
            sz_bulk_g2s(dst + (size_t)i * bytes, kbase + (size_t)gi * bytes, bytes, bar);
            sz_bulk_g2s(dst + SZ_AT_T * A::HB + (size_t)i * bytes, vbase + (size_t)gi * bytes, bytes, bar);
        }
    };
    if (sparse) { if (warp == 0 && nchunk > 0) issue_sparse(0); }
    else if (threadIdx.x == 0 && nchunk > 0 && !early) issue(0);
    __syncthreads();
    float o[NQT][A::NT][4];
#pragma unroll
    for (int a = 0; a < NQT; a++)
#pragma unroll
        for (int b = 0; b < A::NT; b++) { o[a][b][0] = 0.f; o[a][b][1] = 0.f; o[a][b][2] = 0.f; o[a][b][3] = 0.f; }
    int failed = 0;
    for (int ci = 0; ci < nchunk; ci++) {
        if (sparse) { if (warp == 0 && ci + 1 < nchunk) issue_sparse(ci + 1); }
        else if (threadIdx.x == 0 && ci + 1 < nchunk) issue(ci + 1);
        if (!sz_mbar_wait(&bars[ci & 1], (ci >> 1) & 1)) failed = 1;
        if (__syncthreads_or(failed)) { failed = 1; break; }
        const u8* kch = stage + (size_t)(ci & 1) * A::STAGE;
        const u8* vch = kch + SZ_AT_T * A::HB;
        const int tbase = t0 + ci * SZ_AT_T;
        // ---- scores of the chunk: warp w takes positions 8 w .. 8 w + 7
        {
            float sacc[NQT][4];
#pragma unroll
            for (int a = 0; a < NQT; a++) { sacc[a][0] = 0.f; sacc[a][1] = 0.f; sacc[a][2] = 0.f; sacc[a][3] = 0.f; }
            const u8* krow = kch + (size_t)(8 * warp + g8) * A::HB;                 // the position this lane feeds as B
            const u16* ksc0 = (const u16*)(kch + (size_t)(8 * warp + 2 * q4) * A::HB + HD);  // scales of the positions of its C columns
            const u16* ksc1 = (const u16*)(kch + (size_t)(8 * warp + 2 * q4 + 1) * A::HB + HD);
#pragma unroll 2
            for (int grp = 0; grp < HD / 32; grp++) {
                float t[NQT][4];
#pragma unroll
                for (int a = 0; a < NQT; a++) { t[a][0] = 0.f; t[a][1] = 0.f; t[a][2] = 0.f; t[a][3] = 0.f; }
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    const int ks = grp * 2 + kk;
                    const u32 b0 = sz_q8_pair(*(const u16*)(krow + ks * 16 + 2 * q4));
                    const u32 b1 = sz_q8_pair(*(const u16*)(krow + ks * 16 + 8 + 2 * q4));
#pragma unroll
                    for (int a = 0; a < NQT; a++) {
                        const uint4 ah = qhi[(a * A::KS + ks) * 32 + lane], al = qlo[(a * A::KS + ks) * 32 + lane];
                        sz_mma16816_z(t[a], (const u32*)&ah, b0, b1);
                        sz_mma16816_z(t[a], (const u32*)&al, b0, b1);
                    }
                }
                const float s0 = sz_f16_to_f32(ksc0[grp]), s1 = sz_f16_to_f32(ksc1[grp]);
#pragma unroll
                for (int a = 0; a < NQT; a++) {
                    sacc[a][0] = fmaf(s0, t[a][0], sacc[a][0]); sacc[a][1] = fmaf(s1, t[a][1], sacc[a][1]);
                    sacc[a][2] = fmaf(s0, t[a][2], sacc[a][2]); sacc[a][3] = fmaf(s1, t[a][3], sacc[a][3]);
                }
            }
#pragma unroll
            for (int a = 0; a < NQT; a++) {
                float* r0 = S + (size_t)(a * 16 + g8) * A::SST + 8 * warp + 2 * q4;
                float* r1 = S + (size_t)(a * 16 + g8 + 8) * A::SST + 8 * warp + 2 * q4;
                r0[0] = sacc[a][0]; r0[1] = sacc[a][1]; r1[0] = sacc[a][2]; r1[1] = sacc[a][3];
            }
        }
        __syncthreads();
        // ---- online softmax: four threads a query, 16 positions each
        {
            const int qv = threadIdx.x >> 2, sub = threadIdx.x & 3;
            if (qv < NQT * 16) {
                // positions of the chunk this query may see: every committed one, and among the pass's own rows those of its mask
                // (a chain: rows 0 .. j; a tree: its ancestors and itself).  vis: bit i = position sub * 16 + i of the chunk.
                u32 vis = 0;
                if (qv < QV && sparse) {
                    // position i of this thread's 16: list position c0 + i, in group cgrp[(c0 - tbase + i) / ratio]; the row sees it
                    // up to its own position (the last group of a list may reach past it)
                    const int c0 = tbase + sub * 16;
                    for (int i = 0; i < 16; i++) {
                        const int cl = sub * 16 + i;
                        if (c0 + i >= t1) break;
                        const int ap = cgrp[ci & 1][cl / ratio] * ratio + cl % ratio;
                        vis |= ap <= pos0 + jz ? 1u << i : 0u;
                    }
                } else if (qv < QV) {
                    const int jr = qv / G;
                    const u32 mk = tr ? tr->mask[jr] : (2u << jr) - 1u;
                    const int c0 = tbase + sub * 16;                  // first position of this thread's 16
                    const int ncom = min(max(min(pos0, t1) - c0, 0), 16);   // committed positions among them
                    vis = ncom >= 16 ? 0xffffu : ((1u << ncom) - 1u);
                    const int sh = c0 - pos0;                         // the pass's row that position c0 is, when >= 0
                    const u32 own = sh >= 0 ? (sh < 32 ? mk >> sh : 0u) : (sh > -32 ? mk << (-sh) : 0u);
                    vis |= own & 0xffffu;
                    const int room = t1 - c0;                          // positions past the block's range are not there
                    vis &= room >= 16 ? 0xffffu : (room > 0 ? (1u << room) - 1u : 0u);
                }
                float* row = S + (size_t)qv * A::SST + sub * 16;
                float mx = -INFINITY;
#pragma unroll
                for (int i = 0; i < 16; i++) if ((vis >> i) & 1u) mx = fmaxf(mx, row[i]);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float mo = rmax[qv];
                const float mn = fmaxf(mo, mx);
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float p = ((vis >> i) & 1u) ? __expf(row[i] - mn) : 0.f;
                    row[i] = p;
                    sum += p;
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (sub == 0) {
                    const float al = mn == -INFINITY ? 1.f : __expf(mo - mn);
                    ralpha[qv] = al;
                    rsum[qv] = rsum[qv] * al + sum;
                    rmax[qv] = mn;
                }
            }
        }
        __syncthreads();
        // ---- out += P V: warp w takes dimensions w DW .. w DW + DW - 1, whose values share one scale group
        {
            const int d0 = warp * A::DW, vgrp = d0 >> 5;
#pragma unroll
            for (int a = 0; a < NQT; a++) {
                const float al0 = ralpha[a * 16 + g8], al1 = ralpha[a * 16 + g8 + 8];
#pragma unroll
                for (int b = 0; b < A::NT; b++) { o[a][b][0] *= al0; o[a][b][1] *= al0; o[a][b][2] *= al1; o[a][b][3] *= al1; }
            }
#pragma unroll
            for (int kk = 0; kk < SZ_AT_T / 16; kk++) {
                const int p0 = kk * 16 + 2 * q4;  // positions p0, p0 + 1, p0 + 8, p0 + 9 are this lane's k slots
                float vs[4];
#pragma unroll
                for (int r = 0; r < 4; r++) vs[r] = sz_f16_to_f32(*(const u16*)(vch + (size_t)(p0 + (r & 1) + 8 * (r >> 1)) * A::HB + HD + 2 * vgrp));
                u32 bf[A::NT][2];
#pragma unroll
                for (int b = 0; b < A::NT; b++) {
                    const int dim = d0 + 8 * b + g8;
                    const u32 v00 = vch[(size_t)p0 * A::HB + dim], v01 = vch[(size_t)(p0 + 1) * A::HB + dim];
                    const u32 v10 = vch[(size_t)(p0 + 8) * A::HB + dim], v11 = vch[(size_t)(p0 + 9) * A::HB + dim];
                    bf[b][0] = sz_q8_pair(v00 | (v01 << 8));
                    bf[b][1] = sz_q8_pair(v10 | (v11 << 8));
                }
#pragma unroll
                for (int a = 0; a < NQT; a++) {
                    u32 af[4];
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        // a0: (query g, k p0..), a1: (query g + 8, k p0..), a2: (query g, k p0 + 8..), a3: (query g + 8, k p0 + 8..)
                        const float* pr = S + (size_t)(a * 16 + g8 + 8 * (r & 1)) * A::SST + p0 + 8 * (r >> 1);
                        const float pa = pr[0], pb = pr[1];
                        const float wa = pa > 0.f ? pa * vs[2 * (r >> 1)] : 0.f, wb = pb > 0.f ? pb * vs[2 * (r >> 1) + 1] : 0.f;
                        af[r] = (u32)__half_as_ushort(__float2half_rn(wa)) | ((u32)__half_as_ushort(__float2half_rn(wb)) << 16);
                    }
#pragma unroll
                    for (int b = 0; b < A::NT; b++) sz_mma16816_z(o[a][b], af, bf[b][0], bf[b][1]);
                }
            }
        }
        __syncthreads();
    }
    if (failed) { if (threadIdx.x == 0) atomicExch(err, 2u); return; }
    // ---- the block's partial result, in the merge kernel's layout: [row][head][split][HD + 2]
#pragma unroll
    for (int a = 0; a < NQT; a++)
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int qv = a * 16 + g8 + 8 * r;
            if (qv < QV) {
                const int j = jz + qv / G, h = kvh * G + qv % G;
                float* out = part + (((size_t)j * nh + h) * splits + sp) * (HD + 2);
#pragma unroll
                for (int b = 0; b < A::NT; b++) {
                    const int dim = warp * A::DW + 8 * b + 2 * q4;
                    out[dim] = o[a][b][2 * r];
                    out[dim + 1] = o[a][b][2 * r + 1];
                }
            }
        }
    if (threadIdx.x < QV) {
        const int qv = threadIdx.x, j = jz + qv / G, h = kvh * G + qv % G;
        float* out = part + (((size_t)j * nh + h) * splits + sp) * (HD + 2);
        out[HD] = rmax[qv];
        out[HD + 1] = rsum[qv];
    }
}

// merge the splits and gate: o = (acc / z) * sigmoid(gate).  grid (nh, m), block 256.  The splits' (max, sum) pairs are read by one
// thread each, the coefficients exp(max_s - max) go through shared memory, and the weighted sum over the splits runs in four
// interleaved groups of threads so that many partial rows are in flight at once.
__global__ void __launch_bounds__(256)
sz_attn_merge_kernel(const float* __restrict__ part, const float* __restrict__ gate, int nh, int hd, int splits, float* __restrict__ o) {
    __shared__ float coef[512];
    __shared__ float red[8];
    __shared__ float accs[4][256];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int h = blockIdx.x, j = blockIdx.y, t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const float* p = part + ((size_t)j * nh + h) * splits * (hd + 2);
    const float g = t < hd ? __ldcg(gate + ((size_t)j * nh + h) * hd + t) : 0.f;
    float mm[2], zz[2];
    float M = -INFINITY;
#pragma unroll
    for (int q = 0; q < 2; q++) {
        const int s = t + 256 * q;
        mm[q] = s < splits ? __ldcg(p + (size_t)s * (hd + 2) + hd) : -INFINITY;
        zz[q] = s < splits ? __ldcg(p + (size_t)s * (hd + 2) + hd + 1) : 0.f;
        M = fmaxf(M, mm[q]);
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, of));
    if (lane == 0) red[warp] = M;
    __syncthreads();
    M = red[0];
    for (int q = 1; q < 8; q++) M = fmaxf(M, red[q]);
    __syncthreads();
    float z = 0.f;
#pragma unroll
    for (int q = 0; q < 2; q++) {
        const int s = t + 256 * q;
        const float c = mm[q] == -INFINITY ? 0.f : __expf(mm[q] - M);
        if (s < splits) coef[s] = c;
        z += zz[q] * c;
    }
    z = sz_warp_sum(z);
    if (lane == 0) red[warp] = z;
    __syncthreads();
    z = 0.f;
    for (int q = 0; q < 8; q++) z += red[q];
    // group gq of threads takes splits gq, gq + 4, ...; a thread four consecutive dimensions
    const int per = hd / 4;              // threads a partial row needs (64 at hd = 256)
    const int ngrp = 256 / per > 4 ? 4 : 256 / per;
    const int gq = t / per, i4 = (t % per) * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gq < ngrp) {
#pragma unroll 4
        for (int s = gq; s < splits; s += ngrp) {
            const float c = coef[s];
            const float2* row = (const float2*)(p + (size_t)s * (hd + 2) + i4);  // rows are 8-byte aligned (hd + 2 is even)
            const float2 v0 = __ldcg(row), v1 = __ldcg(row + 1);
            a.x = fmaf(v0.x, c, a.x); a.y = fmaf(v0.y, c, a.y); a.z = fmaf(v1.x, c, a.z); a.w = fmaf(v1.y, c, a.w);
        }
        accs[gq][i4] = a.x; accs[gq][i4 + 1] = a.y; accs[gq][i4 + 2] = a.z; accs[gq][i4 + 3] = a.w;
    }
    __syncthreads();
    if (t < hd) {
        float v = 0.f;
        for (int q = 0; q < ngrp; q++) v += accs[q][t];
        o[((size_t)j * nh + h) * hd + t] = (v / z) * sz_sigmoid(g);
    }
}

// A drafted token that ends generation is never accepted: the one end-of-generation id of the launch, or one of the session's stop
// ids (the reference's loop leaves `tok.is_eog(d)` and `stops.contains(&d)` drafts for the loop's top: engine.rs:2381-2390).  The
// stop list rides in the pass's staging block: word 24 = how many (at most 7), words 25.. the ids.
__device__ __forceinline__ bool sz_is_stop(const int32_t* __restrict__ ids, int d, int eog) {
    if (d == eog) return true;
    const int n = ids[24];
    for (int i = 0; i < n && i < 7; i++)
        if (ids[25 + i] == d) return true;
    return false;
}

// ---- greedy acceptance on the device (the host loop of crates/shadowzero-serve/src/engine.rs:2377-2408 for the greedy case):
// row i's best token must equal the next drafted token ids[i + 1]; a drafted end-of-generation token is never accepted.
// res[0] = rows kept (1 .. m), res[1] = the token after the kept rows (best of row keep - 1).
__global__ void sz_accept_greedy_kernel(const u32* __restrict__ top, const int32_t* __restrict__ ids, int m, int eog, int keep_all,
                                        int has_head, int32_t* __restrict__ res) {
    sz_pdl_wait();
    sz_pdl_trigger();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int keep = 1;
    if (keep_all) keep = m;
    else
        for (int i = 0; i + 1 < m; i++) {
            const int want = (int)top[(size_t)i * 128 + 64];
            const int d = ids[i + 1];
            if (want != d || sz_is_stop(ids, d, eog)) break;
            keep++;
        }
    res[0] = keep;
    res[1] = has_head ? (int)top[(size_t)(keep - 1) * 128 + 64] : -1;
}

// ---- greedy acceptance over a draft tree (the chain's rule, engine.rs:2377-2408, applied down the tree; no counterpart in the
// reference).  From the root: the target's best token after the current row must be the token of one of its children; that child is
// kept and becomes the current row (lowest row index among equal children); a drafted end-of-generation token is never accepted.
// res[0] = rows kept (the path's length, root included), res[1] = the token after the path, res[2 ..] = the path's row indices.
__global__ void sz_accept_tree_kernel(const u32* __restrict__ top, const int32_t* __restrict__ ids, const SzTree* __restrict__ tr, int m, int eog,
                                      int32_t* __restrict__ res) {
    sz_pdl_wait();
    sz_pdl_trigger();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int cur = 0, keep = 1;
    res[2] = 0;
    for (;;) {
        const int want = (int)top[(size_t)cur * 128 + 64];
        int next = -1;
        for (int c = cur + 1; c < m; c++)
            if (tr->parents[c] == cur && ids[c] == want && !sz_is_stop(ids, want, eog)) { next = c; break; }
        if (next < 0) break;
        cur = next;
        res[2 + keep] = cur;
        keep++;
    }
    res[0] = keep;
    res[1] = (int)top[(size_t)cur * 128 + 64];
}

// The kept rows of a tree pass wrote their keys and values at slot committed + row; the sequence wants them at committed + depth.
// Path entry d (depth d) moves from slot committed + path[d] to committed + d; path[d] >= d and the path ascends, so moving in
// order of d never overwrites a slot that is still to be read.  grid (kv heads, attention layers, 2: keys / values), block 128.
__global__ void __launch_bounds__(128)
sz_kv_compact_kernel(u8* __restrict__ kc, u8* __restrict__ vc, const int32_t* __restrict__ state, const int32_t* __restrict__ res, int ctx, int nkv,
                     int head_bytes) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int keep = res[0];
    u8* base = (blockIdx.z ? vc : kc) + ((size_t)blockIdx.y * nkv + blockIdx.x) * (size_t)ctx * head_bytes;
    const int pos0 = state[0];
    for (int d = 1; d < keep; d++) {
        const int from = res[2 + d];
        if (from != d) {
            const u32* src = (const u32*)(base + (size_t)(pos0 + from) * head_bytes);
            u32* dst = (u32*)(base + (size_t)(pos0 + d) * head_bytes);
            for (int i = threadIdx.x; i < head_bytes / 4; i += 128) dst[i] = src[i];
        }
        __syncthreads();
    }
}

// ---- sampled acceptance on the device: Sampler::sample_top (crates/shadowzero-serve/src/sampler.rs:159-210) for every row of the
// pass, then the host loop's rule (engine.rs:2377-2408).  A warp a row: the exponentials in parallel, everything whose order of
// operations decides a rounding (the f64 sums, the walk along the cumulative distribution) sequentially in lane 0, as the host does.
struct SzSampleArgs { float temperature; int top_k; float top_p; float min_p; unsigned long long seed; unsigned long long pos; };
__device__ __forceinline__ unsigned long long sz_splitmix64_dev(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__global__ void __launch_bounds__(32 * SZ_MAX_VERIFY)
sz_accept_sampled_kernel(const u32* __restrict__ top, const int32_t* __restrict__ ids, int m, int eog, const SzSampleArgs* __restrict__ sa,
                         int32_t* __restrict__ res) {
    __shared__ double probs[SZ_MAX_VERIFY][64];
    __shared__ u32 picks[SZ_MAX_VERIFY];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int j = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (j < m) {
        const SzSampleArgs a = *sa;
        const u32* row = top + (size_t)j * 128;
        const float v0 = __uint_as_float(row[lane]), v1 = __uint_as_float(row[lane + 32]);
        const float mx = __shfl_sync(0xffffffffu, v0, 0);
        u32 pick = row[64];
        if (isfinite(mx)) {   // (uniform over the warp)
            const float cut = __fsub_rn(mx, __fmul_rn(18.0f, a.temperature));
            // the values are sorted: the candidates are a prefix
            const u32 b0 = __ballot_sync(0xffffffffu, v0 >= cut), b1 = __ballot_sync(0xffffffffu, v1 >= cut);
            int n = b0 == 0xffffffffu ? 32 + (b1 == 0xffffffffu ? 32 : __ffs(~b1) - 1) : __ffs(~b0) - 1;
            const int tk = a.top_k < 1 ? 1 : a.top_k;
            if (n > tk) n = tk;
            const float inv_t = __fdiv_rn(1.0f, a.temperature);
            if (lane < n) probs[j][lane] = exp((double)__fmul_rn(__fsub_rn(v0, mx), inv_t));
            if (lane + 32 < n) probs[j][lane + 32] = exp((double)__fmul_rn(__fsub_rn(v1, mx), inv_t));
            __syncwarp();
            if (lane == 0) {
                double total = 0.0;
                for (int i = 0; i < n; i++) total += probs[j][i];
                for (int i = 0; i < n; i++) probs[j][i] = probs[j][i] / total;
                const double floor_p = (double)a.min_p * probs[j][0];
                int keep = 0;
                while (keep < n && probs[j][keep] >= floor_p) keep++;
                if (keep < 1) keep = 1;
                if (a.top_p < 1.0f) {
                    double acc = 0.0;
                    int cnt = 0;
                    for (int i = 0; i < keep; i++) { acc += probs[j][i]; cnt++; if (acc >= (double)a.top_p) break; }
                    keep = cnt < 1 ? 1 : cnt;
                }
                double mass = 0.0;
                for (int i = 0; i < keep; i++) mass += probs[j][i];
                const unsigned long long bits = sz_splitmix64_dev(sz_splitmix64_dev(a.seed) ^ ((a.pos + (unsigned long long)j) * 0xD6E8FEB86659FD93ull));
                double u = ((double)(bits >> 11) / 9007199254740992.0) * mass;
                int at = keep - 1;
                for (int i = 0; i < keep; i++) {
                    if (u < probs[j][i]) { at = i; break; }
                    u -= probs[j][i];
                }
                pick = row[64 + at];
            }
        }
        if (lane == 0) picks[j] = pick;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int keep = 1;
        for (int i = 0; i + 1 < m; i++) {
            const int d = ids[i + 1];
            if ((int)picks[i] != d || sz_is_stop(ids, d, eog)) break;
            keep++;
        }
        res[0] = keep;
        res[1] = (int)picks[keep - 1];
    }
}

#endif  // __CUDACC__
