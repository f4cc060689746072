// Dense projections of a verify pass: y[j] = W x[j] for the 1..8 rows of the pass, W in any of the stored types.
// The role of the reference's matvec_cols_* family (kernels/matvec.cu:677-756) and multi_cols (crates/shadowzero-cuda/src/session.rs:
// 7346-7398: several projections of one input in a launch).  A warp takes a matrix row, a lane four consecutive weights of every
// 128, the inputs sit in shared memory; f32 accumulate.
#pragma once

#include "sz_formats.cuh"

#define SZ_DENSE_MAX_JOBS 6
#define SZ_EPI_NONE 0
#define SZ_EPI_SILU_DIV 1      // silu(v / div)            (hyper-connection down, forward.rs:803)
#define SZ_EPI_SIGMOID 2       // sigmoid(v)
#define SZ_EPI_SIGMOID2_DIV 3  // 2 * sigmoid(v / div)     (hyper-connection inject, forward.rs:812)

struct SzDenseJob {
    const u8* w;     // matrix, rows contiguous
    float* out;      // out[j * ostride + r]
    int rows;
    int type;
    int ostride;
    int epi;
    float div;
    int row0;        // first global row index of this job (filled by the launcher)
};

struct SzDenseArgs {
    SzDenseJob job[SZ_DENSE_MAX_JOBS];
    int n_jobs;
    int total_rows;
    const float* x;  // [m][xstride]
    int xstride;
    int cols;
    int m;
    u32* err;        // set to 1 when a bounded wait on a copy ran out (null: not reported)
};

#ifdef __CUDACC__

__device__ __forceinline__ size_t sz_dense_row_bytes(int type, int cols) {
    switch (type) {
        case SZ_TYPE_F32: return (size_t)cols * 4;
        case SZ_TYPE_F16: case SZ_TYPE_BF16: return (size_t)cols * 2;
        case SZ_TYPE_Q8_0: return (size_t)(cols / 32) * 34;
        default: return (size_t)(cols / 256) * 110;
    }
}

template <typename T, bool GLOBAL>
__device__ __forceinline__ T sz_ld(const void* p) {
    if (GLOBAL) return __ldg((const T*)p);
    return *(const T*)p;
}

// the lane's four weights at columns e .. e + 3 of `row`, and the scale they share.  GLOBAL: `row` is in global memory (read-only
// path); otherwise any address space (a staged copy in shared memory)
template <bool GLOBAL = true>
__device__ __forceinline__ void sz_dense_w4(int type, const u8* __restrict__ row, int e, const u32* grid, float* w, float& scale) {
    if (type == SZ_TYPE_F32) {
        const float4 v = sz_ld<float4, GLOBAL>(row + (size_t)e * 4);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; scale = 1.f;
    } else if (type == SZ_TYPE_BF16) {
        const uint2 v = sz_ld<uint2, GLOBAL>(row + (size_t)e * 2);
        w[0] = __uint_as_float(v.x << 16); w[1] = __uint_as_float(v.x & 0xffff0000u);
        w[2] = __uint_as_float(v.y << 16); w[3] = __uint_as_float(v.y & 0xffff0000u); scale = 1.f;
    } else if (type == SZ_TYPE_F16) {
        const uint2 v = sz_ld<uint2, GLOBAL>(row + (size_t)e * 2);
        w[0] = sz_f16_to_f32((u16)(v.x & 0xffff)); w[1] = sz_f16_to_f32((u16)(v.x >> 16));
        w[2] = sz_f16_to_f32((u16)(v.y & 0xffff)); w[3] = sz_f16_to_f32((u16)(v.y >> 16)); scale = 1.f;
    } else if (type == SZ_TYPE_Q8_0) {
        const u8* blk = row + (e >> 5) * 34;
        const int i = e & 31;
        scale = sz_f16_to_f32(sz_ld<u16, GLOBAL>(blk));
        const u32 q01 = sz_ld<u16, GLOBAL>(blk + 2 + i), q23 = sz_ld<u16, GLOBAL>(blk + 4 + i);
        w[0] = (float)(int8_t)(q01 & 0xff); w[1] = (float)(int8_t)(q01 >> 8);
        w[2] = (float)(int8_t)(q23 & 0xff); w[3] = (float)(int8_t)(q23 >> 8);
    } else {  // IQ3_S
        const u8* blk = row + (e >> 8) * 110;
        const int jj = (e & 255) >> 2;
        const int idx = blk[2 + jj] | (((blk[66 + (jj >> 3)] >> (jj & 7)) & 1) << 8);
        const int g = jj >> 3;
        const int s = (blk[106 + (g >> 1)] >> (4 * (g & 1))) & 15;
        scale = sz_f16_to_f32(sz_ld16(blk)) * (float)(1 + 2 * s);
        const u32 mags = grid[idx];
        const u32 sg = blk[74 + (jj >> 1)] >> (4 * (jj & 1));
        w[0] = (float)(mags & 0xff); w[1] = (float)((mags >> 8) & 0xff); w[2] = (float)((mags >> 16) & 0xff); w[3] = (float)(mags >> 24);
        w[0] = (sg & 1) ? -w[0] : w[0]; w[1] = (sg & 2) ? -w[1] : w[1]; w[2] = (sg & 4) ? -w[2] : w[2]; w[3] = (sg & 8) ? -w[3] : w[3];
    }
}

__device__ __forceinline__ float sz_epilogue(int epi, float v, float div) {
    switch (epi) {
        case SZ_EPI_SILU_DIV: return sz_silu(v / div);
        case SZ_EPI_SIGMOID: return sz_sigmoid(v);
        case SZ_EPI_SIGMOID2_DIV: return 2.0f * sz_sigmoid(v / div);
        default: return v;
    }
}

// grid: any (blocks stride over the rows of all jobs, 8 rows a block at a time); block 256; dynamic shared memory 2048 + mt * cols * 4
// where mt = rows of x handled per sweep (the launcher picks the largest that fits).
template <int MT>
__global__ void __launch_bounds__(256) sz_dense_kernel(const SzDenseArgs a) {
    extern __shared__ __align__(128) u8 smem[];
    u32* grid = (u32*)smem;
    float* xs = (float*)(smem + 2048);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    sz_pdl_wait();
    sz_pdl_trigger();
    for (int i = threadIdx.x; i < 512; i += 256) grid[i] = c_iq3s_grid[i];
    for (int j0 = 0; j0 < a.m; j0 += MT) {
        const int mt = min(MT, a.m - j0);
        __syncthreads();
        for (int j = 0; j < mt; j++) {
            const float4* src = (const float4*)(a.x + (size_t)(j0 + j) * a.xstride);
            float4* dst = (float4*)(xs + (size_t)j * a.cols);
            for (int i = threadIdx.x; i < a.cols / 4; i += 256) dst[i] = __ldcg(src + i);
        }
        __syncthreads();
        for (int r = blockIdx.x * 8 + warp; r < a.total_rows; r += gridDim.x * 8) {
            int ji = 0;
#pragma unroll
            for (int q = 1; q < SZ_DENSE_MAX_JOBS; q++)
                if (q < a.n_jobs && r >= a.job[q].row0) ji = q;
            const SzDenseJob& jb = a.job[ji];
            const int rr = r - jb.row0;
            const u8* row = jb.w + (size_t)rr * sz_dense_row_bytes(jb.type, a.cols);
            float acc[MT];
#pragma unroll
            for (int j = 0; j < MT; j++) acc[j] = 0.f;
            for (int e = 4 * lane; e < a.cols; e += 128) {
                float w[4], scale;
                sz_dense_w4<true>(jb.type, row, e, grid, w, scale);
#pragma unroll
                for (int j = 0; j < MT; j++) {
                    if (j < mt) {
                        const float4 v = *(const float4*)(xs + (size_t)j * a.cols + e);
                        float p = w[0] * v.x;
                        p = fmaf(w[1], v.y, p);
                        p = fmaf(w[2], v.z, p);
                        p = fmaf(w[3], v.w, p);
                        acc[j] = fmaf(scale, p, acc[j]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < MT; j++) {
                if (j < mt) {
                    const float v = sz_warp_sum(acc[j]);
                    if (lane == 0) jb.out[(size_t)(j0 + j) * jb.ostride + rr] = sz_epilogue(jb.epi, v, jb.div);
                }
            }
        }
    }
}

// ---- streaming form -------------------------------------------------------------------------------------------------------------------
// Units of R whole rows (about 32 KB) are copied into a ring of shared-memory stages by the TMA engine (cp.async.bulk) while the
// warps work on the previous ones.  Warp w takes RW rows of the unit (row group w % NG) and one of KP column ranges (w / NG), so an
// x value read from shared memory feeds RW rows: the kernel is bound by the weight stream, not by shared-memory reads of x.
// Column-range partial sums meet in shared memory.  Needs row bytes that are a multiple of 16.
struct SzDense2Cfg {
    int R, RW, KP, NS;       // rows a unit, rows a warp, column parts, stages
    int unit_bytes;          // R * row bytes (the same for every job: one input width, and the jobs of a launch share a type size class)
    int units[SZ_DENSE_MAX_JOBS + 1];  // first unit of each job; units[n_jobs] = total
};

template <int MT, int RW>
__global__ void __launch_bounds__(256) sz_dense2_kernel(const SzDenseArgs a, const SzDense2Cfg c) {
    extern __shared__ __align__(128) u8 smem[];
    u64* bars = (u64*)smem;                               // NS barriers (64 bytes reserved)
    u32* grid = (u32*)(smem + 64);                        // IQ3_S codebook
    float* red = (float*)(smem + 64 + 2048);              // [8 warps][RW][MT]
    float* xs = (float*)(smem + 64 + 2048 + 8 * 4 * 8 * 4);
    u8* stages = smem + 64 + 2048 + 1024 + (size_t)MT * a.cols * 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NG = c.R / RW;
    const int grp = warp % NG, kp = warp / NG;
    const int part = a.cols / c.KP;
    const int e0 = kp * part, e1 = e0 + part;
    if (threadIdx.x == 0) {
        for (int i = 0; i < c.NS; i++) sz_mbar_init(&bars[i], 1);
        sz_mbar_fence_init();
    }
    for (int i = threadIdx.x; i < 512; i += 256) grid[i] = c_iq3s_grid[i];
    __syncthreads();
    const int total = c.units[a.n_jobs];
    auto locate = [&](int u, int& ji, int& row0, int& nrows) {
        ji = 0;
#pragma unroll
        for (int q = 1; q < SZ_DENSE_MAX_JOBS; q++)
            if (q < a.n_jobs && u >= c.units[q]) ji = q;
        row0 = (u - c.units[ji]) * c.R;
        nrows = min(c.R, a.job[ji].rows - row0);
    };
    // weights do not depend on the previous kernel: start streaming before waiting for it
    const int first = blockIdx.x, step = gridDim.x;
    const int count = first < total ? (total - first + step - 1) / step : 0;
    auto issue = [&](int local, int gi) {  // local: which of this block's units; gi: running copy index over all sweeps
        int ji, row0, nrows;
        locate(first + local * step, ji, row0, nrows);
        const size_t rb = sz_dense_row_bytes(a.job[ji].type, a.cols);
        u64* bar = &bars[gi % c.NS];
        const u32 bytes = (u32)(nrows * rb);
        sz_mbar_expect_tx(bar, bytes);
        sz_bulk_g2s(stages + (size_t)(gi % c.NS) * c.unit_bytes, a.job[ji].w + (size_t)row0 * rb, bytes, bar);
    };
    int failed = 0;
    for (int j0 = 0; j0 < a.m; j0 += MT) {
        const int mt = min(MT, a.m - j0);
        const int base = (j0 / MT) * count;  // units issued so far (each sweep streams every unit again)
        if (threadIdx.x == 0)
            for (int i = 0; i < c.NS - 1 && i < count; i++) issue(i, base + i);
        if (j0 == 0) { sz_pdl_wait(); sz_pdl_trigger(); }
        __syncthreads();
        for (int j = 0; j < mt; j++) {
            const float4* src = (const float4*)(a.x + (size_t)(j0 + j) * a.xstride);
            float4* dst = (float4*)(xs + (size_t)j * a.cols);
            for (int i = threadIdx.x; i < a.cols / 4; i += 256) dst[i] = __ldcg(src + i);
        }
        __syncthreads();
        for (int i = 0; i < count; i++) {
            const int gi = base + i;
            if (threadIdx.x == 0 && i + c.NS - 1 < count) issue(i + c.NS - 1, gi + c.NS - 1);
            int ji, row0, nrows;
            locate(first + i * step, ji, row0, nrows);
            const SzDenseJob& jb = a.job[ji];
            const size_t rb = sz_dense_row_bytes(jb.type, a.cols);
            if (!sz_mbar_wait(&bars[gi % c.NS], (gi / c.NS) & 1)) failed = 1;
            const u8* st = stages + (size_t)(gi % c.NS) * c.unit_bytes;
            float acc[RW][MT];
#pragma unroll
            for (int r = 0; r < RW; r++)
#pragma unroll
                for (int j = 0; j < MT; j++) acc[r][j] = 0.f;
            if (!failed && kp < c.KP && grp * RW < nrows) {
                for (int e = e0 + 4 * lane; e < e1; e += 128) {
                    float4 xv[MT];
#pragma unroll
                    for (int j = 0; j < MT; j++) xv[j] = j < mt ? *(const float4*)(xs + (size_t)j * a.cols + e) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int r = 0; r < RW; r++) {
                        const int rr = grp * RW + r;
                        if (rr < nrows) {
                            float w[4], scale;
                            sz_dense_w4<false>(jb.type, st + (size_t)rr * rb, e, grid, w, scale);
#pragma unroll
                            for (int j = 0; j < MT; j++) {
                                float p = w[0] * xv[j].x;
                                p = fmaf(w[1], xv[j].y, p);
                                p = fmaf(w[2], xv[j].z, p);
                                p = fmaf(w[3], xv[j].w, p);
                                acc[r][j] = fmaf(scale, p, acc[r][j]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < RW; r++)
#pragma unroll
                for (int j = 0; j < MT; j++) {
                    const float v = sz_warp_sum(acc[r][j]);
                    if (lane == 0) red[(warp * RW + r) * MT + j] = v;
                }
            if (__syncthreads_or(failed)) { failed = 1; break; }
            // the column parts of a row meet here: thread t finishes (row rr, input row j)
            for (int t = threadIdx.x; t < nrows * mt; t += 256) {
                const int rr = t / mt, j = t % mt;
                const int g2 = rr / RW, r2 = rr % RW;
                float v = 0.f;
                for (int q = 0; q < c.KP; q++) v += red[((q * NG + g2) * RW + r2) * MT + j];
                jb.out[(size_t)(j0 + j) * jb.ostride + row0 + rr] = sz_epilogue(jb.epi, v, jb.div);
            }
            __syncthreads();
        }
        if (failed) break;
    }
    if (failed && threadIdx.x == 0 && a.err) atomicExch(a.err, 1u);
}

// ---- Q8_0 on the tensor pipe ----------------------------------------------------------------------------------------------------------
// The same streaming skeleton for Q8_0 matrices, with the multiply-adds on mma.sync: a warp owns one eighth of the columns of a
// 16-row unit; per 32-column block it turns each row's 32 int8 codes into f16 exactly (0x6400 | (q ^ 0x80) is the f16 1024 + q + 128),
// multiplies them with the rows of the pass (the B operand, split into f16 high and low parts so the activations keep f32 accuracy)
// into a fresh accumulator and adds that, times the block's scale, to the running sums.  Per weight this is ~2.6 issue slots
// whatever the number of rows, against ~8 for the scalar form at 4 rows, which is what lets the kernel follow the HBM stream.
// Lane (g, q) takes the block's bytes 8 q .. 8 q + 7 of rows g and g + 8; the k slots of the two MMAs are permuted accordingly and
// the B fragments use the same permutation (x columns 8 q .. 8 q + 7 of row-of-the-pass g).
__device__ __forceinline__ void sz_mma16816_z(float* c, const u32* a, u32 b0, u32 b1) {  // c += a * b
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// two int8 codes (the low 16 bits of p) as an f16 pair
__device__ __forceinline__ u32 sz_q8_pair(u32 p) {
    const u32 t = __byte_perm(p ^ 0x8080u, 0x64646464u, 0x4140);  // 0x64 b1' 0x64 b0' with b' = b ^ 0x80
    const __half2 h = __hsub2(*(const __half2*)&t, __halves2half2(__ushort_as_half((u16)0x6480), __ushort_as_half((u16)0x6480)));  // - 1152
    return *(const u32*)&h;
}

struct SzDenseQ8Cfg {
    int NS, unit_bytes;
    int rbp;   // bytes between the rows of a staged unit: the row bytes padded so that rows 0..7 start in different banks
    int xsp;   // halves between the staged rows of the pass, padded likewise
    int units[SZ_DENSE_MAX_JOBS + 1];
};

// Shared-memory layout matters more than anything else here: a matrix row is cols / 32 * 34 bytes, a multiple of 128 for the usual
// widths, so eight lanes reading the same block of eight different rows would hit one bank eight times over.  Every row of a unit
// is therefore its own bulk copy to a padded stride (rbp), and the rows of the pass are padded the same way (xsp).
// grid: any; block 256; dynamic shared memory: 64 (barriers) + 4096 (reduction) + 2 * m * xsp * 2 (x as f16 hi | lo) + NS * unit_bytes
static __global__ void __launch_bounds__(256, 2) sz_dense_q8_kernel(const SzDenseArgs a, const SzDenseQ8Cfg c) {
    extern __shared__ __align__(128) u8 smem[];
    u64* bars = (u64*)smem;
    float* red = (float*)(smem + 64);                       // [8 warps][16 rows][8 rows of the pass]
    __half* xhi = (__half*)(smem + 64 + 4096);              // [m][xsp]
    __half* xlo = xhi + (size_t)a.m * c.xsp;
    u8* stages = smem + 64 + 4096 + (size_t)a.m * c.xsp * 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const size_t rb = (size_t)(a.cols / 32) * 34;
    if (threadIdx.x == 0) {
        for (int i = 0; i < c.NS; i++) sz_mbar_init(&bars[i], 1);
        sz_mbar_fence_init();
    }
    __syncthreads();
    const int total = c.units[a.n_jobs];
    auto locate = [&](int u, int& ji, int& row0, int& nrows) {
        ji = 0;
#pragma unroll
        for (int t = 1; t < SZ_DENSE_MAX_JOBS; t++)
            if (t < a.n_jobs && u >= c.units[t]) ji = t;
        row0 = (u - c.units[ji]) * 16;
        nrows = min(16, a.job[ji].rows - row0);
    };
    const int first = blockIdx.x, step = gridDim.x;
    const int count = first < total ? (total - first + step - 1) / step : 0;
    auto issue = [&](int i) {
        int ji, row0, nrows;
        locate(first + i * step, ji, row0, nrows);
        u64* bar = &bars[i % c.NS];
        sz_mbar_expect_tx(bar, (u32)(nrows * rb));
        u8* dst = stages + (size_t)(i % c.NS) * c.unit_bytes;
        const u8* src = a.job[ji].w + (size_t)row0 * rb;
        for (int r = 0; r < nrows; r++) sz_bulk_g2s(dst + (size_t)r * c.rbp, src + (size_t)r * rb, (u32)rb, bar);
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < c.NS - 1 && i < count; i++) issue(i);
    sz_pdl_wait();
    sz_pdl_trigger();
    for (int j = 0; j < a.m; j++)
      for (int c4 = threadIdx.x; c4 < a.cols / 4; c4 += 256) {
        const float4 v = __ldcg((const float4*)(a.x + (size_t)j * a.xstride) + c4);
        const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        const __half2 l0 = __floats2half2_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2half2_rn(v.z - f1.x, v.w - f1.y);
        *(uint2*)(xhi + (size_t)j * c.xsp + 4 * c4) = make_uint2(*(const u32*)&h0, *(const u32*)&h1);
        *(uint2*)(xlo + (size_t)j * c.xsp + 4 * c4) = make_uint2(*(const u32*)&l0, *(const u32*)&l1);
    }
    __syncthreads();
    const int part = a.cols / 8;          // columns of this warp: [warp * part, (warp + 1) * part), whole 32-column blocks
    const int nblk = part / 32;
    int failed = 0;
    for (int i = 0; i < count; i++) {
        if (threadIdx.x == 0 && i + c.NS - 1 < count) issue(i + c.NS - 1);
        int ji, row0, nrows;
        locate(first + i * step, ji, row0, nrows);
        const SzDenseJob& jb = a.job[ji];
        if (!sz_mbar_wait(&bars[i % c.NS], (i / c.NS) & 1)) failed = 1;
        const u8* st = stages + (size_t)(i % c.NS) * c.unit_bytes;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};  // rows g, g + 8 x rows of the pass 2 q, 2 q + 1
        if (!failed) {
            const u8* r0 = st + (size_t)(g < nrows ? g : 0) * c.rbp;
            const u8* r1 = st + (size_t)(g + 8 < nrows ? g + 8 : 0) * c.rbp;
            for (int b = 0; b < nblk; b++) {
                const int blk = warp * nblk + b;
                const int col = blk * 32 + 8 * q;
                uint4 bh = make_uint4(0, 0, 0, 0), bl = make_uint4(0, 0, 0, 0);
                if (g < a.m) {
                    bh = *(const uint4*)(xhi + (size_t)g * c.xsp + col);
                    bl = *(const uint4*)(xlo + (size_t)g * c.xsp + col);
                }
                const u8* p0 = r0 + (size_t)blk * 34;
                const u8* p1 = r1 + (size_t)blk * 34;
                const float d0 = sz_f16_to_f32(*(const u16*)p0), d1 = sz_f16_to_f32(*(const u16*)p1);
                const u16* c0 = (const u16*)(p0 + 2 + 8 * q);
                const u16* c1 = (const u16*)(p1 + 2 + 8 * q);
                u32 a1[4], a2[4];
                a1[0] = sz_q8_pair(c0[0]); a1[2] = sz_q8_pair(c0[1]); a2[0] = sz_q8_pair(c0[2]); a2[2] = sz_q8_pair(c0[3]);
                a1[1] = sz_q8_pair(c1[0]); a1[3] = sz_q8_pair(c1[1]); a2[1] = sz_q8_pair(c1[2]); a2[3] = sz_q8_pair(c1[3]);
                float t[4] = {0.f, 0.f, 0.f, 0.f};
                sz_mma16816_z(t, a1, bh.x, bh.y);
                sz_mma16816_z(t, a2, bh.z, bh.w);
                sz_mma16816_z(t, a1, bl.x, bl.y);
                sz_mma16816_z(t, a2, bl.z, bl.w);
                acc[0] = fmaf(d0, t[0], acc[0]); acc[1] = fmaf(d0, t[1], acc[1]);
                acc[2] = fmaf(d1, t[2], acc[2]); acc[3] = fmaf(d1, t[3], acc[3]);
            }
        }
        // the eight column parts of a row meet in shared memory
        red[(warp * 16 + g) * 8 + 2 * q] = acc[0];
        red[(warp * 16 + g) * 8 + 2 * q + 1] = acc[1];
        red[(warp * 16 + g + 8) * 8 + 2 * q] = acc[2];
        red[(warp * 16 + g + 8) * 8 + 2 * q + 1] = acc[3];
        if (__syncthreads_or(failed)) { failed = 1; break; }
        for (int t = threadIdx.x; t < 16 * 8; t += 256) {
            const int rr = t >> 3, j = t & 7;
            if (rr < nrows && j < a.m) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < 8; w++) v += red[(w * 16 + rr) * 8 + j];
                jb.out[(size_t)j * jb.ostride + row0 + rr] = sz_epilogue(jb.epi, v, jb.div);
            }
        }
        __syncthreads();
    }
    if (failed && threadIdx.x == 0 && a.err) atomicExch(a.err, 1u);
}

// ---- Q8_0 projections over MANY rows (the rows of a batch of sequences), the arithmetic of sz_dense_q8_kernel --------------------------
// What the kernel above computes for the (up to) 8 rows of a pass, for any multiple of 8 rows, with the matrices read once for all
// of them instead of once per 8 rows.  A row's result is bit for bit the kernel above's: there a warp owns one eighth of the columns
// (a "part") and runs, per 32-column block of its part in order, four MMAs into a fresh accumulator and one fused multiply-add with
// the block's scale into the part's running sum; the eight parts' sums are then added in order.  Here the same chains run in
// another place: a thread block owns ONE part, a range of row groups (8 rows each, as many as fit shared memory) and a range of
// 16-row units of the matrices; it stages its part of the rows once (f16 high + low, as above) and streams the units' slices of
// that part through a ring of shared-memory stages (cp.async, 8 units a stage, one a warp); a warp decodes a block's A fragments
// once and uses them for every row group (the chains of the groups are independent accumulators).  The parts' sums go to
// `partial` [8][rows][outputs] and sz_dense_rows_reduce_kernel adds them in order and applies the epilogue.
// A slice of a matrix row starts at a multiple of 34 bytes, not of 16: the copy starts at the 16-byte boundary below it and the
// reads skip the difference (the same for every row of a block, matrix rows being whole 16-byte chunks).
struct SzDenseRowsCfg {
    int units[SZ_DENSE_MAX_JOBS + 1];   // 16-row units before each job
    int upc;          // units a block takes (a multiple of 8)
    int G, nz, gb;    // row groups in all, blocks along the rows, row groups a block at most
    int sb;           // bytes of a matrix row's slice of one part
    int rs;           // bytes between the staged slices
    int xs;           // halves between the staged rows
    int rows;         // rows in all (8 G)
    float* partial;
};

__device__ __forceinline__ void sz_cp_async16(void* smem_dst, const void* src) {
    const u32 d = (u32)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void sz_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void sz_cp_async_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// grid (8 parts, unit chunks, row blocks); block 256; dynamic shared memory gb * 8 * xs * 4 + 2 * 128 * rs
template <int GB>
static __global__ void __launch_bounds__(256) sz_dense_rows_q8_kernel(const SzDenseArgs a, const SzDenseRowsCfg c) {
    extern __shared__ __align__(128) u8 smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int p = blockIdx.x;
    const int part = a.cols / 8, nblk = part / 32;
    const int g0 = (int)((long long)c.G * blockIdx.z / c.nz), g1 = (int)((long long)c.G * (blockIdx.z + 1) / c.nz);
    const int ng = g1 - g0;                       // <= GB
    const int total = c.units[a.n_jobs];
    const int u0 = blockIdx.y * c.upc, u1 = min(total, u0 + c.upc);
    if (ng <= 0 || u0 >= u1) return;
    __half* xhi = (__half*)smem;                  // [GB * 8][xs]
    __half* xlo = xhi + (size_t)GB * 8 * c.xs;
    u8* stages = smem + (size_t)GB * 8 * c.xs * 4;
    const size_t stage_bytes = (size_t)128 * c.rs;
    const size_t rb = (size_t)(a.cols / 32) * 34;
    const int s_off = (p * c.sb) & 15;
    const int chunks = (s_off + c.sb + 15) >> 4;
    const int nstage = (u1 - u0 + 7) >> 3;
    auto locate = [&](int u, int& ji, int& row0, int& nrows) {
        ji = 0;
#pragma unroll
        for (int t = 1; t < SZ_DENSE_MAX_JOBS; t++)
            if (t < a.n_jobs && u >= c.units[t]) ji = t;
        row0 = (u - c.units[ji]) * 16;
        nrows = min(16, a.job[ji].rows - row0);
    };
    // two threads a staged row: thread t copies the chunks t & 1, (t & 1) + 2, ... of row t >> 1 of the stage
    auto issue = [&](int si) {
        const int r = threadIdx.x >> 1;
        const int u = u0 + 8 * si + (r >> 4);
        if (u < u1) {
            int ji, row0, nrows;
            locate(u, ji, row0, nrows);
            const int rr = (r & 15) < nrows ? (r & 15) : 0;   // (a unit's missing rows: its first row again; nothing of them is kept)
            const u8* src = a.job[ji].w + (size_t)(row0 + rr) * rb + (size_t)p * c.sb - s_off;
            u8* dst = stages + (size_t)(si & 1) * stage_bytes + (size_t)r * c.rs;
            for (int ch = threadIdx.x & 1; ch < chunks; ch += 2) sz_cp_async16(dst + ch * 16, src + ch * 16);
        }
        sz_cp_async_commit();
    };
    issue(0);   // (the matrices are constants: their first stage is on its way before the kernel waits for its inputs)
    sz_pdl_wait();
    sz_pdl_trigger();
    for (int i = threadIdx.x; i < ng * 8 * (part / 4); i += 256) {
        const int j = i / (part / 4), c4 = i - j * (part / 4);
        const float4 v = __ldcg((const float4*)(a.x + (size_t)(g0 * 8 + j) * a.xstride + (size_t)p * part) + c4);
        const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        const __half2 l0 = __floats2half2_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2half2_rn(v.z - f1.x, v.w - f1.y);
        *(uint2*)(xhi + (size_t)j * c.xs + 4 * c4) = make_uint2(*(const u32*)&h0, *(const u32*)&h1);
        *(uint2*)(xlo + (size_t)j * c.xs + 4 * c4) = make_uint2(*(const u32*)&l0, *(const u32*)&l1);
    }
    for (int si = 0; si < nstage; si++) {
        if (si + 1 < nstage) issue(si + 1); else sz_cp_async_commit();
        sz_cp_async_wait1();          // this thread's copies of stage si have landed ...
        __syncthreads();              // ... and everybody's (and, the first time, the rows)
        const int u = u0 + 8 * si + warp;
        if (u < u1) {
            int ji, row0, nrows;
            locate(u, ji, row0, nrows);
            const SzDenseJob& jb = a.job[ji];
            const u8* st = stages + (size_t)(si & 1) * stage_bytes + (size_t)(warp * 16) * c.rs + s_off;
            const u8* r0 = st + (size_t)(g < nrows ? g : 0) * c.rs;
            const u8* r1 = st + (size_t)(g + 8 < nrows ? g + 8 : 0) * c.rs;
            float acc[GB][4];
#pragma unroll
            for (int gi = 0; gi < GB; gi++) { acc[gi][0] = 0.f; acc[gi][1] = 0.f; acc[gi][2] = 0.f; acc[gi][3] = 0.f; }
            for (int b = 0; b < nblk; b++) {
                const int col = b * 32 + 8 * q;
                const u8* p0 = r0 + (size_t)b * 34;
                const u8* p1 = r1 + (size_t)b * 34;
                const float d0 = sz_f16_to_f32(*(const u16*)p0), d1 = sz_f16_to_f32(*(const u16*)p1);
                const u16* c0 = (const u16*)(p0 + 2 + 8 * q);
                const u16* c1 = (const u16*)(p1 + 2 + 8 * q);
                u32 a1[4], a2[4];
                a1[0] = sz_q8_pair(c0[0]); a1[2] = sz_q8_pair(c0[1]); a2[0] = sz_q8_pair(c0[2]); a2[2] = sz_q8_pair(c0[3]);
                a1[1] = sz_q8_pair(c1[0]); a1[3] = sz_q8_pair(c1[1]); a2[1] = sz_q8_pair(c1[2]); a2[3] = sz_q8_pair(c1[3]);
#pragma unroll
                for (int gi = 0; gi < GB; gi++) {
                    if (gi < ng) {
                        const uint4 bh = *(const uint4*)(xhi + (size_t)(gi * 8 + g) * c.xs + col);
                        const uint4 bl = *(const uint4*)(xlo + (size_t)(gi * 8 + g) * c.xs + col);
                        float t[4] = {0.f, 0.f, 0.f, 0.f};
                        sz_mma16816_z(t, a1, bh.x, bh.y);
                        sz_mma16816_z(t, a2, bh.z, bh.w);
                        sz_mma16816_z(t, a1, bl.x, bl.y);
                        sz_mma16816_z(t, a2, bl.z, bl.w);
                        acc[gi][0] = fmaf(d0, t[0], acc[gi][0]); acc[gi][1] = fmaf(d0, t[1], acc[gi][1]);
                        acc[gi][2] = fmaf(d1, t[2], acc[gi][2]); acc[gi][3] = fmaf(d1, t[3], acc[gi][3]);
                    }
                }
            }
            const size_t T = (size_t)a.total_rows;
            const size_t o = (size_t)jb.row0 + row0 + g;
#pragma unroll
            for (int gi = 0; gi < GB; gi++) {
                if (gi < ng) {
                    float* P = c.partial + ((size_t)p * c.rows + (size_t)(g0 + gi) * 8 + 2 * q) * T + o;
                    if (g < nrows) { P[0] = acc[gi][0]; P[T] = acc[gi][1]; }
                    if (g + 8 < nrows) { P[8] = acc[gi][2]; P[T + 8] = acc[gi][3]; }
                }
            }
        }
        __syncthreads();              // the stage is free for the copies of stage si + 2
    }
}

// grid (ceil(outputs / 256), rows); block 256: the eight parts' sums in order, the epilogue, the job's output
static __global__ void __launch_bounds__(256) sz_dense_rows_reduce_kernel(const SzDenseArgs a, const float* __restrict__ partial, int rows) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int o = blockIdx.x * 256 + threadIdx.x, row = blockIdx.y;
    if (o >= a.total_rows) return;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) v += __ldcg(partial + ((size_t)w * rows + row) * a.total_rows + o);
    int ji = 0;
#pragma unroll
    for (int t = 1; t < SZ_DENSE_MAX_JOBS; t++)
        if (t < a.n_jobs && o >= a.job[t].row0) ji = t;
    const SzDenseJob& jb = a.job[ji];
    jb.out[(size_t)row * jb.ostride + (o - jb.row0)] = sz_epilogue(jb.epi, v, jb.div);
}

#endif  // __CUDACC__

// host: launches the jobs of `a` (row0 / total_rows are filled here)
int sz_dense_launch(SzDenseArgs& a, cudaStream_t st, const char* name);
// a.m rows, a multiple of 8 (any number of them), through the many-row form of the Q8_0 tensor-pipe kernel when sz_dense_launch would
// take that kernel for 8 rows of these jobs: *taken = 1 and the rows are computed (bit for bit as 8 at a time); otherwise *taken = 0
// and nothing is launched.  partial: a.m * total rows * 8 floats of scratch.
int sz_dense_rows_launch(SzDenseArgs& a, float* partial, int64_t partial_floats, cudaStream_t st, const char* name, int* taken);
int sz_dense_check(const sz_tensor* t, const char* what, int64_t rows, int64_t cols);
