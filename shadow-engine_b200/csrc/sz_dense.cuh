// Dense projections of a verify pass: y[j] = W x[j] for the 1..8 rows of the pass, W in any of the stored types.
// The role of the reference's matvec_cols_* family (kernels/matvec.cu:677-756) and multi_cols (crates/shadowzero-cuda/src/session.rs:
// 7346-7398: several projections of one input in a launch).  A warp takes a matrix row, a lane four consecutive weights of every
// 128, the inputs sit in shared memory; f32 accumulate.
#pragma once

#include "sz_formats.cuh"

#define SZ_DENSE_MAX_JOBS 4
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

// the lane's four weights at columns e .. e + 3 of `row`, and the scale they share
__device__ __forceinline__ void sz_dense_w4(int type, const u8* __restrict__ row, int e, const u32* grid, float* w, float& scale) {
    if (type == SZ_TYPE_F32) {
        const float4 v = __ldg((const float4*)(row + (size_t)e * 4));
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; scale = 1.f;
    } else if (type == SZ_TYPE_BF16) {
        const uint2 v = __ldg((const uint2*)(row + (size_t)e * 2));
        w[0] = __uint_as_float(v.x << 16); w[1] = __uint_as_float(v.x & 0xffff0000u);
        w[2] = __uint_as_float(v.y << 16); w[3] = __uint_as_float(v.y & 0xffff0000u); scale = 1.f;
    } else if (type == SZ_TYPE_F16) {
        const uint2 v = __ldg((const uint2*)(row + (size_t)e * 2));
        w[0] = sz_f16_to_f32((u16)(v.x & 0xffff)); w[1] = sz_f16_to_f32((u16)(v.x >> 16));
        w[2] = sz_f16_to_f32((u16)(v.y & 0xffff)); w[3] = sz_f16_to_f32((u16)(v.y >> 16)); scale = 1.f;
    } else if (type == SZ_TYPE_Q8_0) {
        const u8* blk = row + (e >> 5) * 34;
        const int i = e & 31;
        scale = sz_f16_to_f32(__ldg((const u16*)blk));
        const u32 q01 = __ldg((const u16*)(blk + 2 + i)), q23 = __ldg((const u16*)(blk + 4 + i));
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
                sz_dense_w4(jb.type, row, e, grid, w, scale);
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

#endif  // __CUDACC__

// host: launches the jobs of `a` (row0 / total_rows are filled here)
int sz_dense_launch(SzDenseArgs& a, cudaStream_t st, const char* name);
int sz_dense_check(const sz_tensor* t, const char* what, int64_t rows, int64_t cols);
