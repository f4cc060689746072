// Expert FFN of a verify pass for the ggml block formats (Q8_0, IQ3_S), streaming form.
//
// The same skeleton as the dense Q8_0 projection kernel: units of 16 matrix rows are copied into a ring of shared-memory stages by the
// TMA engine (cp.async.bulk) while the warps work on the previous unit; a warp owns one eighth of the columns; per 32-column block it
// turns the two rows' codes into f16 exactly, multiplies them on mma.sync with the rows of the group (the B operand, f16 high and low
// parts) and adds the product, times the block's scale, to its running sums; the eight column parts of a row meet in shared memory.
// What differs is the bookkeeping of a mixture of experts: a unit belongs to a group of the routed plan (an expert and the rows
// that chose it), the B operand holds only that group's rows (gathered once per group), and the results go to the rows of the
// per-pair buffers.  Gate and up are staged and multiplied together and leave as silu(gate) * up.
// The decode follows crates/shadowzero-model/src/quant.rs:148-159 (IQ3_S) and :174-179 (Q8_0).
#pragma once

#include "sz_dense.cuh"
#include "sz_moe.cuh"

struct SzBlkCfg {
    int NS;          // stages
    int rbp;         // bytes between staged rows (the row bytes, padded when rows are copied one by one)
    int by_row;      // 1: one bulk copy a row (row bytes are a multiple of 16); 0: the 16 rows of a unit in one copy
    int unit_bytes;  // a stage: 16 rows (x 2 matrices for gate / up)
    int xsp;         // halves between the staged rows of the group
    int slices;      // units an expert's matrix has (16 * RT rows each)
};

// the A fragments (two k-halves: columns 8q..8q+3 | 8q+4..8q+7 of the block) of rows r0, r1 for 32-column block `blk`, and the rows' scales
template <int TYPE>
__device__ __forceinline__ void sz_blk_frag(const u8* r0, const u8* r1, int blk, int q, const u32* grid, const uint4* slut, u32* a1, u32* a2,
                                            float& d0, float& d1) {
    if (TYPE == SZ_TYPE_Q8_0) {
        const u8* p0 = r0 + (size_t)blk * 34;
        const u8* p1 = r1 + (size_t)blk * 34;
        d0 = sz_f16_to_f32(*(const u16*)p0); d1 = sz_f16_to_f32(*(const u16*)p1);
        const u16* c0 = (const u16*)(p0 + 2 + 8 * q);
        const u16* c1 = (const u16*)(p1 + 2 + 8 * q);
        a1[0] = sz_q8_pair(c0[0]); a1[2] = sz_q8_pair(c0[1]); a2[0] = sz_q8_pair(c0[2]); a2[2] = sz_q8_pair(c0[3]);
        a1[1] = sz_q8_pair(c1[0]); a1[3] = sz_q8_pair(c1[1]); a2[1] = sz_q8_pair(c1[2]); a2[3] = sz_q8_pair(c1[3]);
    } else {  // IQ3_S: superblock of 256 = 8 blocks of 32; this lane's 8 weights are two grid entries and one byte of signs
        const int sb = blk >> 3, b32 = blk & 7;
        const __half2 k1024 = __halves2half2(__ushort_as_half((u16)0x6400), __ushort_as_half((u16)0x6400));
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const u8* p = (r ? r1 : r0) + (size_t)sb * 110;
            const float d = sz_f16_to_f32(*(const u16*)p);
            const u32 qs2 = *(const u16*)(p + 2 + 8 * b32 + 2 * q);
            const u32 qh = p[66 + b32] >> (2 * q);
            const u32 sg = p[74 + 4 * b32 + q];
            const u32 sc = (p[106 + (b32 >> 1)] >> (4 * (b32 & 1))) & 15u;
            const u32 m0 = grid[(qs2 & 0xffu) | ((qh & 1u) << 8)];
            const u32 m1 = grid[(qs2 >> 8) | ((qh & 2u) << 7)];
            const uint4 sm = slut[sg];  // sign masks of the four f16 pairs
            u32 t0 = __byte_perm(m0, 0x64646464u, 0x4140), t1 = __byte_perm(m0, 0x64646464u, 0x4342);
            u32 t2 = __byte_perm(m1, 0x64646464u, 0x4140), t3 = __byte_perm(m1, 0x64646464u, 0x4342);
            __half2 h0 = __hsub2(*(const __half2*)&t0, k1024), h1 = __hsub2(*(const __half2*)&t1, k1024);
            __half2 h2 = __hsub2(*(const __half2*)&t2, k1024), h3 = __hsub2(*(const __half2*)&t3, k1024);
            a1[r] = *(const u32*)&h0 ^ sm.x; a1[2 + r] = *(const u32*)&h1 ^ sm.y;
            a2[r] = *(const u32*)&h2 ^ sm.z; a2[2 + r] = *(const u32*)&h3 ^ sm.w;
            (r ? d1 : d0) = d * (float)(1u + 2u * sc);
        }
    }
}

// grid: any; block 256.  DOWN = false: out[pair][r] = silu(gate_r . x_row) * (up_r . x_row) with x = in[rows of the group]; true:
// out[pair][r] = down_r . in[pair].  n_in: columns (a multiple of 256); n_out: rows of the matrices (a multiple of 16).
// RT: 16-row tiles of a unit (the down matrices have short rows - FF columns - so a unit takes several tiles to be worth its barriers).
// dynamic shared memory: 64 (barriers) | 2048 (IQ3_S grid) | 4096 (sign masks) | NM * RT * 4096 (reduction) | 2 * 8 * xsp * 2 (B operand) | NS * unit_bytes
template <int TYPE, bool DOWN, int RT>
__global__ void __launch_bounds__(256)
sz_blk_ffn_kernel(const SzPlan* __restrict__ plan, const u8* __restrict__ w0, u64 stride0, const u8* __restrict__ w1, u64 stride1,
                  const float* __restrict__ in, int n_in, int n_out, float* __restrict__ out, const SzBlkCfg c, u32* __restrict__ ctrl) {
    extern __shared__ __align__(128) u8 smem[];
    constexpr int NM = DOWN ? 1 : 2;   // matrices staged per unit
    constexpr int UR = 16 * RT;        // rows of a unit (per matrix)
    static_assert(NM * RT <= 4, "the reduction buffer holds four 16-row tiles");
    u64* bars = (u64*)smem;
    u32* grid = (u32*)(smem + 64);
    uint4* slut = (uint4*)(smem + 64 + 2048);
    float* red = (float*)(smem + 64 + 2048 + 4096);           // [NM * RT][8 warps][16 rows][8 group rows]
    __half* xhi = (__half*)(smem + 64 + 2048 + 4096 + NM * RT * 4096); // [8][xsp]
    __half* xlo = xhi + (size_t)SZ_MAX_VERIFY * c.xsp;
    u8* stages = (u8*)(xlo + (size_t)SZ_MAX_VERIFY * c.xsp);
    __shared__ __align__(16) SzPlan splan;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const size_t rb = TYPE == SZ_TYPE_Q8_0 ? (size_t)(n_in / 32) * 34 : (size_t)(n_in / 256) * 110;
    if (threadIdx.x == 0) {
        for (int i = 0; i < c.NS; i++) sz_mbar_init(&bars[i], 1);
        sz_mbar_fence_init();
    }
    if (TYPE == SZ_TYPE_IQ3_S) {
        for (int i = threadIdx.x; i < 512; i += 256) grid[i] = c_iq3s_grid[i];
        {   // sign byte -> the sign bits of the four f16 pairs (bit 2k of the byte: low half of pair k, bit 2k + 1: high half)
            const u32 s = threadIdx.x;
            slut[s] = make_uint4(((s & 1u) << 15) | ((s & 2u) << 30), ((s & 4u) << 13) | ((s & 8u) << 28), ((s & 16u) << 11) | ((s & 32u) << 26),
                                 ((s & 64u) << 9) | ((s & 128u) << 24));
        }
    }
    sz_pdl_wait();
    sz_pdl_trigger();
    plan = sz_plan_stage(plan, &splan);
    __syncthreads();
    const int NG = plan->n_groups;
    const long long U = (long long)NG * c.slices;
    const int u0 = (int)(U * blockIdx.x / gridDim.x), u1 = (int)(U * (blockIdx.x + 1) / gridDim.x);
    const int count = u1 - u0;
    if (count <= 0) return;
    auto issue = [&](int i) {  // thread 0
        const int u = u0 + i, gi = u / c.slices, sl = u - gi * c.slices;
        const u64 e = (u64)plan->expert[gi];
        u64* bar = &bars[i % c.NS];
        u8* dst = stages + (size_t)(i % c.NS) * c.unit_bytes;
        sz_mbar_expect_tx(bar, (u32)(NM * UR * rb));
#pragma unroll
        for (int mtx = 0; mtx < NM; mtx++) {
            const u8* src = (mtx ? w1 + e * stride1 : w0 + e * stride0) + (size_t)sl * UR * rb;
            u8* d = dst + (size_t)mtx * UR * c.rbp;
            if (c.by_row) {
                for (int r = 0; r < UR; r++) sz_bulk_g2s(d + (size_t)r * c.rbp, src + (size_t)r * rb, (u32)rb, bar);
            } else {
                sz_bulk_g2s(d, src, (u32)(UR * rb), bar);
            }
        }
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < c.NS - 1 && i < count; i++) issue(i);
    const int part = n_in / 8, nblk = part / 32;   // this warp's columns: [warp * part, (warp + 1) * part)
    int cur_g = -1, n = 0;
    int failed = 0;
    for (int i = 0; i < count; i++) {
        if (threadIdx.x == 0 && i + c.NS - 1 < count) issue(i + c.NS - 1);
        const int u = u0 + i, gi = u / c.slices, sl = u - gi * c.slices;
        if (gi != cur_g) {  // a new group: its rows become the B operand (f16 high and low parts)
            __syncthreads();
            cur_g = gi;
            n = plan->count[gi];
            const u8* src_rows = DOWN ? plan->pairs[gi] : plan->rows[gi];
            for (int idx = threadIdx.x; idx < n * (n_in / 4); idx += 256) {
                const int t = idx / (n_in / 4), c4 = idx - t * (n_in / 4);
                const float4 v = __ldcg((const float4*)(in + (size_t)src_rows[t] * n_in) + c4);
                const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
                const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
                const __half2 l0 = __floats2half2_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2half2_rn(v.z - f1.x, v.w - f1.y);
                *(uint2*)(xhi + (size_t)t * c.xsp + 4 * c4) = make_uint2(*(const u32*)&h0, *(const u32*)&h1);
                *(uint2*)(xlo + (size_t)t * c.xsp + 4 * c4) = make_uint2(*(const u32*)&l0, *(const u32*)&l1);
            }
            __syncthreads();
        }
        if (!sz_mbar_wait(&bars[i % c.NS], (i / c.NS) & 1)) failed = 1;
        const u8* st = stages + (size_t)(i % c.NS) * c.unit_bytes;
        float acc[NM * RT][4];
#pragma unroll
        for (int mtx = 0; mtx < NM * RT; mtx++) { acc[mtx][0] = 0.f; acc[mtx][1] = 0.f; acc[mtx][2] = 0.f; acc[mtx][3] = 0.f; }
        if (!failed) {
            for (int b = 0; b < nblk; b++) {
                const int blk = warp * nblk + b;
                const int col = blk * 32 + 8 * q;
                uint4 bh = make_uint4(0, 0, 0, 0), bl = make_uint4(0, 0, 0, 0);
                if (g < n) {
                    bh = *(const uint4*)(xhi + (size_t)g * c.xsp + col);
                    bl = *(const uint4*)(xlo + (size_t)g * c.xsp + col);
                }
#pragma unroll
                for (int mtx = 0; mtx < NM * RT; mtx++) {  // tile mtx: rows 16 mtx .. 16 mtx + 15 of the stage (gate tiles, then up tiles)
                    const u8* r0 = st + (size_t)(mtx * 16 + g) * c.rbp;
                    const u8* r1 = st + (size_t)(mtx * 16 + g + 8) * c.rbp;
                    u32 a1[4], a2[4];
                    float d0, d1;
                    sz_blk_frag<TYPE>(r0, r1, blk, q, grid, slut, a1, a2, d0, d1);
                    float t[4] = {0.f, 0.f, 0.f, 0.f};
                    sz_mma16816_z(t, a1, bh.x, bh.y);
                    sz_mma16816_z(t, a2, bh.z, bh.w);
                    sz_mma16816_z(t, a1, bl.x, bl.y);
                    sz_mma16816_z(t, a2, bl.z, bl.w);
                    acc[mtx][0] = fmaf(d0, t[0], acc[mtx][0]); acc[mtx][1] = fmaf(d0, t[1], acc[mtx][1]);
                    acc[mtx][2] = fmaf(d1, t[2], acc[mtx][2]); acc[mtx][3] = fmaf(d1, t[3], acc[mtx][3]);
                }
            }
        }
        // the eight column parts of a row meet in shared memory
#pragma unroll
        for (int mtx = 0; mtx < NM * RT; mtx++) {
            float* rd = red + (size_t)mtx * 1024;
            rd[(warp * 16 + g) * 8 + 2 * q] = acc[mtx][0];
            rd[(warp * 16 + g) * 8 + 2 * q + 1] = acc[mtx][1];
            rd[(warp * 16 + g + 8) * 8 + 2 * q] = acc[mtx][2];
            rd[(warp * 16 + g + 8) * 8 + 2 * q + 1] = acc[mtx][3];
        }
        if (__syncthreads_or(failed)) { failed = 1; break; }
        for (int idx = threadIdx.x; idx < UR * 8; idx += 256) {
            const int rr = idx >> 3, t = idx & 7;   // row of the unit, row of the group
            if (t < n) {
                const int tile = rr >> 4, r16 = rr & 15;
                float v = 0.f, v2 = 0.f;
#pragma unroll
                for (int w = 0; w < 8; w++) {
                    v += red[tile * 1024 + (w * 16 + r16) * 8 + t];
                    if (!DOWN) v2 += red[(RT + tile) * 1024 + (w * 16 + r16) * 8 + t];
                }
                const int pair = plan->pairs[gi][t];
                out[(size_t)pair * n_out + sl * UR + rr] = DOWN ? v : sz_silu(v) * v2;
            }
        }
        __syncthreads();
    }
    if (failed && threadIdx.x == 0) atomicExch(&ctrl[1], 1u);
}
