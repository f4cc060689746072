// EXL3 expert FFN for a verify pass, streaming form.
//
// Work is cut into units of one 128-input block (8 tile rows) by 8 * NTC tile columns of one matrix: 8 * (8 NTC) tiles, 24 KB at
// K = 3, NTC = 4.  A block of 8 warps walks a contiguous range of units; the TMA engine (cp.async.bulk) keeps the next units'
// trellis bytes arriving in a ring of shared-memory stages while the warps decode the current one.  Each lane decodes the 8
// weights of a tile that the format assigns it (crates/shadowzero-model/src/exl3.rs:9-14) straight into the A fragment of
// mma.sync.m16n8k16 - a tile IS one 16 (outputs) x 16 (inputs) A fragment - and the rows of the pass are the B operand, split into
// an f16 high and low part (two MMAs into one f32 accumulator) so the activations keep f32 accuracy.  The multiply-adds thus cost
// no issue slots; what is left on the ALUs is the trellis decode itself.
//
// A unit only covers part of the input, so its results are partial sums.  They are added into 64-bit fixed-point accumulators
// (scale 2^34) with integer atomics: integer addition is associative, so the sum does not depend on which block finishes first and
// the result is bit-for-bit reproducible, which float atomics would not give.
#pragma once

#include "sz_moe.cuh"

#define SZ_X3_THREADS 256
#define SZ_X3_STAGES 4
#define SZ_X3_TICKET 2   // ctrl[2]: the unit counter of the gate / up kernel, ctrl[3]: of the down kernel (the router kernel clears both)
#define SZ_FIX_SCALE 17179869184.0f           // 2^34
#define SZ_FIX_INV (1.0 / 17179869184.0)

template <int K, int NTC>
struct SzX3 {
    static constexpr int TILE_BYTES = 32 * K;
    static constexpr int ROW_BYTES = 8 * NTC * TILE_BYTES;  // one tile row of the unit
    static constexpr int STAGE_BYTES = 8 * ROW_BYTES;
    static constexpr int FRAG_BYTES = 2 * 8 * 32 * 16;
    static constexpr int SMEM_BYTES = SZ_X3_STAGES * STAGE_BYTES + FRAG_BYTES + SZ_X3_STAGES * 8 + 16;
};

__device__ __forceinline__ void sz_mma16816(float* c, const u32* a, u32 b0, u32 b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The lane's 8 weights of a tile as the A fragment (outputs x inputs) of m16n8k16: a0 = (out g, in 2q..), a1 = (out g + 8, in 2q..),
// a2 = (out g, in 2q + 8..), a3 = (out g + 8, in 2q + 8..) with g = lane / 4, q = lane % 4: tile positions j = {0,1}, {4,5}, {2,3}, {6,7}.
// The codebook's byte sum (exl3.rs:66-86: the four bytes of state * 0x83DCD12D, plus 0x6400) for four states at once on the integer
// tensor pipe: the products are the A operand of mma.m16n8k32.u8 as they stand (a register = one product = four k slots), the B
// operand is a constant 0/1 matrix that routes each register's four bytes to an output column of the same lane, and the
// accumulator starts at 0x6400.  c[i] = 0x6400 + bytes of x[i].  Two of these replace eight dp4a in the issue stream.
__device__ __forceinline__ void sz_bytesum4(const u32* x, u32 sel0, u32 sel1, u32* c) {
    c[0] = 0x6400u; c[1] = 0x6400u; c[2] = 0x6400u; c[3] = 0x6400u;
    // A registers: a0 = (row g, k 4q..), a1 = (row g + 8, k 4q..), a2 = (row g, k 16 + 4q..), a3 = (row g + 8, k 16 + 4q..)
    // C registers: c0 = (row g, col 2q), c1 = (row g, col 2q + 1), c2 = (row g + 8, col 2q), c3 = (row g + 8, col 2q + 1)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(x[0]), "r"(x[2]), "r"(x[1]), "r"(x[3]), "r"(sel0), "r"(sel1));
}

template <int K>
__device__ __forceinline__ void sz_exl3_afrag(const u32* tile, int lane, const typename SzExl3Tile<K>::Lane& LS, u32* a) {
    u32 st[8];
    SzExl3Tile<K>::states_pre(tile, LS, st);
    const __half2 kinv = __halves2half2(__ushort_as_half((u16)0x1eee), __ushort_as_half((u16)0x1eee));
    const __half2 kbias = __halves2half2(__ushort_as_half((u16)0xc931), __ushort_as_half((u16)0xc931));
    // B operand (k x n, column n = lane / 4 of this lane, k rows 4q.. in the first register, 16 + 4q.. in the second): column 2q'
    // takes the bytes k = 4q'.. (register a0 / a1 of lane q'), column 2q' + 1 the bytes k = 16 + 4q'.. (a2 / a3)
    const int n = lane >> 2, q = lane & 3;
    const u32 sel0 = ((n & 1) == 0 && (n >> 1) == q) ? 0x01010101u : 0u;
    const u32 sel1 = ((n & 1) == 1 && (n >> 1) == q) ? 0x01010101u : 0u;
    u32 x[8];
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = st[i] * 0x83DCD12Du;
    u32 c[8];
    sz_bytesum4(x, sel0, sel1, c);          // c0 = sum(x0), c1 = sum(x1), c2 = sum(x2), c3 = sum(x3)
    sz_bytesum4(x + 4, sel0, sel1, c + 4);
    u32 p[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const u32 packed = __byte_perm(c[2 * i], c[2 * i + 1], 0x5410);
        const __half2 h = __hfma2(*(const __half2*)&packed, kinv, kbias);
        p[i] = *(const u32*)&h;
    }
    a[0] = p[0]; a[1] = p[2]; a[2] = p[1]; a[3] = p[3];
}

// One unit's description.
struct SzX3Unit {
    const u8* src;        // first byte of the unit's first tile row
    u64 row_stride;       // bytes between the unit's tile rows in global memory
    const u16* suh;       // the 128 input signs/scales of the unit's input block
    int n;                // rows in the group
    const u8* rows;   // null: rows are 0..n-1 (the shared expert)
    const u8* pairs; // null: pair = pair0 + t
    int pair0;
    int in_off;           // first input index of the block
};

// Writes the B fragments (the group's rows, rotated into the trellis' basis, f16 high and low parts) of one 128-input block.
// v[e]: warp t's row t, element lane + 32 e, already multiplied by suh.  frag: [8 tile rows][32 lanes] of {hi b0, hi b1, lo b0, lo b1}.
__device__ __forceinline__ void sz_x3_store_frag(uint4* frag, int t, int n, float* v, int lane) {
    if (t < n) {
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
    } else {
        frag[(lane >> 2) * 32 + 4 * t + (lane & 3)] = make_uint4(0, 0, 0, 0);
    }
}

// Decodes and multiplies one staged unit: c[tc] accumulates outputs (warp * NTC + tc) * 16 + {g, g + 8} for rows 2q, 2q + 1.
template <int K, int NTC>
__device__ __forceinline__ void sz_x3_compute(const u8* stage, const uint4* frag, int warp, int lane, float (*c)[4]) {
#pragma unroll
    for (int tc = 0; tc < NTC; tc++) { c[tc][0] = 0.f; c[tc][1] = 0.f; c[tc][2] = 0.f; c[tc][3] = 0.f; }
    const typename SzExl3Tile<K>::Lane LS = SzExl3Tile<K>::lane_setup(lane);
    const u8* wbase = stage + (size_t)(warp * NTC) * (32 * K);
    const uint4* fl = frag + lane;
#pragma unroll
    for (int kr = 0; kr < 8; kr++) {
        const uint4 b = fl[kr * 32];
#pragma unroll
        for (int tc = 0; tc < NTC; tc++) {
            const u32* tile = (const u32*)(wbase + (size_t)(kr * 8 * NTC + tc) * (32 * K));
            u32 a[4];
            sz_exl3_afrag<K>(tile, lane, LS, a);
            sz_mma16816(c[tc], a, b.x, b.y);
            sz_mma16816(c[tc], a, b.z, b.w);
        }
    }
}

// The routed plan into shared memory in one cooperative sweep: its fields are then a shared-memory read away instead of a chain of
// dependent loads from L2 (group count -> expert -> rows -> activations).
__device__ __forceinline__ const SzPlan* sz_plan_stage(const SzPlan* __restrict__ plan, SzPlan* sp) {
    if (!plan) return nullptr;
    static_assert(sizeof(SzPlan) % 16 == 0, "SzPlan is copied in 16-byte pieces");
    const uint4* src = (const uint4*)plan;
    uint4* dst = (uint4*)sp;
    for (int i = threadIdx.x; i < (int)(sizeof(SzPlan) / 16); i += blockDim.x) dst[i] = __ldcg(src + i);
    return sp;
}

__device__ __forceinline__ void sz_fix_add(long long* dst, float v) {
    atomicAdd((unsigned long long*)dst, (unsigned long long)__float2ll_rn(v * SZ_FIX_SCALE));
}

// ---- gate / up --------------------------------------------------------------------------------------------------------------------
// Units: group x input block x {gate, up}; a unit is contiguous in memory (every tile column of 8 tile rows).
// acc: i64 [pairs][2][FF]: pre-rotation sums of gate (0) and up (1) for every pair, zero on entry.
template <int K, int NTC>
__global__ void __launch_bounds__(SZ_X3_THREADS, 2)
sz_x3_gateup_kernel(const SzPlan* __restrict__ plan, const u8* __restrict__ gate, u64 gstride, const u8* __restrict__ up, u64 ustride,
                    const u8* __restrict__ sh_gate, const u8* __restrict__ sh_up, const float* __restrict__ x, int m, int H, int top_k,
                    long long* __restrict__ acc, u32* __restrict__ ctrl) {
    using X = SzX3<K, NTC>;
    constexpr int FF = 128 * NTC;
    extern __shared__ __align__(128) u8 smem[];
    u8* stages = smem;
    uint4* frags = (uint4*)(smem + SZ_X3_STAGES * X::STAGE_BYTES);
    u64* bars = (u64*)(smem + SZ_X3_STAGES * X::STAGE_BYTES + X::FRAG_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    SZ_PH_DECL;
    SZ_PH();  // 0
    if (threadIdx.x == 0) {
        for (int i = 0; i < SZ_X3_STAGES; i++) sz_mbar_init(&bars[i], 1);
        sz_mbar_fence_init();
    }
    sz_pdl_wait();
    sz_pdl_trigger();
    __shared__ __align__(16) SzPlan splan;
    plan = sz_plan_stage(plan, &splan);
    __syncthreads();
    SZ_PH();  // 1 after wait
#ifdef SZ_PHASES
    if (threadIdx.x == 0 && blockIdx.x == 0) { sz_phase_t[5][4] = (long long)sz_gtime(); sz_phase_t[5][0] = 0; sz_phase_t[5][1] = 0x7fffffffffffffffll; sz_phase_t[5][2] = 0; }
#endif
    const int D = plan ? plan->n_groups : 0;
    const int NG = D + (sh_gate ? 1 : 0);
    const int NS = H / 128;
    const long long U = (long long)NG * NS * 2;
    // Which units a block takes.  Few units (a pass of one or two rows): a fixed contiguous share, so that nobody ends up with three
    // where others have one.  Many: the first unit is the block's number, the rest are drawn from a counter as the block goes, so
    // that blocks which got heavier units (more rows a group) or a slower start take fewer and all blocks end together.
    const bool dyn = U >= 3LL * gridDim.x;
    const int u0 = dyn ? (int)blockIdx.x : (int)(U * blockIdx.x / gridDim.x);
    const int u1 = dyn ? (int)U : (int)(U * (blockIdx.x + 1) / gridDim.x);
    if (u0 >= u1) return;
    const size_t hdr = 2 * (size_t)H + 2 * (size_t)FF + 4;

    auto unit = [&](int u) {
        SzX3Unit d;
        const int g = u / (2 * NS), rem = u % (2 * NS), s = rem >> 1, mat = rem & 1;
        const u8* blob;
        if (g < D) {
            const u64 e = (u64)plan->expert[g];
            blob = mat ? up + e * ustride : gate + e * gstride;
            d.n = plan->count[g]; d.rows = plan->rows[g]; d.pairs = plan->pairs[g]; d.pair0 = 0;
        } else {
            blob = mat ? sh_up : sh_gate;
            d.n = m; d.rows = nullptr; d.pairs = nullptr; d.pair0 = m * top_k;
        }
        d.src = blob + hdr + (size_t)s * X::STAGE_BYTES;
        d.row_stride = X::ROW_BYTES;
        d.suh = (const u16*)blob + s * 128;
        d.in_off = s * 128 + (mat << 30);  // bit 30 carries the matrix index
        return d;
    };
    // the block's i-th unit lives in slot i % RING: its number (-1: the block has no i-th unit) and its description
    constexpr int RING = 16, LA = SZ_X3_STAGES - 1;
    __shared__ SzX3Unit ud[RING];
    __shared__ int uid[RING];
    auto issue = [&](int i) {  // thread 0: start the copy of the block's i-th unit into stage i % STAGES
        u64* bar = &bars[i % SZ_X3_STAGES];
        sz_mbar_expect_tx(bar, X::STAGE_BYTES);
        sz_bulk_g2s(stages + (size_t)(i % SZ_X3_STAGES) * X::STAGE_BYTES, ud[i % RING].src, X::STAGE_BYTES, bar);
    };
    auto prep_load = [&](const SzX3Unit& d, float* v) {  // warp t: row t of the group times suh, element lane + 32 e
        if (warp < d.n) {
            const int row = d.rows ? d.rows[warp] : warp;
            const int off = d.in_off & 0x3fffffff;
#pragma unroll
            for (int e = 0; e < 4; e++)
                v[e] = __ldg(x + (size_t)row * H + off + lane + 32 * e) * sz_f16_to_f32(__ldg(d.suh + lane + 32 * e));
        }
    };
    u32 pending = 0xffffffffu;  // thread 0, dynamic mode: the ticket asked for one round ago (for slot i + LA of round i)
    if (!dyn) {  // every slot now, in parallel (the static share is at most RING - 2 units long)
        if (threadIdx.x < RING) {
            const int u = u0 + threadIdx.x;
            uid[threadIdx.x] = u < u1 ? u : -1;
            if (u < u1) ud[threadIdx.x] = unit(u);
        }
        __syncthreads();
        if (threadIdx.x == 0)
            for (int i = 0; i < LA && uid[i] >= 0; i++) issue(i);
    } else {
        if (threadIdx.x == 0) {
            u32 t[LA];
            for (int i = 1; i < LA; i++) t[i] = atomicAdd(&ctrl[SZ_X3_TICKET], 1u) + gridDim.x;
            pending = atomicAdd(&ctrl[SZ_X3_TICKET], 1u) + gridDim.x;
            uid[0] = u0; ud[0] = unit(u0);
            issue(0);
            for (int i = 1; i < LA; i++) {
                const bool ok = t[i] < (u32)U;
                uid[i] = ok ? (int)t[i] : -1;
                if (ok) { ud[i] = unit((int)t[i]); issue(i); }
            }
        }
        __syncthreads();
    }
    SzX3Unit cur = ud[0];
    {
        float v[4];
        prep_load(cur, v);
        sz_x3_store_frag(frags, warp, cur.n, v, lane);
    }
    __syncthreads();
    SZ_PH();  // 2 first fragments
    int failed = 0, count = 0;
    for (int i = 0; uid[i % RING] >= 0; i++) {
        count++;
        if (threadIdx.x == 0) {  // slot i + LA: read by everybody from round i + LA - 1 on, two barriers from here
            const int sl = (i + LA) % RING;
            if (dyn) {
                const bool ok = pending < (u32)U;
                uid[sl] = ok ? (int)pending : -1;
                if (ok) {
                    ud[sl] = unit((int)pending);
                    issue(i + LA);
                    pending = atomicAdd(&ctrl[SZ_X3_TICKET], 1u) + gridDim.x;  // (its value is not looked at before the next round)
                }
            } else if (i + LA < RING ? uid[sl] >= 0 : false) {
                issue(i + LA);
            }
        }
        const bool more = uid[(i + 1) % RING] >= 0;
        SzX3Unit nxt = cur;
        float v[4];
        if (more) { nxt = ud[(i + 1) % RING]; prep_load(nxt, v); }
        if (i == 1) SZ_PH();  // unit 1: start
        if (!sz_mbar_wait(&bars[i % SZ_X3_STAGES], (i / SZ_X3_STAGES) & 1)) failed = 1;
        if (i == 1) SZ_PH();  // unit 1: data arrived
        float c[NTC][4];
        if (!failed) {
            sz_x3_compute<K, NTC>(stages + (size_t)(i % SZ_X3_STAGES) * X::STAGE_BYTES, frags + (i & 1) * 256, warp, lane, c);
            if (i == 1) SZ_PH();  // unit 1: decoded and multiplied
            const int mat = cur.in_off >> 30, q = lane & 3, g8 = lane >> 2;
#pragma unroll
            for (int tt = 0; tt < 2; tt++) {
                const int t = 2 * q + tt;
                if (t < cur.n) {
                    const int pair = cur.pairs ? cur.pairs[t] : cur.pair0 + t;
                    long long* dst = acc + ((size_t)pair * 2 + mat) * FF + (warp * NTC) * 16 + g8;
#pragma unroll
                    for (int tc = 0; tc < NTC; tc++) {
                        sz_fix_add(dst + tc * 16, c[tc][tt]);
                        sz_fix_add(dst + tc * 16 + 8, c[tc][2 + tt]);
                    }
                }
            }
        }
        if (i == 1) SZ_PH();  // unit 1: atomics issued
        if (more) sz_x3_store_frag(frags + ((i + 1) & 1) * 256, warp, nxt.n, v, lane);
        if (i == 1) SZ_PH();  // unit 1: next fragments stored
        cur = nxt;
        if (__syncthreads_or(failed)) { failed = 1; break; }
        SZ_PH();  // 3.. a unit
    }
    if (failed && threadIdx.x == 0) atomicExch(&ctrl[1], 1u);
    SZ_PH_FLUSH(4, blockIdx.x == 7);
#ifdef SZ_PHASES
    if (threadIdx.x == 0) {  // spread of the blocks' end times, and of their unit counts
        const unsigned long long te = sz_gtime();
        atomicMax((unsigned long long*)&sz_phase_t[5][0], te);
        atomicMin((unsigned long long*)&sz_phase_t[5][1], te);
        atomicMax((unsigned long long*)&sz_phase_t[5][2], (unsigned long long)count);
        if (blockIdx.x == 0) sz_phase_t[5][3] = (long long)te;
    }
#endif
}

// ---- down ---------------------------------------------------------------------------------------------------------------------------
// Units: group x input block (128 of FF) x output chunk (512 outputs = 32 tile columns); 8 tile rows of 32 tiles each, strided.
// The input of a unit is the SwiGLU product of its pairs, finished here from the gate/up accumulators: rotate back (H), scale by
// svh, silu(g) * u, then into the down trellis' basis (suh, H).  out: i64 [pairs][H], zero on entry.
template <int K>
__global__ void __launch_bounds__(SZ_X3_THREADS, 2)
sz_x3_down_kernel(const SzPlan* __restrict__ plan, const u8* __restrict__ gate, u64 gstride, const u8* __restrict__ up, u64 ustride,
                  const u8* __restrict__ down, u64 dstride, const u8* __restrict__ sh_gate, const u8* __restrict__ sh_up,
                  const u8* __restrict__ sh_down, int m, int H, int FF, int top_k, const long long* __restrict__ acc,
                  long long* __restrict__ out, u32* __restrict__ ctrl) {
    using X = SzX3<K, 4>;
    extern __shared__ __align__(128) u8 smem[];
    u8* stages = smem;
    uint4* frags = (uint4*)(smem + SZ_X3_STAGES * X::STAGE_BYTES);
    u64* bars = (u64*)(smem + SZ_X3_STAGES * X::STAGE_BYTES + X::FRAG_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < SZ_X3_STAGES; i++) sz_mbar_init(&bars[i], 1);
        sz_mbar_fence_init();
    }
    // the plan was finished two kernels ago; only the gate/up accumulators need the wait below
    __shared__ __align__(16) SzPlan splan;
    plan = sz_plan_stage(plan, &splan);
    __syncthreads();
    const int D = plan ? plan->n_groups : 0;
    const int NG = D + (sh_down ? 1 : 0);
    const int KB = FF / 128, NC = H / 512;
    const long long U = (long long)NG * KB * NC;
    const int u0 = (int)(U * blockIdx.x / gridDim.x), u1 = (int)(U * (blockIdx.x + 1) / gridDim.x);
    const int count = u1 - u0;
    const size_t hdr_d = 2 * (size_t)FF + 2 * (size_t)H + 4, hdr_g = 2 * (size_t)H + 2 * (size_t)FF + 4;
    (void)hdr_g;
    const u64 drow = (u64)(H / 16) * X::TILE_BYTES;  // bytes of one tile row of the down matrix

    struct DUnit { const u8* src; const u16 *svg, *svu, *suh; int n; const u8* pairs; int pair0; int kb, c; };
    auto unit = [&](int u) {
        DUnit d;
        const int g = u / (KB * NC), rem = u % (KB * NC);
        d.kb = rem / NC; d.c = rem % NC;
        const u8 *bg, *bu, *bd;
        if (g < D) {
            const u64 e = (u64)plan->expert[g];
            bg = gate + e * gstride; bu = up + e * ustride; bd = down + e * dstride;
            d.n = plan->count[g]; d.pairs = plan->pairs[g]; d.pair0 = 0;
        } else {
            bg = sh_gate; bu = sh_up; bd = sh_down;
            d.n = m; d.pairs = nullptr; d.pair0 = m * top_k;
        }
        d.src = bd + hdr_d + (size_t)d.kb * 8 * drow + (size_t)d.c * X::ROW_BYTES;
        d.svg = (const u16*)(bg + 2 * (size_t)H) + d.kb * 128;
        d.svu = (const u16*)(bu + 2 * (size_t)H) + d.kb * 128;
        d.suh = (const u16*)bd + d.kb * 128;
        return d;
    };
    constexpr int UD = 12;
    __shared__ DUnit ud[UD];
    auto unit_at = [&](int i) { return i < UD ? ud[i] : unit(u0 + i); };
    auto issue = [&](int i) {
        const DUnit d = unit_at(i);
        u64* bar = &bars[i % SZ_X3_STAGES];
        u8* dst = stages + (size_t)(i % SZ_X3_STAGES) * X::STAGE_BYTES;
        sz_mbar_expect_tx(bar, X::STAGE_BYTES);
#pragma unroll
        for (int kr = 0; kr < 8; kr++) sz_bulk_g2s(dst + kr * X::ROW_BYTES, d.src + kr * drow, X::ROW_BYTES, bar);
    };
    // warp t: gate and up sums of pair t (elements lane + 32 e of block kb) and the scales that finish them
    auto prep_load = [&](const DUnit& d, long long* ag, long long* au, float* sc) {
        if (warp < d.n) {
            const int pair = d.pairs ? d.pairs[warp] : d.pair0 + warp;
            const long long* a = acc + (size_t)pair * 2 * FF + d.kb * 128;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = lane + 32 * e;
                ag[e] = __ldcg(a + i);
                au[e] = __ldcg(a + FF + i);
                sc[e] = sz_f16_to_f32(__ldg(d.svg + i));
                sc[4 + e] = sz_f16_to_f32(__ldg(d.svu + i));
                sc[8 + e] = sz_f16_to_f32(__ldg(d.suh + i));
            }
        }
    };
    auto prep_store = [&](const DUnit& d, long long* ag, long long* au, float* sc, uint4* frag) {
        float v[4];
        if (warp < d.n) {
            float g[4], u[4];
#pragma unroll
            for (int e = 0; e < 4; e++) { g[e] = (float)((double)ag[e] * SZ_FIX_INV); u[e] = (float)((double)au[e] * SZ_FIX_INV); }
            sz_wht128_warp(g, lane);
            sz_wht128_warp(u, lane);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float gv = (g[e] * SZ_RSQRT128) * sc[e], uv = (u[e] * SZ_RSQRT128) * sc[4 + e];
                v[e] = (sz_silu(gv) * uv) * sc[8 + e];
            }
        }
        sz_x3_store_frag(frag, warp, d.n, v, lane);
    };

    if (threadIdx.x < UD && threadIdx.x < count) ud[threadIdx.x] = unit(u0 + threadIdx.x);
    __syncthreads();
    if (count > 0 && threadIdx.x == 0)
        for (int i = 0; i < SZ_X3_STAGES - 1 && i < count; i++) issue(i);
    sz_pdl_wait();
    sz_pdl_trigger();
    if (count <= 0) return;
    DUnit cur = unit_at(0);
    {
        long long ag[4], au[4];
        float sc[12];
        prep_load(cur, ag, au, sc);
        prep_store(cur, ag, au, sc, frags);
    }
    __syncthreads();
    int failed = 0;
    int fb = 0;  // which of the two fragment buffers holds the current unit's input
    for (int i = 0; i < count; i++) {
        if (threadIdx.x == 0 && i + SZ_X3_STAGES - 1 < count) issue(i + SZ_X3_STAGES - 1);
        DUnit nxt = cur;
        long long ag[4], au[4];
        float sc[12];
        // the output chunks of one (group, input block) follow one another and share their input: it is prepared once
        bool fresh = false;
        if (i + 1 < count) {
            nxt = unit_at(i + 1);
            fresh = nxt.kb != cur.kb || nxt.suh != cur.suh;
            if (fresh) prep_load(nxt, ag, au, sc);
        }
        if (!sz_mbar_wait(&bars[i % SZ_X3_STAGES], (i / SZ_X3_STAGES) & 1)) failed = 1;
        float c[4][4];
        if (!failed) {
            sz_x3_compute<K, 4>(stages + (size_t)(i % SZ_X3_STAGES) * X::STAGE_BYTES, frags + fb * 256, warp, lane, c);
            const int q = lane & 3, g8 = lane >> 2;
#pragma unroll
            for (int tt = 0; tt < 2; tt++) {
                const int t = 2 * q + tt;
                if (t < cur.n) {
                    const int pair = cur.pairs ? cur.pairs[t] : cur.pair0 + t;
                    long long* dst = out + (size_t)pair * H + cur.c * 512 + (warp * 4) * 16 + g8;
#pragma unroll
                    for (int tc = 0; tc < 4; tc++) {
                        sz_fix_add(dst + tc * 16, c[tc][tt]);
                        sz_fix_add(dst + tc * 16 + 8, c[tc][2 + tt]);
                    }
                }
            }
        }
        if (fresh) { prep_store(nxt, ag, au, sc, frags + (fb ^ 1) * 256); fb ^= 1; }
        cur = nxt;
        if (__syncthreads_or(failed)) { failed = 1; break; }
    }
    if (failed && threadIdx.x == 0) atomicExch(&ctrl[1], 1u);
}

// ---- combine ----------------------------------------------------------------------------------------------------------------------
// y[j] = sum over ranks of w * (H eo * svh) + sigmoid(shared gate logit) * (H so * svh_shared).  A block a (row, 128-output block);
// warp t finishes rank t's contribution (warp top_k: the shared expert's), then warp 0 adds them in rank order in f64.
// so_f32 != null: the shared expert's output comes finished (f32 [m][H]) from the generic kernels instead of the accumulators.
static __global__ void __launch_bounds__((SZ_MAX_TOPK + 1) * 32)
sz_x3_combine_kernel(const long long* __restrict__ out, const int32_t* __restrict__ ridx, const double* __restrict__ rw,
                     const u8* __restrict__ down, u64 dstride, const u8* __restrict__ sh_down, const float* __restrict__ so_f32,
                     const float* __restrict__ logits, int ne, int top_k, int m, int H, int FF, int has_shared, float* __restrict__ y,
                     long long* __restrict__ y_fix, int e_lo, int e_hi, const SzEpPush push) {
    __shared__ float part[SZ_MAX_TOPK + 1][128];
    __shared__ int local[SZ_MAX_TOPK];
    __shared__ double rws[SZ_MAX_TOPK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = H / 128;
    const int j = blockIdx.x / nb, b = blockIdx.x % nb;
    // Routing and scales do not come from the kernel before this one (the router ran three launches back, the scales are weights):
    // they are fetched ahead of the dependency wait, so that only the expert sums themselves are read after it.
    int e = 0;
    bool mine = false;
    float sv[4] = {0.f, 0.f, 0.f, 0.f};
    float sg = 0.f;
    if (warp < top_k) {
        const int pair = j * top_k + warp;
        e = (int)sz_ldg32_here(ridx + pair);
        mine = !y_fix || (e >= e_lo && e < e_hi);  // with expert parallelism only the experts held here count
        const u16* svh = (const u16*)(down + (u64)(mine ? e : e_lo) * dstride + 2 * (size_t)FF) + b * 128;
#pragma unroll
        for (int q = 0; q < 4; q++) sv[q] = sz_f16_to_f32(sz_ldg16b_here(svh + lane + 32 * q));
        if (lane == 0) { local[warp] = mine; rws[warp] = sz_ldg64f_here(rw + pair); }
    } else if (warp == top_k && has_shared) {
        sg = sz_sigmoid(__uint_as_float(sz_ldg32_here(logits + (size_t)j * (ne + 1) + ne)));
        if (!so_f32) {
            const u16* svh = (const u16*)(sh_down + 2 * (size_t)FF) + b * 128;
#pragma unroll
            for (int q = 0; q < 4; q++) sv[q] = sz_f16_to_f32(sz_ldg16b_here(svh + lane + 32 * q));
        }
    }
    sz_pdl_wait();
    sz_pdl_trigger();
    // which of the two slots of the exchange buffers this round writes (read once, early: it is a load from L2)
    const int slot = y_fix && push.world > 0 ? (int)(__ldcg(&((const SzEpHeader*)push.buf[push.me])->epoch) & 1ull) : 0;
    if (warp < top_k) {
        const int pair = j * top_k + warp;
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) v[q] = (float)((double)__ldcg(out + (size_t)pair * H + b * 128 + lane + 32 * q) * SZ_FIX_INV);
        sz_wht128_warp(v, lane);
#pragma unroll
        for (int q = 0; q < 4; q++) part[warp][lane + 32 * q] = (v[q] * SZ_RSQRT128) * sv[q];
    } else if (warp == top_k && has_shared) {
        float v[4];
        if (so_f32) {
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = __ldcg(so_f32 + (size_t)j * H + b * 128 + lane + 32 * q);
        } else {
            const int pair = m * top_k + j;
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = (float)((double)__ldcg(out + (size_t)pair * H + b * 128 + lane + 32 * q) * SZ_FIX_INV);
            sz_wht128_warp(v, lane);
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = (v[q] * SZ_RSQRT128) * sv[q];
        }
#pragma unroll
        for (int q = 0; q < 4; q++) part[top_k][lane + 32 * q] = sg * v[q];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int i = lane + 32 * e;
            if (y_fix) {  // every term in 64-bit fixed point: the sum over ranks is then exact
                long long f = 0;
                for (int t = 0; t < top_k; t++)
                    if (local[t]) f += __double2ll_rn(rws[t] * (double)part[t][i] * 1099511627776.0);
                if (has_shared) f += __double2ll_rn((double)part[top_k][i] * 1099511627776.0);
                if (push.world > 0) {
                    for (int r = 0; r < push.world; r++)
                        sz_ep_slot(push.buf[r], push.world, push.row_elems, slot, push.me)[(size_t)j * H + b * 128 + i] = f;
                } else {
                    y_fix[(size_t)j * H + b * 128 + i] = f;
                }
            } else {
                double a = 0.0;
                for (int t = 0; t < top_k; t++) a += rws[t] * (double)part[t][i];
                if (has_shared) a += (double)part[top_k][i];
                y[(size_t)j * H + b * 128 + i] = (float)a;
            }
        }
        if (y_fix && push.world > 0) {  // the block's stores are out: make them visible system-wide, then announce them to every rank
            __threadfence_system();
            __syncwarp();
            if (lane < push.world) atomicAdd_system(sz_ep_arrive(push.buf[lane], push.me), 1ull);
        }
    }
}
