// Many-row dense projections on the 5th-generation tensor cores (tcgen05 + TMEM): Y[token][row] = sum_k W[row][k] * X[token][k].
//
// This is the prompt / batched form of a dense projection, the one place of the engine where the work is a contraction and not a
// stream: with 64..256 token rows a Q8_0 weight is used a few hundred times once it is decoded.  It replaces the reference's
// tensor-core family for a long prompt's projections, kernels/matvec.cu:758-1260 (`mma_core`, `mma_cols_<type>`, `mma_cols64_<type>`:
// mma.sync m16n8k16, 64 weight rows x 32 or 64 tokens a block), launched by crates/shadowzero-cuda/src/session.rs:7276, and keeps
// its arithmetic: a weight is decoded as the reference decodes it (the float d * q) and rounded to f16, the input is rounded to
// f16, products accumulate in f32; the order of the sum is the tensor core's.  The reference calls this mode inexact and uses it
// for prompts only; so does this build (the verify step's projections stay on the bit-stable kernels).
//
// Shape of the kernel.  A block owns 128 weight rows (the M side of the instruction) and one tile of up to 256 tokens (the N side);
// the accumulator D[128 rows][NT tokens] lives in tensor memory (NT columns of 128 lanes), so no register holds a partial sum until
// the end.  K advances in steps of 64:
//   warp 0      the copy warp.  Raw Q8_0 bytes of the block's 128 rows arrive 256 columns at a time (272 bytes a row: a multiple of
//               16, which the 68 bytes of one 64-column step are not) as ONE tiled TMA copy (cp.async.bulk.tensor.2d over the
//               matrix seen as [rows][row bytes / 2] 16-bit words, box 136 x 128; 128 separate 272-byte bulk copies a piece kept
//               the copy engine, not the tensor core, as the bound), double-buffered; the token tile of a step, already in f16 and
//               in the instruction's own shared-memory order (written once by sz_x16_pack_kernel), is one bulk copy.
//   warps 1..8  decode: two threads a weight row turn a step's 2 blocks a row into f16 and store them in the canonical K-major
//               no-swizzle order (8 rows x 16 bytes core matrices), then fence.proxy.async and arrive.
//   warp 9      one thread issues the step's 4 tcgen05.mma (K = 16 each) from shared-memory descriptors and commits them to the
//               stage's "empty" barrier, which frees the stage for the decoders and the copy warp.
// After the last step warps 1..8 read the accumulator with tcgen05.ld (lane = weight row, column = token) and write Y: for one
// token, the 32 lanes of a warp write 32 consecutive rows.
// Every wait is bounded; a wait that runs out records where in the error word, and the block still frees its tensor memory.
#include <cuda.h>   // CUtensorMap and its enums; the encoder's entry point is asked of the runtime, nothing links against the driver
#include "sz_common.cuh"
#include "sz_formats.cuh"

namespace {

constexpr int MC_BM = 128;        // weight rows a block
constexpr int MC_KT = 64;         // columns a step
constexpr int MC_SS = 256;        // columns a raw copy
constexpr int MC_RAW_ROW = 272;   // bytes of a row's 8 Q8_0 blocks
constexpr int MC_STAGES = 3;
constexpr int MC_NT_MAX = 256;    // tokens a tile
constexpr int MC_THREADS = 320;   // copy warp + 8 decode warps + issue warp
constexpr int MC_A_BYTES = MC_BM * MC_KT * 2;
constexpr int MC_RAW_BYTES = MC_BM * MC_RAW_ROW;
constexpr u32 MC_WAIT = 4000000u; // polls before a wait gives up

struct McSmem {
    u64 full[MC_STAGES], empty[MC_STAGES], raw_full[2], raw_empty[2], acc_full;
    u32 tmem_base, failed;
};

__device__ __forceinline__ void mc_arrive(u64* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sz_smem_addr(bar)) : "memory"); }
__device__ __forceinline__ void mc_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mc_tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mc_tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: 8 rows x 16 bytes core matrices; `lbo` = bytes between the two core
// matrices an instruction reads along K, `sbo` = bytes between 8-row groups.  Bits: address >> 4 at 0, lbo >> 4 at 16, sbo >> 4 at
// 32, descriptor version 1 at 46, layout type 0 (none) at 61.
__device__ __forceinline__ u64 mc_desc(u32 smem_addr, u32 lbo, u32 sbo) {
    return (u64)((smem_addr & 0x3ffffu) >> 4) | ((u64)(lbo >> 4) << 16) | ((u64)(sbo >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor, kind::f16: D = f32 (bit 4), A = B = f16 (0), both K-major (0), N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ u32 mc_idesc(int n) { return (1u << 4) | ((u32)(n >> 3) << 17) | ((u32)(MC_BM >> 4) << 24); }

__device__ __forceinline__ void mc_mma(u32 d_tmem, u64 a_desc, u64 b_desc, u32 idesc, u32 accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mc_commit(u64* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sz_smem_addr(bar)) : "memory");
}

// Block KB (0..7) of a row's 272 raw bytes -> 32 f16 weights, stored as the 4 chunks of 8 the block covers (chunk stride 16 * 128
// bytes).  The block starts 34 * KB bytes into the row: not a multiple of 16, so three aligned 16-byte loads cover it and the
// bytes are brought into place by funnel shifts whose amounts are known at compile time.  A weight is d * q rounded once to f16;
// d is f16 and q an integer below 128, so the f16 product (one rounding of the exact product) is that same value.  q as f16: the
// byte with its sign bit flipped is q + 128, placed under exponent 0x64 it reads 1024 + q + 128, and 1152 is subtracted.
template <int KB>
__device__ __forceinline__ void mc_decode_block(const u8* __restrict__ rowp, u8* __restrict__ dst) {
    constexpr int OFF = KB * 34, BASE = OFF & ~15, SH = OFF & 15;
    const uint4 v0 = *(const uint4*)(rowp + BASE), v1 = *(const uint4*)(rowp + BASE + 16), v2 = *(const uint4*)(rowp + BASE + 32);
    const u32 W[12] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w};
    constexpr int DW = SH / 4, DS = (SH % 4) * 8;
    const u32 dbits = (W[DW] >> DS) & 0xffffu;
    const u32 d2 = dbits | (dbits << 16);
    const __half2 dh = *(const __half2*)&d2;
    const u32 bias = 0x64806480u;   // 1152, twice
    const __half2 bh = *(const __half2*)&bias;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        u32 o[4];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int b = SH + 2 + 4 * (2 * c + i);                       // first byte of this word of four q
            const u32 q4 = (b % 4 ? __funnelshift_r(W[b / 4], W[b / 4 + 1], (b % 4) * 8) : W[b / 4]) ^ 0x80808080u;
            const u32 lo = __byte_perm(q4, 0x64646464u, 0x4140), hi = __byte_perm(q4, 0x64646464u, 0x4342);   // {q0, q1}, {q2, q3} as 1024 + q + 128
            const __half2 w0 = __hmul2(dh, __hsub2(*(const __half2*)&lo, bh)), w1 = __hmul2(dh, __hsub2(*(const __half2*)&hi, bh));
            o[2 * i] = *(const u32*)&w0; o[2 * i + 1] = *(const u32*)&w1;
        }
        *(uint4*)(dst + c * 16 * 128) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// The token rows as f16 in the order the instruction reads them from shared memory, so that a step's tile is one contiguous copy:
// out[tile][step][chunk c of 8 columns][token t][8 halves]; tokens past m are zero.  One thread a 16-byte unit.
__global__ void __launch_bounds__(256) sz_x16_pack_kernel(const float* __restrict__ x, long long xs, int m, int cols, int nt, uint4* __restrict__ out) {
    const int steps = cols / MC_KT;
    const long long units = (long long)((m + nt - 1) / nt) * steps * 8 * nt;
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(u % nt);
        long long r = u / nt;
        const int c = (int)(r % 8); r /= 8;
        const int ks = (int)(r % steps);
        const int tile = (int)(r / steps);
        const int tok = tile * nt + t;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < m) {
            const float4* p = (const float4*)(x + (long long)tok * xs + ks * MC_KT + c * 8);
            const float4 a = __ldg(p), b = __ldg(p + 1);
            __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w), h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
            v = make_uint4(*(u32*)&h0, *(u32*)&h1, *(u32*)&h2, *(u32*)&h3);
        }
        out[u] = v;
    }
}

__global__ void __launch_bounds__(MC_THREADS, 1)
sz_mma_cols_q8_kernel(const __grid_constant__ CUtensorMap wmap, const uint4* __restrict__ x16, float* __restrict__ y, long long ys, int rows, int cols,
                      int m, int nt, u32* __restrict__ err) {
    extern __shared__ __align__(128) u8 smem[];
    u8* raw = smem;                                   // [2][128 rows][272]
    u8* sa = raw + 2 * MC_RAW_BYTES;                  // [stages][16 chunks][16 row groups][128]
    u8* sb = sa + MC_STAGES * MC_A_BYTES;             // [stages][8 chunks][nt / 8 token groups][128]
    const int b_bytes = nt * MC_KT * 2;
    McSmem* S = (McSmem*)(sb + MC_STAGES * b_bytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * MC_BM, tile = blockIdx.y;
    const int valid = rows - row0 < MC_BM ? rows - row0 : MC_BM;
    const int steps = cols / MC_KT;

    if (threadIdx.x == 0) {
        for (int i = 0; i < MC_STAGES; i++) { sz_mbar_init(&S->full[i], 256 + 1); sz_mbar_init(&S->empty[i], 1); }
        for (int i = 0; i < 2; i++) { sz_mbar_init(&S->raw_full[i], 1); sz_mbar_init(&S->raw_empty[i], 256); }
        sz_mbar_init(&S->acc_full, 1);
        S->failed = 0;
        sz_mbar_fence_init();
    }
    if (warp == 0) {   // tensor memory for the accumulator: 256 columns (a power of two >= nt), the whole warp asks
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sz_smem_addr(&S->tmem_base)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    mc_tc_fence_before();
    __syncthreads();
    mc_tc_fence_after();
    const u32 tmem = S->tmem_base;
    int failed = 0;

    if (warp == 0) {
        // ---- copies: raw weight bytes one 256-column piece ahead of the decoders, token tiles as stages come free
        const int pieces = steps / 4;
        auto issue_raw = [&](int ss) {   // x = 136 * ss words = 272 * ss bytes: a multiple of 16; rows past the matrix arrive as zeros
            const int rb = ss & 1;
            if (lane == 0) {
                sz_mbar_expect_tx(&S->raw_full[rb], (u32)MC_RAW_BYTES);
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                                 sz_smem_addr(raw + rb * MC_RAW_BYTES)),
                             "l"(&wmap), "r"(ss * (MC_RAW_ROW / 2)), "r"(row0), "r"(sz_smem_addr(&S->raw_full[rb]))
                             : "memory");
            }
        };
        issue_raw(0);
        for (int ks = 0; ks < steps && !failed; ks++) {
            const int st = ks % MC_STAGES;
            if (ks % 4 == 0 && ks / 4 + 1 < pieces) {
                const int ss = ks / 4 + 1;
                if (ss >= 2 && !sz_mbar_wait(&S->raw_empty[ss & 1], ((ss / 2) - 1) & 1, MC_WAIT)) { failed = 2; break; }
                issue_raw(ss);
            }
            if (ks >= MC_STAGES && !sz_mbar_wait(&S->empty[st], ((ks / MC_STAGES) - 1) & 1, MC_WAIT)) { failed = 1; break; }
            if (lane == 0) {
                sz_mbar_expect_tx(&S->full[st], (u32)b_bytes);
                sz_bulk_g2s(sb + st * b_bytes, (const u8*)x16 + ((size_t)tile * steps + ks) * b_bytes, (u32)b_bytes, &S->full[st]);
            }
        }
    } else if (warp <= 8) {
        // ---- decode: thread d takes weight row d % 128 and block d / 128 of the step (a warp: 32 consecutive rows of one block
        // index, so its 16-byte stores fill 512 consecutive bytes and its block index is known when the code is compiled)
        const int d = threadIdx.x - 32, r = d & 127, half = d >> 7;
        for (int ks0 = 0; ks0 < steps && !failed; ks0 += 4) {
            const int ss = ks0 / 4, rb = ss & 1;
            if (!sz_mbar_wait(&S->raw_full[rb], (ss / 2) & 1, MC_WAIT)) { failed = 4; break; }
            const u8* rowp = raw + rb * MC_RAW_BYTES + r * MC_RAW_ROW;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int ks = ks0 + j, st = ks % MC_STAGES;
                if (ks >= MC_STAGES && !sz_mbar_wait(&S->empty[st], ((ks / MC_STAGES) - 1) & 1, MC_WAIT)) { failed = 3; break; }
                u8* dst = sa + st * MC_A_BYTES + ((half * 4) * 16 + (r >> 3)) * 128 + (r & 7) * 16;
                if (r < valid) {
                    switch (2 * j + half) {   // j is an unrolled loop's counter and half is the same for a whole warp
                        case 0: mc_decode_block<0>(rowp, dst); break;
                        case 1: mc_decode_block<1>(rowp, dst); break;
                        case 2: mc_decode_block<2>(rowp, dst); break;
                        case 3: mc_decode_block<3>(rowp, dst); break;
                        case 4: mc_decode_block<4>(rowp, dst); break;
                        case 5: mc_decode_block<5>(rowp, dst); break;
                        case 6: mc_decode_block<6>(rowp, dst); break;
                        default: mc_decode_block<7>(rowp, dst); break;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 4; c++) *(uint4*)(dst + c * 16 * 128) = make_uint4(0, 0, 0, 0);
                }
                mc_fence_async();                 // the tensor core reads shared memory through the async proxy
                mc_arrive(&S->full[st]);
            }
            if (failed) break;
            mc_arrive(&S->raw_empty[rb]);
        }
    } else {
        // ---- issue
        const u32 idesc = mc_idesc(nt);
        for (int ks = 0; ks < steps && !failed; ks++) {
            const int st = ks % MC_STAGES;
            if (!sz_mbar_wait(&S->full[st], (ks / MC_STAGES) & 1, MC_WAIT)) { failed = 5; break; }
            mc_tc_fence_after();
            if (lane == 0) {
                const u32 a0 = sz_smem_addr(sa + st * MC_A_BYTES), b0 = sz_smem_addr(sb + st * b_bytes);
#pragma unroll
                for (int k = 0; k < MC_KT / 16; k++)
                    mc_mma(tmem, mc_desc(a0 + k * 2 * (MC_BM * 16), MC_BM * 16, 128), mc_desc(b0 + k * 2 * (nt * 16), (u32)nt * 16, 128), idesc, (ks | k) ? 1u : 0u);
                mc_commit(&S->empty[st]);
            }
            __syncwarp();
        }
        if (lane == 0) mc_commit(&S->acc_full);   // arrives when every instruction above has finished (also after a failure: nothing pending then)
    }
    if (failed) atomicMax(&S->failed, (u32)failed);

    // ---- the accumulator to Y: warps 1..8; a warp reads the 32 lanes of its quadrant (warp % 4), the two warps of a quadrant take
    // half of the columns each
    if (warp >= 1 && warp <= 8 && !failed) {
        if (!sz_mbar_wait(&S->acc_full, 0, MC_WAIT)) {
            atomicMax(&S->failed, 6u);
        } else {
            mc_tc_fence_after();
            const int q = warp & 3, hcol = (warp - 1) >> 2;
            const int c0 = hcol * (nt / 2), c1 = c0 + nt / 2;
            const int row = row0 + q * 32 + lane;
            for (int c = c0; c < c1; c += 8) {
                u32 v[8];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                             : "r"(tmem + ((u32)(q * 32) << 16) + (u32)c));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int tok = tile * nt + c + i;
                    if (tok < m && row < rows) y[(long long)tok * ys + row] = __uint_as_float(v[i]);
                }
            }
        }
    }
    mc_tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        mc_tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
    if (threadIdx.x == 0 && S->failed) atomicMax(err, S->failed);
}

typedef CUresult (*McEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
McEncodeTiled mc_encoder() {
    static McEncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (McEncodeTiled)p;
    }
    return fn;
}

int mc_nt(int m) {
    const int r = (m + 15) & ~15;
    return r < MC_NT_MAX ? r : MC_NT_MAX;
}

}  // namespace

// Bytes of scratch for up to m token rows of `cols` inputs: an error word and the f16 copy of the rows.
extern "C" int sz_mma_cols_scratch_bytes(int cols, int m, int64_t* bytes) {
    if (!bytes || m < 1 || cols < MC_SS || cols % MC_SS) return sz_fail(SZ_E_ARG, "sz_mma_cols_scratch_bytes: m >= 1 and cols a multiple of %d", MC_SS);
    const int nt = mc_nt(m);
    *bytes = 256 + (int64_t)((m + nt - 1) / nt) * nt * cols * 2;
    return SZ_OK;
}

// y[t * ys + r] = sum_k w[r][k] * x[t * xs + k] for t < m, r < w->rows (strides in floats; x rows 16-byte aligned).  w: Q8_0.
extern "C" int sz_mma_cols(const sz_tensor* w, uint64_t x, int64_t xs, uint64_t y, int64_t ys, int m, uint64_t scratch, int64_t scratch_bytes,
                           uint64_t stream) {
    if (!w || !w->data || !x || !y || !scratch) return sz_fail(SZ_E_ARG, "sz_mma_cols: null argument");
    if (w->type != SZ_TYPE_Q8_0) return sz_fail(SZ_E_TYPE, "sz_mma_cols: Q8_0 weights (type %d given)", w->type);
    int64_t need = 0;
    int rc = sz_mma_cols_scratch_bytes((int)w->cols, m, &need);
    if (rc) return rc;
    if (scratch_bytes < need) return sz_fail(SZ_E_SCRATCH, "sz_mma_cols: %lld bytes of scratch given, %lld needed", (long long)scratch_bytes, (long long)need);
    if ((x & 15) || (xs & 3) || (w->data & 15) || (scratch & 255)) return sz_fail(SZ_E_ARG, "sz_mma_cols: x rows and the weights 16-byte aligned, scratch 256-byte aligned");
    if (w->rows < 1) return sz_fail(SZ_E_ARG, "sz_mma_cols: no rows");
    cudaStream_t st = (cudaStream_t)stream;
    const int nt = mc_nt(m), tiles = (m + nt - 1) / nt, cols = (int)w->cols, rows = (int)w->rows;
    u32* err = (u32*)scratch;
    uint4* x16 = (uint4*)(scratch + 256);
    const size_t smem = 2 * MC_RAW_BYTES + MC_STAGES * (MC_A_BYTES + (size_t)nt * MC_KT * 2) + sizeof(McSmem);
    static bool set = false;
    if (!set) {
        SZ_CUDA(cudaFuncSetAttribute(sz_mma_cols_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * MC_RAW_BYTES + MC_STAGES * (MC_A_BYTES + MC_NT_MAX * MC_KT * 2) + (int)sizeof(McSmem)));
        set = true;
    }
    McEncodeTiled enc = mc_encoder();
    if (!enc) return sz_fail(SZ_E_CUDA, "sz_mma_cols: the driver has no cuTensorMapEncodeTiled");
    CUtensorMap wmap;
    {   // the matrix as [rows][row bytes / 2] 16-bit words; a box is 272 bytes of 128 rows
        const cuuint64_t row_bytes = (cuuint64_t)(cols / 32) * 34;
        const cuuint64_t gdim[2] = {row_bytes / 2, (cuuint64_t)rows}, gstride[1] = {row_bytes};
        const cuuint32_t box[2] = {MC_RAW_ROW / 2, MC_BM}, es[2] = {1, 1};
        const CUresult r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*)w->data, gdim, gstride, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return sz_fail(SZ_E_CUDA, "sz_mma_cols: cuTensorMapEncodeTiled failed (%d)", (int)r);
    }
    const long long units = (long long)tiles * (cols / MC_KT) * 8 * nt;
    SZ_CUDA(sz_launch("x16_pack", sz_x16_pack_kernel, dim3((unsigned)((units + 255) / 256 < 1184 ? (units + 255) / 256 : 1184)), dim3(256), 0, st, false,
                      (const float*)x, (long long)xs, m, cols, nt, x16));
    SZ_CUDA(sz_launch("mma_cols_q8", sz_mma_cols_q8_kernel, dim3((rows + MC_BM - 1) / MC_BM, tiles), dim3(MC_THREADS), smem, st, false, wmap,
                      (const uint4*)x16, (float*)y, (long long)ys, rows, cols, m, nt, err));
    return SZ_OK;
}

// Clears (init != 0) or reads the scratch's error word; reading synchronises the stream.  0: no wait of a kernel ran out.
extern "C" int sz_mma_cols_status(uint64_t scratch, int init, int* code, uint64_t stream) {
    if (!scratch) return sz_fail(SZ_E_ARG, "sz_mma_cols_status: null scratch");
    cudaStream_t st = (cudaStream_t)stream;
    if (init) { SZ_CUDA(cudaMemsetAsync((void*)scratch, 0, 256, st)); return SZ_OK; }
    if (!code) return sz_fail(SZ_E_ARG, "sz_mma_cols_status: null code");
    u32 v = 0;
    SZ_CUDA(cudaMemcpyAsync(&v, (const void*)scratch, 4, cudaMemcpyDeviceToHost, st));
    SZ_CUDA(cudaStreamSynchronize(st));
    *code = (int)v;
    return v ? sz_fail(SZ_E_CUDA, "sz_mma_cols: a bounded wait of the kernel ran out (stage %u)", v) : SZ_OK;
}
