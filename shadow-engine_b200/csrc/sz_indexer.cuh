// The sparse indexer of the gated-attention layers (crates/shadowzero-model/src/forward.rs:930-976; the reference's kernels:
// kernels/forward.cu:2461-2508, 2964-3117).  Positions are grouped in blocks of `ratio`; every COMPLETE block has a pooled key
// (mean of its positions' raw indexer keys, RMS-normed, rotated at the block's first position); a query scores every complete
// block (sum over the indexer heads of relu(q_h . key), over sqrt(width)) and attends to the best budget / ratio blocks plus the
// incomplete tail.  With no more complete blocks than that it attends to everything.
//
// A verify pass has up to 8 queries (rows) with selections of their own.  Each row's attention runs over its own list (the grouped
// attention kernel takes one row a block in this form): what a row computes then depends on nothing but the row, which is what
// makes a pass of several rows equal, bit for bit, to the same rows read one at a time (tests/reference.rs:258-290 asks for that).
//   sz_idx_prep_kernel    indexer queries (norm, rotation), raw keys into their cache slots, pooled keys of the blocks this pass completes
//   sz_idx_score_kernel   block scores of every row: a warp a block, the dot products in f64 (one fixed order, a butterfly over the lanes)
//   sz_idx_select_kernel  per row the `keep` best blocks (score descending, block ascending among equals) by a radix select, then the
//                         row's ascending list of position groups
// Caches: raw keys [position][width] f32; pooled keys [block][width] f32.  Nothing is rolled back on a rejection: a slot is
// rewritten when its position is read again, and a block counts only while the committed length covers it.
#pragma once
#include "sz_common.cuh"

#define SZ_IDX_MAX_DIM 256

struct SzIdxGeom {
    int heads, dim, ratio, keep;   // keep = budget / ratio blocks
    int ctx_blocks;                // blocks the caches have room for
    int words;                     // 32-bit words of a row's block set
};

// RMS norm (weights w), rotation at position rpos, store: the tail of every indexer vector (128 threads; tmp holds the vector).
__device__ __forceinline__ void sz_idx_finish(float* tmp, double* red, int id, const float* __restrict__ w, float eps, int rpos, int rope_dims,
                                              const double* __restrict__ rope_den, float* __restrict__ dst) {
    __syncthreads();
    double ss = 0.0;
    for (int i = threadIdx.x; i < id; i += 128) ss += (double)tmp[i] * (double)tmp[i];
    ss = sz_block_sum(ss, red);
    const double rr = sz_rsqrt64(ss / (double)id + (double)eps);
    __syncthreads();
    for (int i = threadIdx.x; i < id; i += 128) tmp[i] = (float)((double)tmp[i] * rr) * w[i];
    __syncthreads();
    const int half = rope_dims / 2;
    for (int i = threadIdx.x; i < half; i += 128) {   // forward.rs:290-299, as the attention front end rotates q and k
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
    for (int i = threadIdx.x; i < id; i += 128) dst[i] = tmp[i];
}

// ---- grid (heads + 2, m), block 128 ------------------------------------------------------------------------------------------------
// b < heads: query head b of row j.  b == heads: the row's raw key into its slot.  b == heads + 1: the block this row completes.
__global__ void __launch_bounds__(128)
sz_idx_prep_kernel(const float* __restrict__ iq, const float* __restrict__ ik, const float* __restrict__ wq, const float* __restrict__ wk, SzIdxGeom g,
                   float eps, const int32_t* __restrict__ state, int rope_dims, const double* __restrict__ rope_den, float* __restrict__ raw,
                   float* __restrict__ blocks, float* __restrict__ qn) {
    __shared__ float tmp[SZ_IDX_MAX_DIM];
    __shared__ double red[4];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int b = blockIdx.x, j = blockIdx.y, id = g.dim;
    const int pos0 = state[0], pos = pos0 + j;
    if (b == g.heads) {
        for (int i = threadIdx.x; i < id; i += 128) raw[(size_t)pos * id + i] = ik[(size_t)j * id + i];
        return;
    }
    const float* w;
    int rpos;
    float* dst;
    if (b < g.heads) {
        const float* x = iq + ((size_t)j * g.heads + b) * id;
        for (int i = threadIdx.x; i < id; i += 128) tmp[i] = x[i];
        w = wq; rpos = pos; dst = qn + ((size_t)j * g.heads + b) * id;
    } else {
        if ((pos + 1) % g.ratio != 0) return;
        const int blk = (pos + 1) / g.ratio - 1;
        // mean of the block's raw keys, added in position order; a position of this pass comes from the pass's rows (its slot is
        // written by another block of this launch), an earlier one from the cache
        for (int i = threadIdx.x; i < id; i += 128) {
            float acc = 0.0f;
            for (int r = 0; r < g.ratio; r++) {
                const int p = blk * g.ratio + r;
                acc += p >= pos0 ? ik[(size_t)(p - pos0) * id + i] : raw[(size_t)p * id + i];
            }
            tmp[i] = acc / (float)g.ratio;
        }
        w = wk; rpos = blk * g.ratio; dst = blocks + (size_t)blk * id;
    }
    sz_idx_finish(tmp, red, id, w, eps, rpos, rope_dims, rope_den, dst);
}

// ---- grid (any), block 256: scores[j][b] for every row j whose complete blocks include b ------------------------------------------
// A warp takes a block: its lanes hold the pooled key (dimension lane, lane + 32, ...), and for every (row, head) the lanes' f64
// partial products meet in a butterfly, so the sum has one fixed order whatever the pass looks like.  (One thread a block with the
// dot product as one serial f64 chain was 184 us a launch at 6,144 blocks x 4 rows; the f64 pipe wants parallel chains.)  The f64
// sum differs from the reference's serial one far below the f32 it is rounded to.
__global__ void __launch_bounds__(256)
sz_idx_score_kernel(const float* __restrict__ qn, const float* __restrict__ blocks, SzIdxGeom g, int m, const int32_t* __restrict__ state,
                    float* __restrict__ scores) {
    extern __shared__ float sq[];   // [m][heads][dim]
    sz_pdl_wait();
    sz_pdl_trigger();
    const int id = g.dim, nq = m * g.heads * id;
    for (int i = threadIdx.x; i < nq; i += 256) sq[i] = qn[i];
    __syncthreads();
    const int pos0 = state[0];
    const int lane = threadIdx.x & 31;
    const int nb_last = (pos0 + m) / g.ratio;
    const float norm = sqrtf((float)id);
    constexpr int MAXT = SZ_IDX_MAX_DIM / 32;
    const int nt = (id + 31) / 32;
    for (int b = blockIdx.x * 8 + (threadIdx.x >> 5); b < nb_last; b += gridDim.x * 8) {
        float kb[MAXT];
#pragma unroll
        for (int t = 0; t < MAXT; t++) kb[t] = t < nt && lane + 32 * t < id ? __ldg(blocks + (size_t)b * id + lane + 32 * t) : 0.0f;
        for (int j = 0; j < m; j++) {
            const int nb = (pos0 + j + 1) / g.ratio;
            if (b >= nb || nb <= g.keep) continue;     // not complete for this row yet, or the row attends to everything
            float sc = 0.0f;
            for (int h = 0; h < g.heads; h++) {
                const float* q = sq + ((size_t)j * g.heads + h) * id;
                double dot = 0.0;
#pragma unroll
                for (int t = 0; t < MAXT; t++)
                    if (t < nt && lane + 32 * t < id) dot = fma((double)q[lane + 32 * t], (double)kb[t], dot);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                const float f = (float)dot;
                sc += f > 0.0f ? f : 0.0f;
            }
            if (lane == 0) scores[(size_t)j * g.ctx_blocks + b] = sc / norm;
        }
    }
}

// ---- grid (m), block 1024 ------------------------------------------------------------------------------------------------------------
// Row j: bit b of sel[j] = the row attends to complete block b; list[j] = the groups of `ratio` positions it attends to, ascending:
// those blocks and, when the row's position leaves an incomplete block, that one (the attention kernel cuts it at the row's own
// position); count[j] = how many.  A row's list depends on nothing but the row, so a pass of several rows attends exactly as the same
// rows read one at a time.  trace, when not null, receives a copy of sel (one [8][words] array per attention layer).
__global__ void __launch_bounds__(1024)
sz_idx_select_kernel(const float* __restrict__ scores, SzIdxGeom g, int m, const int32_t* __restrict__ state, u32* __restrict__ sel, int32_t* __restrict__ list,
                     int32_t* __restrict__ count, u32* __restrict__ trace) {
    extern __shared__ u32 sbits[];          // [words]
    __shared__ u32 hist[256];
    __shared__ u32 wsum[32];
    __shared__ u32 s_prefix, s_remaining;
    sz_pdl_wait();
    sz_pdl_trigger();
    const int j = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos0 = state[0];
    const int n = pos0 + j + 1, nb = n / g.ratio;
    for (int i = tid; i < g.words; i += 1024) sbits[i] = 0;
    __syncthreads();
    if (nb <= g.keep) {
        for (int i = tid; i < g.words; i += 1024) {
            const int lo = i * 32;
            sbits[i] = nb >= lo + 32 ? 0xffffffffu : (nb > lo ? (1u << (nb - lo)) - 1u : 0u);
        }
    } else {
        const u32* key = (const u32*)(scores + (size_t)j * g.ctx_blocks);   // scores are >= 0: their bit patterns order as they do
        if (tid == 0) { s_prefix = 0; s_remaining = (u32)g.keep; }
        u32 kmask = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) hist[tid] = 0;
            __syncthreads();
            const u32 prefix = s_prefix;
            for (int b = tid; b < nb; b += 1024) {
                const u32 k = key[b];
                if ((k & kmask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (warp == 0) {   // the digit where the count from the top reaches what is still wanted: lane l owns digits 255 - 8 l .. 248 - 8 l
                const u32 need = s_remaining;
                u32 own = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) own += hist[255 - 8 * lane - i];
                u32 incl = own;
                for (int o = 1; o < 32; o <<= 1) { const u32 v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
                const u32 hit = __ballot_sync(0xffffffffu, incl >= need);
                const int owner = hit ? __ffs((int)hit) - 1 : 31;   // (need <= the count of matching keys, so some lane reaches it)
                if (lane == owner) {
                    u32 cum = incl - own;
                    int d = 255 - 8 * lane;
                    for (int i = 0; i < 7; i++, d--) {
                        if (cum + hist[d] >= need) break;
                        cum += hist[d];
                    }
                    s_remaining = need - cum;
                    s_prefix = prefix | ((u32)d << shift);
                }
            }
            kmask |= 255u << shift;
            __syncthreads();
        }
        const u32 T = s_prefix, want_eq = s_remaining;   // the keep-th best score, and how many blocks of exactly that score are taken
        // blocks with a score above T, and the first want_eq blocks (ascending) of score T: each thread owns a contiguous range
        const int per = (nb + 1023) / 1024;
        const int b0 = tid * per, b1 = min(nb, b0 + per);
        u32 eq = 0;
        for (int b = b0; b < b1; b++) eq += key[b] == T ? 1u : 0u;
        u32 inc = eq;   // inclusive scan over the block's threads
        for (int o = 1; o < 32; o <<= 1) { const u32 v = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += v; }
        if (lane == 31) wsum[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            u32 v = wsum[lane];
            for (int o = 1; o < 32; o <<= 1) { const u32 t = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += t; }
            wsum[lane] = v;
        }
        __syncthreads();
        u32 before = inc - eq + (warp > 0 ? wsum[warp - 1] : 0u);   // equal-score blocks below this thread's range
        for (int b = b0; b < b1; b++) {
            const u32 k = key[b];
            bool take = k > T;
            if (k == T) { take = before < want_eq; before++; }
            if (take) atomicOr(&sbits[b >> 5], 1u << (b & 31));
        }
    }
    __syncthreads();
    for (int i = tid; i < g.words; i += 1024) {
        sel[(size_t)j * g.words + i] = sbits[i];
        if (trace) trace[(size_t)j * g.words + i] = sbits[i];
    }
    // ---- the set as an ascending list: each thread owns a contiguous range of words
    const int wper = (g.words + 1023) / 1024;
    const int w0 = tid * wper, w1 = min(g.words, w0 + wper);
    u32 cnt = 0;
    for (int w = w0; w < w1; w++) cnt += (u32)__popc(sbits[w]);
    u32 inc = cnt;
    for (int o = 1; o < 32; o <<= 1) { const u32 v = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += v; }
    __syncthreads();
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        u32 v = wsum[lane];
        for (int o = 1; o < 32; o <<= 1) { const u32 t = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += t; }
        wsum[lane] = v;
    }
    __syncthreads();
    u32 at = inc - cnt + (warp > 0 ? wsum[warp - 1] : 0u);
    int32_t* out = list + (size_t)j * g.ctx_blocks;
    for (int w = w0; w < w1; w++) {
        u32 bits = sbits[w];
        while (bits) {
            const int b = __ffs((int)bits) - 1;
            bits &= bits - 1;
            out[at++] = w * 32 + b;
        }
    }
    if (tid == 1023) {
        if (n % g.ratio) out[at++] = nb;    // the incomplete block the row's own position is in
        count[j] = (int32_t)at;
    }
}

// ---- a synthetic history (benchmarks and long-context tests): raw keys from an integer hash of (position, element, layer, seed), as
// the CPU restatement fills them, then the pooled key of every complete block.  grid (blocks, attention layers).
__global__ void __launch_bounds__(128)
sz_idx_fill_kernel(float* __restrict__ raw, long long layer_floats, int len, int id, u32 seed) {
    const int layer = blockIdx.y;
    float* base = raw + (size_t)layer * layer_floats;
    for (long long pos = blockIdx.x; pos < len; pos += gridDim.x)
        for (int i = threadIdx.x; i < id; i += 128) {
            u32 x = (u32)((unsigned long long)pos * 2654435761u) ^ (u32)(i * 40503u) ^ seed ^ (u32)(layer * 97u);
            x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
            base[(size_t)pos * id + i] = ((float)(x % 2001u) - 1000.0f) * 1e-3f;
        }
}
// grid (complete blocks), block 128: the pooled key of block blockIdx.x of one layer from the raw keys in the cache
__global__ void __launch_bounds__(128)
sz_idx_rebuild_kernel(const float* __restrict__ raw, const float* __restrict__ wk, int id, int ratio, float eps, int rope_dims,
                      const double* __restrict__ rope_den, float* __restrict__ blocks) {
    __shared__ float tmp[SZ_IDX_MAX_DIM];
    __shared__ double red[4];
    const int blk = blockIdx.x;
    for (int i = threadIdx.x; i < id; i += 128) {
        float acc = 0.0f;
        for (int r = 0; r < ratio; r++) acc += raw[(size_t)(blk * ratio + r) * id + i];
        tmp[i] = acc / (float)ratio;
    }
    sz_idx_finish(tmp, red, id, wk, eps, blk * ratio, rope_dims, rope_den, blocks + (size_t)blk * id);
}
