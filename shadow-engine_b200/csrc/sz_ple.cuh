// The per-layer embedding of one layer: a hashed n-gram memory added to the whole residual stream before that layer's first read
// (crates/shadowzero-model/src/forward.rs:1036-1074 `ple`, :1177-1198 `ple_rows`; the reference's kernels are the `ple_*` family of
// kernels/forward.cu and reads its 27 GB table from disk through a prefetch thread: here the table is resident in HBM and the rows
// are gathered on the device).
//   sz_ple_embed_kernel   the table rows the last tokens select, decoded side by side: e [m][hidden]
//   (dense launcher)      key = ple_key . e [m][streams * hidden], val = ple_value . e [m][hidden]
//   sz_ple_gate_kernel    per (stream, row): the pending residual write applied, qry = norm_query(r), key normed, the stream's gate,
//                         gv = gate * val and gvn = norm_conv(gv)
//   sz_ple_conv_kernel    r += gv + silu(depthwise causal conv over gvn: kernel conv_k, dilation ngram, taps from this pass's earlier
//                         rows or from the carried history)
//   sz_ple_commit_kernel  after acceptance: the history and the token tail as the kept rows leave them (into the other buffer; the
//                         state word that flips the DeltaNet buffers flips these)
// State: history [2][(conv_k - 1) * ngram][streams * hidden] f32, oldest row first; tail [2][8] tokens, most recent first.
#pragma once
#include "sz_common.cuh"
#include "sz_dense.cuh"

struct SzPleGeom {
    int ngram, heads_per_ngram, head_dim, conv_k, eos, table_type;
    long long multipliers[SZ_PLE_MAX_NGRAM];
    long long vocab[SZ_PLE_MAX_HEADS], offsets[SZ_PLE_MAX_HEADS];
};

// token `dist` steps before row j's own (dist = 0: its own): a row of the pass, or the committed tail
__device__ __forceinline__ int sz_ple_token(const int32_t* __restrict__ ids, const int32_t* __restrict__ tail, int j, int dist) {
    return dist <= j ? ids[j - dist] : tail[dist - j - 1];
}

// ---- grid ((ngram - 1) * heads_per_ngram, m), block 64 ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(64)
sz_ple_embed_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ tails, const int32_t* __restrict__ state, SzPleGeom g,
                    const u8* __restrict__ table, long long table_rows, int H, float* __restrict__ e) {
    __shared__ u32 grid[512];
    sz_pdl_wait();
    sz_pdl_trigger();
    for (int i = threadIdx.x; i < 512; i += 64) grid[i] = c_iq3s_grid[i];
    __syncthreads();
    const int i = blockIdx.x, j = blockIdx.y;
    const int32_t* tail = tails + (state[1] ? 8 : 0);
    const int order = 2 + i / g.heads_per_ngram;
    // tokens before the last end-of-text token count as end-of-text (and so do positions before the sequence: the tail starts as eos)
    unsigned long long mixed = 0;
    bool past_eos = false;
    for (int s = 0; s < order; s++) {
        int tk = past_eos ? g.eos : sz_ple_token(ids, tail, j, s);
        if (tk == g.eos) past_eos = true;
        const unsigned long long term = (unsigned long long)(long long)tk * (unsigned long long)g.multipliers[s];
        mixed = s == 0 ? term : (mixed ^ term);
    }
    const long long v = g.vocab[i];
    long long rem = (long long)mixed % v;
    if (rem < 0) rem += v < 0 ? -v : v;
    long long row = rem + g.offsets[i];
    row = row < 0 ? 0 : (row >= table_rows ? table_rows - 1 : row);
    const u8* src = table + (size_t)row * sz_dense_row_bytes(g.table_type, g.head_dim);
    float* dst = e + (size_t)j * H + (size_t)i * g.head_dim;
    for (int c = 4 * threadIdx.x; c < g.head_dim; c += 256) {
        float w[4], sc;
        sz_dense_w4(g.table_type, src, c, grid, w, sc);
        *(float4*)(dst + c) = make_float4(sc * w[0], sc * w[1], sc * w[2], sc * w[3]);
    }
}

// ---- grid (streams, m), block 256 -------------------------------------------------------------------------------------------------------
// r: the residual as the previous sublayer left it, WITHOUT that sublayer's own write: the write (gate g of the stream, output y) is
// applied here and stored back, so the read that follows has nothing pending.  The gate comes from the fused hyper-connection
// read's fixed-point accumulator (g_acc: row stride acc_rows, the inject sums after `rank` entries) or from a float array (g_f).
__global__ void __launch_bounds__(256)
sz_ple_gate_kernel(float* __restrict__ r, const long long* __restrict__ g_acc, int acc_rows, int rank, const float* __restrict__ g_f,
                   const float* __restrict__ y, const float* __restrict__ key, const float* __restrict__ val, const float* __restrict__ w_key,
                   const float* __restrict__ w_query, const float* __restrict__ w_conv, int H, int C, float eps, float* __restrict__ gv,
                   float* __restrict__ gvn) {
    extern __shared__ float sm[];   // [H] the stream of the row, then [H] its normed key
    __shared__ double red[8];
    sz_pdl_wait();
    sz_pdl_trigger();
    const int s = blockIdx.x, j = blockIdx.y, t = threadIdx.x;
    float* rs = r + ((size_t)j * C + s) * H;
    float* xr = sm;
    float* xk = sm + H;
    float gate_w = 0.0f;
    const bool pending = g_acc != nullptr || g_f != nullptr;
    if (g_acc) gate_w = 2.0f * sz_sigmoid((float)((double)__ldcg(g_acc + (size_t)j * acc_rows + rank + s) * (1.0 / 1099511627776.0)) / (float)C);
    else if (g_f) gate_w = g_f[(size_t)j * C + s];
    double sr = 0.0, sk = 0.0;
    for (int i = t; i < H; i += 256) {
        float v = rs[i];
        if (pending) { v += gate_w * y[(size_t)j * H + i]; rs[i] = v; }
        xr[i] = v;
        const float k = key[((size_t)j * C + s) * H + i];
        xk[i] = k;
        sr += (double)v * (double)v;
        sk += (double)k * (double)k;
    }
    sr = sz_block_sum(sr, red);
    sk = sz_block_sum(sk, red);
    const double rr = sz_rsqrt64(sr / (double)H + (double)eps), rk = sz_rsqrt64(sk / (double)H + (double)eps);
    double dot = 0.0;
    for (int i = t; i < H; i += 256) {
        const float q = (float)((double)xr[i] * rr) * w_query[(size_t)s * H + i];
        const float k = (float)((double)xk[i] * rk) * w_key[(size_t)s * H + i];
        dot += (double)k * (double)q;
    }
    dot = sz_block_sum(dot, red) / sqrt((double)H);
    const double ad = fabs(dot) > 1e-6 ? fabs(dot) : 1e-6;
    const double gg = sqrt(ad) * (signbit(dot) ? -1.0 : 1.0);
    const float sg = sz_sigmoid((float)gg);
    double sv = 0.0;
    for (int i = t; i < H; i += 256) {
        const float v = sg * val[(size_t)j * H + i];
        xr[i] = v;
        sv += (double)v * (double)v;
    }
    sv = sz_block_sum(sv, red);
    const double rv = sz_rsqrt64(sv / (double)H + (double)eps);
    for (int i = t; i < H; i += 256) {
        const size_t o = ((size_t)j * C + s) * H + i;
        gv[o] = xr[i];
        gvn[o] = (float)((double)xr[i] * rv) * w_conv[(size_t)s * H + i];
    }
}

// ---- grid (ceil(streams * hidden / 256), m), block 256 ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
sz_ple_conv_kernel(float* __restrict__ r, const float* __restrict__ gv, const float* __restrict__ gvn, const float* __restrict__ hist0,
                   const float* __restrict__ hist1, const int32_t* __restrict__ state, const float* __restrict__ w, int CH, int k, int dil) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int i = blockIdx.x * 256 + threadIdx.x, j = blockIdx.y;
    if (i >= CH) return;
    const float* hist = state[1] ? hist1 : hist0;
    const int hist_len = (k - 1) * dil;
    double acc = (double)w[(size_t)i * k + (k - 1)] * (double)gvn[(size_t)j * CH + i];
    for (int t = 0; t + 1 < k; t++) {
        const int back = (k - 1 - t) * dil;
        const float x = back <= j ? gvn[(size_t)(j - back) * CH + i] : hist[(size_t)(hist_len - (back - j)) * CH + i];
        acc += (double)w[(size_t)i * k + t] * (double)x;
    }
    r[(size_t)j * CH + i] += gv[(size_t)j * CH + i] + sz_silu((float)acc);
}

// ---- grid ((conv_k - 1) * ngram), block 256; res[0] = rows kept (nothing is written when it is 0) -----------------------------------
__global__ void __launch_bounds__(256)
sz_ple_commit_kernel(const float* __restrict__ gvn, float* __restrict__ hist0, float* __restrict__ hist1, int32_t* __restrict__ tails,
                     const int32_t* __restrict__ ids, const int32_t* __restrict__ state, const int32_t* __restrict__ res, int CH, int hist_len) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int keep = res[0];
    if (keep <= 0) return;
    const int cur = state[1];
    const float* src_h = cur ? hist1 : hist0;
    float* dst_h = cur ? hist0 : hist1;
    const int t = blockIdx.x;                       // row of the new history, oldest first
    const int tau = keep - hist_len + t;            // index into the kept rows, negative: into the old history
    const float* src = tau >= 0 ? gvn + (size_t)tau * CH : src_h + (size_t)(hist_len + tau) * CH;
    for (int i = threadIdx.x; i < CH; i += 256) dst_h[(size_t)t * CH + i] = src[i];
    if (t == 0 && threadIdx.x < 8) {
        const int32_t* old = tails + (cur ? 8 : 0);
        int32_t* nw = tails + (cur ? 0 : 8);
        const int q = threadIdx.x;                  // the token q + 1 steps before the next pass's first row
        nw[q] = q < keep ? ids[keep - 1 - q] : old[q - keep];
    }
}
