/* CPU oracle, part 3: the lm_head's 2-bit screening proxy (Q2_P) and the block selection that follows it.
 *
 * TEST INFRASTRUCTURE ONLY (see sz_oracle.h).  The reference has no CPU form of this stage: it exists as GPU kernels
 * only (kernels/exl3.cu:915-987, kernels/forward.cu:4367-4632) and is never used by the scalar `--exact` path.  What
 * follows restates the arithmetic of those kernels operation by operation (f32, the same order of the fused
 * multiply-adds), so that every intermediate of the CUDA library (proxy codes and scales, quantised inputs, block
 * maxima, the selected block list) can be compared bit for bit.  The exact logits of the selected blocks are the
 * ordinary EXL3 matvec (szo_matvec).
 *
 * Pins (tests/test_oracle_head.py): the assertions of the reference's own test of this stage
 * (crates/shadowzero-cuda/tests/head_proxy.rs:84-236) on the blob its xorshift generator builds from the same seed.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "sz_oracle.h"

static uint16_t h_u16(const uint8_t* p, size_t off) { return (uint16_t)(p[off] | (p[off + 1] << 8)); }

/* The butterflies of kernels/exl3.cu:21-29 (h = 1, 2, .. 64, no scaling): the same sums in the same order as
 * exl3.rs:583-594 before its final multiply. */
static void wht128_raw(float* v) {
    for (int h = 1; h < 128; h *= 2)
        for (int i = 0; i < 128; i += 2 * h)
            for (int j = i; j < i + h; j++) {
                float a = v[j], b = v[j + h];
                v[j] = a + b;
                v[j + h] = a - b;
            }
}

/* kernels/exl3.cu:609-625 (exl3_rotate_rows_f32), one row: xr = H (x * suh) on every 128-block, not normalised. */
void szo_head_rotate(const uint8_t* blob, const float* x, size_t cols, float* xr) {
    for (size_t i = 0; i < cols; i++) xr[i] = x[i] * szo_f16_to_f32(h_u16(blob, 2 * i));
    for (size_t b = 0; b < cols / 128; b++) wht128_raw(xr + b * 128);
}

/* kernels/exl3.cu:915-987 (exl3_build_q2_proxy_impl).  rows = outputs (vocabulary), cols = inputs (hidden), both whole
 * 128-blocks.  w_q2: rows * cols / 4 bytes, w_sc: rows * cols / 128 f16. */
void szo_head_proxy_build(size_t rows, size_t cols, int bits, const uint8_t* blob, uint8_t* w_q2, uint16_t* w_sc) {
    const size_t n_b = cols / 128, n_ob = rows / 128, nt = rows / 16;
    const size_t osv = 2 * cols, otr = 2 * cols + 2 * rows + 4;
    const int tw = 16 * bits; /* u16 words of a tile */
    uint16_t* tile = (uint16_t*)malloc((size_t)tw * sizeof(uint16_t));
    float* wsrc = (float*)malloc(128 * 128 * sizeof(float));     /* [input within b][output within ob] */
    uint16_t* wh = (uint16_t*)malloc(128 * 128 * sizeof(uint16_t)); /* [output][input], f16 */
    float vals[256], rv[128];
    for (size_t ob = 0; ob < n_ob; ob++)
        for (size_t b = 0; b < n_b; b++) {
            for (size_t kk = 0; kk < 8; kk++)
                for (size_t tc = 0; tc < 8; tc++) {
                    const uint8_t* tb = blob + otr + ((b * 8 + kk) * nt + ob * 8 + tc) * (size_t)tw * 2;
                    for (int i = 0; i < tw; i++) tile[i] = h_u16(tb, 2 * (size_t)i);
                    szo_exl3_decode_tile_fast(tile, bits, 0, 2, vals);
                    for (int p = 0; p < 256; p++) {
                        int r, c;
                        szo_exl3_tile_pos(p, &r, &c);
                        wsrc[(kk * 16 + (size_t)r) * 128 + tc * 16 + (size_t)c] = vals[p];
                    }
                }
            for (int r_in = 0; r_in < 128; r_in++) {
                memcpy(rv, wsrc + (size_t)r_in * 128, sizeof(rv));
                wht128_raw(rv);
                for (int c = 0; c < 128; c++) {
                    float val = rv[c] * 0.0078125f * szo_f16_to_f32(h_u16(blob, osv + 2 * (ob * 128 + (size_t)c)));
                    wh[(size_t)c * 128 + r_in] = szo_f32_to_f16(val);
                }
            }
            for (size_t r = 0; r < 128; r++) {
                float sq = 0.0f;
                for (int c = 0; c < 128; c++) {
                    float fv = szo_f16_to_f32(wh[r * 128 + c]);
                    sq = fmaf(fv, fv, sq);
                }
                float delta = 0.9957f * sqrtf(sq * 0.0078125f);
                uint16_t sh = szo_f32_to_f16(0.5f * delta);
                float thr = 2.0f * szo_f16_to_f32(sh);
                w_sc[(ob * n_b + b) * 128 + r] = sh;
                for (size_t hb = 0; hb < 2; hb++) {
                    uint8_t* dst = w_q2 + (((ob * (n_b * 2) + b * 2 + hb) * 128 + r) * 16);
                    for (size_t wi = 0; wi < 4; wi++) {
                        size_t c0 = hb * 64 + wi * 16;
                        uint32_t pw = 0;
                        for (uint32_t sl = 0; sl < 4; sl++)
                            for (uint32_t bi = 0; bi < 4; bi++) {
                                float fv = szo_f16_to_f32(wh[r * 128 + c0 + sl * 4 + bi]);
                                uint32_t q = (fv >= 0.0f) ? (fv >= thr ? 3u : 2u) : (fv <= -thr ? 0u : 1u);
                                pw |= q << (bi * 8 + sl * 2);
                            }
                        dst[wi * 4 + 0] = (uint8_t)pw;
                        dst[wi * 4 + 1] = (uint8_t)(pw >> 8);
                        dst[wi * 4 + 2] = (uint8_t)(pw >> 16);
                        dst[wi * 4 + 3] = (uint8_t)(pw >> 24);
                    }
                }
            }
        }
    free(tile);
    free(wsrc);
    free(wh);
}

/* kernels/forward.cu:4369-4420 (proxy_q2_quant_x), one row: int8 codes per 128-block, the block's scale and the bias
 * term -3 * scale * sum(codes). */
void szo_proxy_quant_x(const float* xr, size_t cols, int8_t* xq, float* x_sc, float* x_corr) {
    for (size_t b = 0; b < cols / 128; b++) {
        float amax = 0.0f;
        for (int i = 0; i < 128; i++) amax = fmaxf(amax, fabsf(xr[b * 128 + i]));
        float sc = amax > 0.0f ? amax / 127.0f : 0.0f;
        float inv = sc > 0.0f ? 1.0f / sc : 0.0f;
        int tot = 0;
        for (int i = 0; i < 128; i++) {
            float t = fmaxf(-127.0f, fminf(127.0f, xr[b * 128 + i] * inv));
            int q = (int)rintf(t); /* round to nearest even, as __float2int_rn */
            xq[b * 128 + i] = (int8_t)q;
            tot += q;
        }
        x_sc[b] = sc;
        x_corr[b] = -3.0f * (float)tot * sc;
    }
}

/* kernels/forward.cu:4428-4495 (proxy_q2_dp4a_impl), one row of the pass: bmax[ob] = the largest proxy score of the
 * 128 outputs of block ob. */
void szo_proxy_bmax(size_t rows, size_t cols, const uint8_t* w_q2, const uint16_t* w_sc, const int8_t* xq, const float* x_sc,
                    const float* x_corr, float* bmax) {
    const size_t n_b = cols / 128, n_ob = rows / 128;
    for (size_t ob = 0; ob < n_ob; ob++) {
        float best = 0.0f;
        for (size_t r = 0; r < 128; r++) {
            float acc = 0.0f;
            for (size_t b = 0; b < n_b; b++) {
                int ia = 0;
                for (size_t hb = 0; hb < 2; hb++) {
                    const uint8_t* src = w_q2 + (((ob * (n_b * 2) + b * 2 + hb) * 128 + r) * 16);
                    for (size_t wi = 0; wi < 4; wi++) {
                        uint32_t w = (uint32_t)src[wi * 4] | ((uint32_t)src[wi * 4 + 1] << 8) | ((uint32_t)src[wi * 4 + 2] << 16) |
                                     ((uint32_t)src[wi * 4 + 3] << 24);
                        for (uint32_t sl = 0; sl < 4; sl++)
                            for (uint32_t bi = 0; bi < 4; bi++) {
                                int q = (int)((w >> (bi * 8 + sl * 2)) & 3u);
                                ia += q * (int)xq[b * 128 + hb * 64 + wi * 16 + sl * 4 + bi];
                            }
                    }
                }
                float wsc = szo_f16_to_f32(w_sc[(ob * n_b + b) * 128 + r]);
                acc = fmaf(wsc, fmaf(2.0f * x_sc[b], (float)ia, x_corr[b]), acc);
            }
            best = r == 0 ? acc : fmaxf(best, acc);
        }
        bmax[ob] = best;
    }
}

/* crates/shadowzero-cuda/src/session.rs:5964: blocks kept per row of the pass. */
int szo_head_k_use(int k_blk, int need_k) {
    if (need_k > 16) return k_blk;
    int k = k_blk * 3 / 4;
    if (k < 64) k = 64;
    return k < k_blk ? k : k_blk;
}

/* kernels/forward.cu:4536-4632 (proxy_pick_rows + proxy_compact_seen): the k_use best blocks of each of the m rows
 * (value descending, index ascending, NaN below everything), their union in ascending order, cut at max_sel.
 * Returns the number of blocks written to sel.
 * Deviation, stated: the reference's kernel first keeps four candidates per class of (index mod 256), which is the
 * exact k best only while n_ob <= 1024; this is the exact k best for every n_ob. */
int szo_proxy_pick(const float* bmax, int m, int n_ob, int k_use, int max_sel, uint32_t* sel) {
    uint8_t* seen = (uint8_t*)calloc((size_t)n_ob, 1);
    int* order = (int*)malloc((size_t)n_ob * sizeof(int));
    float* v = (float*)malloc((size_t)n_ob * sizeof(float));
    for (int j = 0; j < m; j++) {
        for (int i = 0; i < n_ob; i++) {
            float t = bmax[(size_t)j * n_ob + i];
            v[i] = t != t ? -3.0e38f : t;
            order[i] = i;
        }
        int k = k_use < n_ob ? k_use : n_ob;
        for (int a = 0; a < k; a++) { /* selection: k is small */
            int best = a;
            for (int c = a + 1; c < n_ob; c++) {
                int x = order[c], y = order[best];
                if (v[x] > v[y] || (v[x] == v[y] && x < y)) best = c;
            }
            int t = order[a]; order[a] = order[best]; order[best] = t;
            seen[order[a]] = 1;
        }
    }
    int n = 0;
    for (int i = 0; i < n_ob && n < max_sel; i++)
        if (seen[i]) sel[n++] = (uint32_t)i;
    free(seen);
    free(order);
    free(v);
    return n;
}
