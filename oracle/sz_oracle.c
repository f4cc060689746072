/* CPU oracle, part 1: number formats, dequantisers, EXL3, matvec, router, MoE.
 *
 * TEST INFRASTRUCTURE ONLY (see sz_oracle.h).  Compile with -ffp-contract=off: the reference's Rust never fuses a
 * multiply and an add, and bit-exactness of the dequantised weights depends on that.
 */
#include "sz_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------------------------------------------------------- */
/* a scoped parallel-for over [0, n) in chunks of `per`, one thread per chunk (forward.rs:205-226 spawns per chunk)  */

typedef void (*szo_chunk_fn)(void* ctx, size_t first, size_t last);
typedef struct { szo_chunk_fn fn; void* ctx; size_t first, last; } szo_job;

static void* szo_job_main(void* p) {
    szo_job* j = (szo_job*)p;
    j->fn(j->ctx, j->first, j->last);
    return NULL;
}

static void szo_parallel_chunks(size_t n, size_t per, szo_chunk_fn fn, void* ctx) {
    if (n == 0) return;
    if (per == 0) per = 1;
    size_t chunks = (n + per - 1) / per;
    if (chunks <= 1) { fn(ctx, 0, n); return; }
    pthread_t* th = (pthread_t*)malloc(chunks * sizeof(pthread_t));
    szo_job* jobs = (szo_job*)malloc(chunks * sizeof(szo_job));
    for (size_t c = 0; c < chunks; c++) {
        jobs[c].fn = fn; jobs[c].ctx = ctx; jobs[c].first = c * per;
        jobs[c].last = (c + 1) * per < n ? (c + 1) * per : n;
        if (pthread_create(&th[c], NULL, szo_job_main, &jobs[c]) != 0) { szo_job_main(&jobs[c]); th[c] = 0; }
    }
    for (size_t c = 0; c < chunks; c++) if (th[c]) pthread_join(th[c], NULL);
    free(th); free(jobs);
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* half.rs                                                                                                          */

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* half.rs:4-22 */
float szo_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)(h >> 15)) << 31;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
    if (exp == 0 && man == 0) bits = sign;
    else if (exp == 0) {
        uint32_t shift = (uint32_t)__builtin_clz(man) - 21; /* top set bit to bit 10 */
        uint32_t m = (man << shift) & 0x3ff;
        bits = sign | ((127 - 15 + 1 - shift) << 23) | (m << 13);
    } else if (exp == 31) bits = man == 0 ? (sign | 0x7f800000u) : (sign | 0x7fc00000u | (man << 13));
    else bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    return bits_f32(bits);
}

/* half.rs:24-56: round to nearest, ties to even */
uint16_t szo_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000);
    int32_t exp = (int32_t)((x >> 23) & 0xff);
    uint32_t man = x & 0x7fffff;
    if (exp == 0xff) return (uint16_t)(sign | (man == 0 ? 0x7c00 : (0x7e00 | ((man >> 13) & 0x1ff))));
    int32_t e = exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7c00);
    if (e <= 0) {
        if (e < -10) return sign;
        uint32_t m = man | 0x800000;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half = 1u << (shift - 1);
        uint32_t rem = m & ((1u << shift) - 1);
        uint32_t r = m >> shift;
        if (rem > half || (rem == half && (r & 1))) r += 1;
        return (uint16_t)(sign | r);
    }
    uint32_t r = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fff;
    if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) r += 1;
    return (uint16_t)(sign | r);
}

float szo_bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

/* half.rs:62-69 */
uint16_t szo_f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if (f != f) return (uint16_t)((x >> 16) | 0x40);
    uint32_t bias = 0x7fff + ((x >> 16) & 1);
    return (uint16_t)((x + bias) >> 16);
}

/* exl3.rs:27-60: nearest f16 (ties to even) of a double.  Written from the definition: scale into the f16 grid of the
 * value's binade with frexp (exact), round with rint (ties to even in the default rounding mode). */
uint16_t szo_f64_to_f16_bits(double x) {
    if (x != x) return 0x7e00;
    uint16_t sign = signbit(x) ? 0x8000 : 0;
    double a = fabs(x);
    if (a >= 65520.0) return (uint16_t)(sign | 0x7c00);
    if (a < 6.103515625e-5) return (uint16_t)(sign | (uint16_t)rint(a * 16777216.0));
    int e2;
    double fr = frexp(a, &e2); /* a = fr * 2^e2, fr in [0.5, 1) */
    int e = e2 - 1;            /* a = (2 fr) * 2^e, 2 fr in [1, 2) */
    uint32_t m = (uint32_t)rint((2.0 * fr - 1.0) * 1024.0);
    if (m == 1024) { m = 0; e += 1; }
    if (e + 15 >= 31) return (uint16_t)(sign | 0x7c00);
    return (uint16_t)(sign | ((uint32_t)(e + 15) << 10) | m);
}

static inline float round_f16(double x) { return szo_f16_to_f32(szo_f64_to_f16_bits(x)); }

/* ---------------------------------------------------------------------------------------------------------------- */
/* quant.rs                                                                                                         */

/* The IQ3_S codebook (quant_tables.rs IQ3S_GRID): entry i, byte j = magnitude of weight j of the group of four. */
static const uint32_t g_iq3s_grid[512] = {
#include "iq3s_grid.inc"
};

int szo_block(int type, int* elems, int* bytes) {
    int e = 0, b = 0;
    switch (type) {
        case SZO_F32: e = 1; b = 4; break;
        case SZO_F16: e = 1; b = 2; break;
        case SZO_BF16: e = 1; b = 2; break;
        case SZO_Q8_0: e = 32; b = 34; break;
        case SZO_IQ3_S: e = 256; b = 110; break;
        default: return 0;
    }
    if (elems) *elems = e;
    if (bytes) *bytes = b;
    return 1;
}

static inline float f16_at(const uint8_t* b, size_t i) { return szo_f16_to_f32((uint16_t)(b[i] | (b[i + 1] << 8))); }

/* quant.rs:174-179 */
static void dq_q8_0(const uint8_t* b, float* y) {
    float d = f16_at(b, 0);
    for (int i = 0; i < 32; i++) y[i] = d * (float)(int8_t)b[2 + i];
}

/* quant.rs:148-159 */
static void dq_iq3_s(const uint8_t* b, float* y) {
    float d = f16_at(b, 0);
    const uint8_t *qs = b + 2, *qh = b + 66, *signs = b + 74, *scales = b + 106;
    for (int e = 0; e < 256; e++) {
        int j = e / 4;
        int idx = qs[j] | (((qh[j / 8] >> (j % 8)) & 1) << 8);
        int g = e / 32;
        int s = (scales[g / 2] >> (4 * (g % 2))) & 0x0f;
        float db = d * (float)(1 + 2 * s);
        float sg = ((signs[e / 8] >> (e % 8)) & 1) ? -1.0f : 1.0f;
        y[e] = db * (float)((g_iq3s_grid[idx] >> (8 * (e % 4))) & 0xff) * sg;
    }
}

int szo_dequant(int type, const uint8_t* data, size_t nbytes, float* out, size_t nout) {
    int be, bb;
    if (!szo_block(type, &be, &bb)) return -1;
    if (nbytes % (size_t)bb != 0 || nout != nbytes / (size_t)bb * (size_t)be) return -1;
    size_t nb = nbytes / (size_t)bb;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t* b = data + i * (size_t)bb;
        float* y = out + i * (size_t)be;
        switch (type) {
            case SZO_F32: memcpy(y, b, 4); break;
            case SZO_F16: y[0] = f16_at(b, 0); break;
            case SZO_BF16: y[0] = szo_bf16_to_f32((uint16_t)(b[0] | (b[1] << 8))); break;
            case SZO_Q8_0: dq_q8_0(b, y); break;
            case SZO_IQ3_S: dq_iq3_s(b, y); break;
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* exl3.rs                                                                                                          */

/* exl3.rs:66-70 */
static float two_halves_sum(uint32_t x) {
    x = (x & 0x8fff8fffu) ^ 0x3b603b60u;
    return round_f16((double)szo_f16_to_f32((uint16_t)(x & 0xffff)) + (double)szo_f16_to_f32((uint16_t)(x >> 16)));
}

/* exl3.rs:72-93 */
float szo_exl3_cb(int cb, uint32_t state) {
    if (cb == 0) return two_halves_sum(state * 89226354u + 64248484u);
    if (cb == 1) return two_halves_sum(state * 0xCBAC1FEDu);
    uint32_t x = state * 0x83DCD12Du;
    uint32_t sum = 0x6400u + (x & 0xff) + ((x >> 8) & 0xff) + ((x >> 16) & 0xff) + (x >> 24);
    double h = (double)szo_f16_to_f32((uint16_t)sum);
    double k_inv = (double)szo_f16_to_f32(0x1eee), k_bias = (double)szo_f16_to_f32(0xc931);
    return round_f16(h * k_inv + k_bias); /* exact in f64 before the single rounding: an f16 fma */
}

/* exl3.rs:105-110 */
void szo_exl3_tile_pos(int p, int* row, int* col) {
    int l = p / 8, j = p % 8;
    *row = 2 * (l % 4) + (j & 1) + 8 * ((j >> 1) & 1);
    *col = 2 * (l >> 3) + ((l >> 2) & 1) + 8 * (j >> 2);
}

static inline int ring_words(int bits, int half) { return half ? 4 * (2 * bits + 1) : 8 * bits; } /* exl3.rs:151-154 */
static inline int tile_words(int bits, int half) { return 2 * ring_words(bits, half); }

/* exl3.rs:163-170 */
static inline int end_bit(int bits, int half, int t) {
    if (!half) return (t + 1) * bits;
    int b2 = 2 * bits + 1;
    return (t & 1) ? (t / 2 + 1) * b2 : (t / 2) * b2 + bits;
}

/* exl3.rs:125-130 */
static inline uint32_t stream_bit(const uint16_t* tile, int s) {
    int w = s / 32;
    uint32_t word = (uint32_t)tile[2 * w] | ((uint32_t)tile[2 * w + 1] << 16);
    return (word >> (31 - s % 32)) & 1;
}

/* exl3.rs:173-182 */
uint32_t szo_exl3_state(const uint16_t* tile, int bits, int half, int t) {
    int n = ring_words(bits, half) * 32;
    int end = end_bit(bits, half, t);
    uint32_t w = 0;
    for (int b = 0; b < 16; b++) w = (w << 1) | stream_bit(tile, (end + n - 16 + b) % n);
    return w;
}

/* exl3.rs:190-197 */
void szo_exl3_decode_tile(const uint16_t* tile, int bits, int half, int cb, float* out) {
    for (int t = 0; t < 256; t++) out[t] = szo_exl3_cb(cb, szo_exl3_state(tile, bits, half, t));
}

static float* g_cb_lut[3];
static pthread_mutex_t g_cb_mu = PTHREAD_MUTEX_INITIALIZER;

/* exl3.rs:342-346 */
static const float* cb_table(int cb) {
    if (cb > 2) cb = 2;
    pthread_mutex_lock(&g_cb_mu);
    if (!g_cb_lut[cb]) {
        float* t = (float*)malloc(65536 * sizeof(float));
        for (uint32_t s = 0; s < 65536; s++) t[s] = szo_exl3_cb(cb, s);
        g_cb_lut[cb] = t;
    }
    pthread_mutex_unlock(&g_cb_mu);
    return g_cb_lut[cb];
}

/* exl3.rs:363-374: 64-bit windows and a table for the codebook; the same values as the bit loop */
static void decode_tile_lut(const uint16_t* tile, int bits, int half, const float* lut, float* out) {
    int nw = ring_words(bits, half), n = nw * 32;
    for (int t = 0; t < 256; t++) {
        int s = (end_bit(bits, half, t) + n - 16) % n;
        int wi = s / 32, sh = s % 32;
        int wj = (wi + 1) % nw;
        uint64_t a = (uint32_t)tile[2 * wi] | ((uint32_t)tile[2 * wi + 1] << 16);
        uint64_t b = (uint32_t)tile[2 * wj] | ((uint32_t)tile[2 * wj + 1] << 16);
        uint64_t merged = (a << 32) | b;
        out[t] = lut[(merged >> (48 - sh)) & 0xffff];
    }
}

void szo_exl3_decode_tile_fast(const uint16_t* tile, int bits, int half, int cb, float* out) {
    decode_tile_lut(tile, bits, half, cb_table(cb), out);
}

/* exl3.rs:583-599 */
void szo_wht128(float* v) {
    for (int h = 1; h < 128; h *= 2)
        for (int i = 0; i < 128; i += 2 * h)
            for (int j = i; j < i + h; j++) {
                float a = v[j], b = v[j + h];
                v[j] = a + b;
                v[j + h] = a - b;
            }
    const float s = 0.08838835f; /* 1 / sqrt(128) */
    for (int i = 0; i < 128; i++) v[i] *= s;
}

/* exl3.rs:378-381 */
size_t szo_exl3_blob_len(size_t in, size_t out, int bits, int half) {
    return 2 * in + 2 * out + 4 + in * out * (size_t)(2 * bits + (half ? 1 : 0)) / 16;
}

static inline uint16_t u16_at(const uint8_t* b, size_t i) { return (uint16_t)(b[i] | (b[i + 1] << 8)); }

/* exl3.rs:230-286 (reconstruct_inner then reconstruct), reading the blob layout of exl3.rs:388-398 */
void szo_exl3_reconstruct(size_t in, size_t out, int bits, int half, int cb, const uint8_t* blob, float* w) {
    size_t osv = 2 * in, otr = 2 * in + 2 * out + 4;
    size_t kt = in / 16, nt = out / 16;
    int tw = tile_words(bits, half);
    uint16_t* tile = (uint16_t*)malloc((size_t)tw * 2);
    float vals[256];
    for (size_t k = 0; k < kt; k++)
        for (size_t n = 0; n < nt; n++) {
            const uint8_t* tb = blob + otr + (k * nt + n) * (size_t)tw * 2;
            for (int i = 0; i < tw; i++) tile[i] = u16_at(tb, 2 * (size_t)i);
            szo_exl3_decode_tile(tile, bits, half, cb, vals);
            for (int p = 0; p < 256; p++) {
                int r, c;
                szo_exl3_tile_pos(p, &r, &c);
                w[(k * 16 + (size_t)r) * out + n * 16 + (size_t)c] = vals[p];
            }
        }
    free(tile);
    float col[128];
    for (size_t b = 0; b < in / 128; b++)
        for (size_t c = 0; c < out; c++) {
            for (int i = 0; i < 128; i++) col[i] = w[(b * 128 + (size_t)i) * out + c];
            szo_wht128(col);
            for (int i = 0; i < 128; i++) w[(b * 128 + (size_t)i) * out + c] = col[i];
        }
    for (size_t i = 0; i < in; i++) {
        float s = szo_f16_to_f32(u16_at(blob, 2 * i));
        for (size_t c = 0; c < out; c++) w[i * out + c] *= s;
    }
    for (size_t r = 0; r < in; r++)
        for (size_t b = 0; b < out / 128; b++) szo_wht128(&w[r * out + b * 128]);
    for (size_t r = 0; r < in; r++)
        for (size_t c = 0; c < out; c++) w[r * out + c] *= szo_f16_to_f32(u16_at(blob, osv + 2 * c));
}

typedef struct {
    size_t in, out; int bits, half; const uint8_t* blob; const float* xr; const float* lut; float* y;
} exl3_mv_ctx;

/* exl3.rs:537-563: one 128-output block */
static void exl3_mv_blocks(void* p, size_t first, size_t last) {
    exl3_mv_ctx* c = (exl3_mv_ctx*)p;
    size_t kt = c->in / 16, nt = c->out / 16;
    int tw = tile_words(c->bits, c->half);
    size_t osv = 2 * c->in, otr = 2 * c->in + 2 * c->out + 4;
    uint16_t* tile = (uint16_t*)malloc((size_t)tw * 2);
    int prow[256], pcol[256];
    for (int q = 0; q < 256; q++) szo_exl3_tile_pos(q, &prow[q], &pcol[q]);
    for (size_t ob = first; ob < last; ob++) {
        double acc[128];
        float vals[256], o[128];
        for (int i = 0; i < 128; i++) acc[i] = 0.0;
        for (size_t cc = 0; cc < 8; cc++) {
            size_t n = ob * 8 + cc;
            for (size_t k = 0; k < kt; k++) {
                const uint8_t* tb = c->blob + otr + (k * nt + n) * (size_t)tw * 2;
                for (int i = 0; i < tw; i++) tile[i] = u16_at(tb, 2 * (size_t)i);
                decode_tile_lut(tile, c->bits, c->half, c->lut, vals);
                const float* xk = c->xr + k * 16;
                for (int q = 0; q < 256; q++) acc[cc * 16 + (size_t)pcol[q]] += (double)xk[prow[q]] * (double)vals[q];
            }
        }
        for (int i = 0; i < 128; i++) o[i] = (float)acc[i];
        szo_wht128(o);
        for (int i = 0; i < 128; i++) c->y[ob * 128 + (size_t)i] = o[i] * szo_f16_to_f32(u16_at(c->blob, osv + 2 * (ob * 128 + (size_t)i)));
    }
    free(tile);
}

/* exl3.rs:520-581 */
void szo_exl3_matvec_blob(size_t in, size_t out, int bits, int half, int cb, const uint8_t* blob, const float* x,
                          float* y, int threads) {
    float* xr = (float*)malloc(in * sizeof(float));
    for (size_t i = 0; i < in; i++) xr[i] = x[i] * szo_f16_to_f32(u16_at(blob, 2 * i));
    for (size_t b = 0; b < in / 128; b++) szo_wht128(xr + b * 128);
    exl3_mv_ctx c = { in, out, bits, half, blob, xr, cb_table(cb), y };
    size_t nb = out / 128;
    size_t th = threads > 0 ? (size_t)threads : 1;
    size_t per = (nb + th - 1) / th;
    if (per < 1) per = 1;
    szo_parallel_chunks(nb, per, exl3_mv_blocks, &c);
    free(xr);
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* forward.rs                                                                                                       */

typedef struct { int type; const uint8_t* bytes; size_t cols, rb; const float* x; float* y; } mv_ctx;

/* forward.rs:216-224 */
static void mv_rows(void* p, size_t first, size_t last) {
    mv_ctx* c = (mv_ctx*)p;
    float* w = (float*)malloc(c->cols * sizeof(float));
    for (size_t r = first; r < last; r++) {
        szo_dequant(c->type, c->bytes + r * c->rb, c->rb, w, c->cols);
        double acc = 0.0;
        for (size_t i = 0; i < c->cols; i++) acc += (double)w[i] * (double)c->x[i];
        c->y[r] = (float)acc;
    }
    free(w);
}

int szo_matvec(int type, const uint8_t* bytes, size_t rows, size_t cols, const float* x, float* y, int threads) {
    if (type > SZO_EXL3_BASE && type <= SZO_EXL3_BASE + 8) {
        szo_exl3_matvec_blob(cols, rows, type - SZO_EXL3_BASE, 0, 2, bytes, x, y, threads); /* forward.rs:241-246 */
        return 0;
    }
    int be, bb;
    if (!szo_block(type, &be, &bb) || cols % (size_t)be != 0) return -1;
    mv_ctx c = { type, bytes, cols, cols / (size_t)be * (size_t)bb, x, y };
    size_t th = threads > 0 ? (size_t)threads : 1;
    size_t per = (rows + th - 1) / th;
    if (per < 16) per = 16; /* forward.rs:213 */
    szo_parallel_chunks(rows, per, mv_rows, &c);
    return 0;
}

/* forward.rs:251-255 */
void szo_rmsnorm(const float* x, const float* w, size_t n, float eps, float* y) {
    double ms = 0.0;
    for (size_t i = 0; i < n; i++) ms += (double)x[i] * (double)x[i];
    ms /= (double)n;
    double r = 1.0 / sqrt(ms + (double)eps);
    for (size_t i = 0; i < n; i++) y[i] = (float)((double)x[i] * r) * w[i];
}

float szo_sigmoid(float x) { return (float)(1.0 / (1.0 + exp(-(double)x))); }       /* forward.rs:262-264 */
float szo_silu(float x) { return x * szo_sigmoid(x); }                               /* forward.rs:266-268 */
float szo_softplus(float x) { return x > 20.0f ? x : (float)log1p(exp((double)x)); } /* forward.rs:270-272 */

/* forward.rs:1088-1153.  Both branches of the reference (the fixed-array one for n <= 512, k <= 16 and the general
 * one) keep the first k of the order (ex descending, index ascending); this is that order, by insertion. */
int szo_route(const float* logits, int n, int k, int32_t* idx, double* w) {
    if (k <= 0 || n <= 0) return 0;
    float mx = -3.40282347e+38f; /* f32::MIN */
    for (int i = 0; i < n; i++) mx = logits[i] > mx ? logits[i] : mx; /* f32::max ignores a NaN operand */
    double* ex = (double*)malloc((size_t)n * sizeof(double));
    double z = 0.0;
    for (int i = 0; i < n; i++) { ex[i] = exp((double)(logits[i] - mx)); z += ex[i]; }
    int len = 0;
    for (int i = 0; i < n; i++) {
        if (len == k) {
            int t = idx[k - 1];
            if (!(ex[i] > ex[t])) continue; /* equal: the earlier index stays */
        }
        int pos = len < k ? len : k - 1;
        while (pos > 0) {
            int prev = idx[pos - 1];
            if (ex[prev] > ex[i] || (ex[prev] == ex[i] && prev < i)) break;
            idx[pos] = prev;
            pos--;
        }
        idx[pos] = i;
        if (len < k) len++;
    }
    double tz = 0.0;
    for (int t = 0; t < len; t++) tz += ex[idx[t]] / z;
    for (int t = 0; t < len; t++) w[t] = (ex[idx[t]] / z) / tz;
    free(ex);
    return len;
}

/* forward.rs:1009-1034 */
void szo_moe(const szo_moe_layer* L, const float* u, float* y, int32_t* route_idx, double* route_w, float* logits_out,
             int threads) {
    int H = L->hidden, FF = L->expert_ff, SF = L->shared_ff, k = L->top_k;
    float* logits = (float*)malloc((size_t)L->n_expert * sizeof(float));
    szo_matvec(SZO_F32, (const uint8_t*)L->router, (size_t)L->n_expert, (size_t)H, u, logits, threads);
    int32_t* idx = (int32_t*)malloc((size_t)k * sizeof(int32_t));
    double* rw = (double*)malloc((size_t)k * sizeof(double));
    int nk = szo_route(logits, L->n_expert, k, idx, rw);
    double* acc = (double*)calloc((size_t)H, sizeof(double));
    size_t mff = (size_t)(FF > SF ? FF : SF);
    float* g = (float*)malloc(mff * sizeof(float));
    float* up = (float*)malloc(mff * sizeof(float));
    float* out = (float*)malloc((size_t)H * sizeof(float));
    for (int t = 0; t < nk; t++) {
        size_t e = (size_t)idx[t];
        szo_matvec(L->expert_type, L->gate + e * L->gate_stride, (size_t)FF, (size_t)H, u, g, threads);
        szo_matvec(L->expert_type, L->up + e * L->up_stride, (size_t)FF, (size_t)H, u, up, threads);
        for (int i = 0; i < FF; i++) g[i] = szo_silu(g[i]) * up[i];
        szo_matvec(L->expert_type, L->down + e * L->down_stride, (size_t)H, (size_t)FF, g, out, threads);
        for (int i = 0; i < H; i++) acc[i] += rw[t] * (double)out[i];
    }
    if (SF > 0) {
        szo_matvec(L->shared_type, L->sh_gate, (size_t)SF, (size_t)H, u, g, threads);
        szo_matvec(L->shared_type, L->sh_up, (size_t)SF, (size_t)H, u, up, threads);
        for (int i = 0; i < SF; i++) g[i] = szo_silu(g[i]) * up[i];
        szo_matvec(L->shared_type, L->sh_down, (size_t)H, (size_t)SF, g, out, threads);
        float sgl;
        szo_matvec(SZO_F32, (const uint8_t*)L->shared_router, 1, (size_t)H, u, &sgl, 1);
        float sg = szo_sigmoid(sgl);
        for (int i = 0; i < H; i++) y[i] = (float)(acc[i] + (double)(sg * out[i]));
    } else { /* a layer without a shared expert (not a shape the reference's model has) */
        for (int i = 0; i < H; i++) y[i] = (float)acc[i];
    }
    if (route_idx) for (int t = 0; t < k; t++) route_idx[t] = t < nk ? idx[t] : -1;
    if (route_w) for (int t = 0; t < k; t++) route_w[t] = t < nk ? rw[t] : 0.0;
    if (logits_out) memcpy(logits_out, logits, (size_t)L->n_expert * sizeof(float));
    free(logits); free(idx); free(rw); free(acc); free(g); free(up); free(out);
}
