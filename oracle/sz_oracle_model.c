/* CPU oracle, part 2: the whole forward step (hyper-connections, DeltaNet, gated attention, MoE, head), the Q8_KV
 * quantiser, the top-64 order, the suffix drafter, the sampler and the draft / verify / accept loop.
 *
 * TEST INFRASTRUCTURE ONLY (see sz_oracle.h).  Restates crates/shadowzero-model/src/forward.rs:751-1034,1078-1084,
 * crates/shadowzero-serve/src/engine.rs:823-1011,2204-2419 and crates/shadowzero-serve/src/sampler.rs:83-210; the Q8_KV
 * quantiser and the top-64 order follow kernels/forward.cu:3565-3625,3652-3687 (they exist only as kernels in the reference).
 * Not restated: the per-layer-embedding branch (forward.rs:1037-1074) and the sparse indexer (forward.rs:930-976); a model
 * described by sz_model has neither.
 */
#include "sz_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------------------------------------------------------- */
/* small helpers                                                                                                    */

static size_t row_bytes(const sz_tensor* t) {
    int be, bb;
    if (!szo_block(t->type, &be, &bb)) return 0;
    return (size_t)t->cols / (size_t)be * (size_t)bb;
}

static const float* f32p(const sz_tensor* t) { return (const float*)(uintptr_t)t->data; }

/* y = W x through the reference's matvec (forward.rs:724-740 `mv`; no `.scale` companions in these models) */
static void mv(const sz_tensor* t, const float* x, float* y, int threads) {
    szo_matvec(t->type, (const uint8_t*)(uintptr_t)t->data, (size_t)t->rows, (size_t)t->cols, x, y, threads);
}

/* forward.rs:258-260 */
static void rmsnorm_groups(const float* x, const float* w, size_t n, size_t group, float eps, float* y) {
    for (size_t o = 0; o < n; o += group) szo_rmsnorm(x + o, w + o, group, eps, y + o);
}

/* forward.rs:290-299 */
static void rope_apply(float* x, double pos, int dims, double theta) {
    int half = dims / 2;
    for (int i = 0; i < half; i++) {
        double f = pos / pow(theta, 2.0 * (double)i / (double)dims);
        double cs = cos(f), sn = sin(f);
        double a = (double)x[i], b = (double)x[i + half];
        x[i] = (float)(a * cs - b * sn);
        x[i + half] = (float)(b * cs + a * sn);
    }
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* Q8_KV (kernels/forward.cu:3652-3687)                                                                             */

size_t szo_kv_q8_head_bytes(int hd) { return (size_t)hd + ((((size_t)hd >> 5) * 2u + 15u) & ~(size_t)15u); }

void szo_kv_quant_q8(const float* src, int hd, uint8_t* dst) {
    int ng = hd >> 5;
    memset(dst + hd, 0, szo_kv_q8_head_bytes(hd) - (size_t)hd);
    for (int g = 0; g < ng; g++) {
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) { float a = fabsf(src[g * 32 + i]); amax = a > amax ? a : amax; }
        uint16_t sh = szo_f32_to_f16(amax > 0.0f ? amax * (1.0f / 127.0f) : 0.0f);
        float sr = szo_f16_to_f32(sh);
        float inv = sr > 0.0f ? (1.0f / sr) : 0.0f;
        for (int i = 0; i < 32; i++) {
            int q = (int)lrintf(src[g * 32 + i] * inv); /* round to nearest even: __float2int_rn */
            q = q < -127 ? -127 : (q > 127 ? 127 : q);
            dst[g * 32 + i] = (uint8_t)(int8_t)q;
        }
        dst[hd + 2 * g] = (uint8_t)(sh & 0xff);
        dst[hd + 2 * g + 1] = (uint8_t)(sh >> 8);
    }
}

void szo_kv_dequant_q8(const uint8_t* src, int hd, float* dst) {
    for (int i = 0; i < hd; i++) {
        int g = i >> 5;
        uint16_t sh = (uint16_t)(src[hd + 2 * g] | (src[hd + 2 * g + 1] << 8));
        dst[i] = (float)(int8_t)src[i] * szo_f16_to_f32(sh);
    }
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* top-64 (kernels/forward.cu:3565-3625): largest first, ties to the lower id, NaN counts as -inf, padding (-inf, ~0) */

void szo_top64(const float* logits, int vocab, float* vals, uint32_t* ids) {
    const float ninf = -INFINITY;
    int n = 0;
    for (int i = 0; i < vocab; i++) {
        float v = logits[i];
        if (v != v) v = ninf;
        if (n == 64) {
            float lv = vals[63];
            if (!(v > lv)) continue; /* equal: the earlier id stays */
        }
        int pos = n < 64 ? n : 63;
        while (pos > 0 && (vals[pos - 1] < v)) { vals[pos] = vals[pos - 1]; ids[pos] = ids[pos - 1]; pos--; }
        vals[pos] = v;
        ids[pos] = (uint32_t)i;
        if (n < 64) n++;
    }
    for (int i = n; i < 64; i++) { vals[i] = ninf; ids[i] = 0xffffffffu; }
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* the session (forward.rs:694-794)                                                                                 */

typedef struct {
    float* s;    /* v_heads x d x d */
    float* conv; /* (conv_k - 1) x channels, oldest first */
    float* k;    /* attention: positions x kv_heads x head_dim (f32 mode) */
    float* v;
    uint8_t* kq; /* attention: positions x kv_heads x head_bytes (Q8 mode) */
    uint8_t* vq;
    size_t cap;  /* positions allocated */
    /* the sparse indexer (forward.rs:282-286): raw keys, one per position, and the pooled key of every complete block */
    float* idx_raw;   /* positions x idx_dim */
    float* blocks;    /* complete blocks x idx_dim */
    size_t n_blocks;  /* blocks whose pooled key is valid */
    int32_t* sel;     /* positions the last step attended to, ascending */
    size_t n_sel;
    float* scores;    /* block scores of the last step that selected (n_scores of them) */
    size_t n_scores;
} layer_state;

struct szo_session {
    const sz_model* m;
    int kv_q8, threads;
    size_t len;
    uint32_t* tokens;   /* every token read so far (the PLE hashes the last few) */
    size_t tok_cap;
    float* ple_conv;    /* the PLE's conv history: (conv_k - 1) * ngram rows of streams * hidden, oldest first (forward.rs:701) */
    layer_state* st;
    int32_t* routes; /* [n_layer][top_k] of the last step */
    double* route_w;
};

static size_t ple_hist_floats(const sz_model* m) {
    return (size_t)(m->ple.conv_k - 1) * (size_t)m->ple.ngram * (size_t)m->cfg.streams * (size_t)m->cfg.hidden;
}
static int is_attention(const sz_model_config* c, int l) { return l % c->attn_interval == c->attn_interval - 1; }
static size_t delta_channels(const sz_model_config* c) { return (size_t)(2 * c->ssm_k_heads + c->ssm_v_heads) * (size_t)c->ssm_head_dim; }
static size_t delta_s_floats(const sz_model_config* c) { return (size_t)c->ssm_v_heads * (size_t)c->ssm_head_dim * (size_t)c->ssm_head_dim; }

szo_session* szo_session_new(const sz_model* m, int kv_q8, int threads) {
    const sz_model_config* c = &m->cfg;
    szo_session* s = (szo_session*)calloc(1, sizeof(szo_session));
    s->m = m; s->kv_q8 = kv_q8; s->threads = threads > 0 ? threads : 1;
    s->st = (layer_state*)calloc((size_t)c->n_layer, sizeof(layer_state));
    for (int l = 0; l < c->n_layer; l++) {
        if (!is_attention(c, l)) {
            s->st[l].s = (float*)calloc(delta_s_floats(c), sizeof(float));
            s->st[l].conv = (float*)calloc((size_t)(c->conv_k - 1) * delta_channels(c), sizeof(float));
        }
    }
    s->routes = (int32_t*)calloc((size_t)c->n_layer * (size_t)c->n_expert_used, sizeof(int32_t));
    s->route_w = (double*)calloc((size_t)c->n_layer * (size_t)c->n_expert_used, sizeof(double));
    if (m->ple.ngram >= 2) s->ple_conv = (float*)calloc(ple_hist_floats(m), sizeof(float));
    return s;
}

void szo_session_free(szo_session* s) {
    if (!s) return;
    for (int l = 0; l < s->m->cfg.n_layer; l++) {
        free(s->st[l].s); free(s->st[l].conv); free(s->st[l].k); free(s->st[l].v); free(s->st[l].kq); free(s->st[l].vq);
        free(s->st[l].idx_raw); free(s->st[l].blocks); free(s->st[l].sel); free(s->st[l].scores);
    }
    free(s->st); free(s->routes); free(s->route_w); free(s->tokens); free(s->ple_conv); free(s);
}

int szo_session_len(const szo_session* s) { return (int)s->len; }
const int32_t* szo_session_routes(const szo_session* s) { return s->routes; }
const double* szo_session_route_weights(const szo_session* s) { return s->route_w; }

static void kv_reserve(szo_session* s, layer_state* L, size_t positions) {
    const sz_model_config* c = &s->m->cfg;
    if (positions <= L->cap) return;
    size_t cap = L->cap ? L->cap * 2 : 256;
    while (cap < positions) cap *= 2;
    size_t row = (size_t)c->n_kv_head * (size_t)c->head_dim;
    size_t rowq = (size_t)c->n_kv_head * szo_kv_q8_head_bytes(c->head_dim);
    if (s->kv_q8) { L->kq = (uint8_t*)realloc(L->kq, cap * rowq); L->vq = (uint8_t*)realloc(L->vq, cap * rowq); }
    else { L->k = (float*)realloc(L->k, cap * row * sizeof(float)); L->v = (float*)realloc(L->v, cap * row * sizeof(float)); }
    if (c->idx_heads > 0) {
        L->idx_raw = (float*)realloc(L->idx_raw, cap * (size_t)c->idx_dim * sizeof(float));
        L->blocks = (float*)realloc(L->blocks, cap * (size_t)c->idx_dim * sizeof(float));
        L->sel = (int32_t*)realloc(L->sel, cap * sizeof(int32_t));
        L->scores = (float*)realloc(L->scores, cap * sizeof(float));
    }
    L->cap = cap;
}

/* dst becomes a copy of src (same model): the snapshot / restore the CPU side of the speculation loop uses */
void szo_session_assign(szo_session* dst, const szo_session* src) {
    const sz_model_config* c = &src->m->cfg;
    dst->len = src->len;
    if (src->len > dst->tok_cap) { dst->tok_cap = src->tok_cap; dst->tokens = (uint32_t*)realloc(dst->tokens, dst->tok_cap * sizeof(uint32_t)); }
    if (src->len && src->tokens) memcpy(dst->tokens, src->tokens, src->len * sizeof(uint32_t));
    if (src->ple_conv) memcpy(dst->ple_conv, src->ple_conv, ple_hist_floats(src->m) * sizeof(float));
    size_t row = (size_t)c->n_kv_head * (size_t)c->head_dim, rowq = (size_t)c->n_kv_head * szo_kv_q8_head_bytes(c->head_dim);
    for (int l = 0; l < c->n_layer; l++) {
        if (!is_attention(c, l)) {
            memcpy(dst->st[l].s, src->st[l].s, delta_s_floats(c) * sizeof(float));
            memcpy(dst->st[l].conv, src->st[l].conv, (size_t)(c->conv_k - 1) * delta_channels(c) * sizeof(float));
        } else {
            kv_reserve(dst, &dst->st[l], src->len);
            if (src->kv_q8) { memcpy(dst->st[l].kq, src->st[l].kq, src->len * rowq); memcpy(dst->st[l].vq, src->st[l].vq, src->len * rowq); }
            else { memcpy(dst->st[l].k, src->st[l].k, src->len * row * sizeof(float)); memcpy(dst->st[l].v, src->st[l].v, src->len * row * sizeof(float)); }
            if (c->idx_heads > 0 && src->st[l].idx_raw) {
                memcpy(dst->st[l].idx_raw, src->st[l].idx_raw, src->len * (size_t)c->idx_dim * sizeof(float));
                memcpy(dst->st[l].blocks, src->st[l].blocks, src->st[l].n_blocks * (size_t)c->idx_dim * sizeof(float));
                dst->st[l].n_blocks = src->st[l].n_blocks;
            }
        }
    }
}

szo_session* szo_session_clone(const szo_session* src) {
    szo_session* d = szo_session_new(src->m, src->kv_q8, src->threads);
    szo_session_assign(d, src);
    return d;
}

/* The synthetic history of the library's sz_session_fill_synthetic, value for value: `len` positions of every attention layer's
 * cache from an integer hash of (kv head, position, element, layer, seed), zero recurrent state.  Not part of the reference: a long
 * context for tests and benchmarks without a long prefill.  Packed heads get codes in [-127, 127] and the scale 2^-7 (f16 0x2000). */
static uint32_t fill_hash(uint64_t hp, uint32_t i, uint32_t seed, uint32_t layer) {
    uint32_t x = (uint32_t)(hp * 2654435761u) ^ (uint32_t)(i * 40503u) ^ seed ^ (uint32_t)(layer * 97u);
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}

void szo_session_fill_synthetic(szo_session* s, int len, uint32_t seed) {
    const sz_model_config* c = &s->m->cfg;
    size_t nkv = (size_t)c->n_kv_head, hd = (size_t)c->head_dim, hb = szo_kv_q8_head_bytes((int)hd);
    uint32_t ai = 0;
    for (int l = 0; l < c->n_layer; l++) {
        layer_state* L = &s->st[l];
        if (!is_attention(c, l)) {
            memset(L->s, 0, delta_s_floats(c) * sizeof(float));
            memset(L->conv, 0, (size_t)(c->conv_k - 1) * delta_channels(c) * sizeof(float));
            continue;
        }
        kv_reserve(s, L, (size_t)len);
        for (int which = 0; which < 2; which++) {
            uint32_t sd = which ? seed ^ 0x9e3779b9u : seed;
            for (size_t h = 0; h < nkv; h++)
                for (size_t pos = 0; pos < (size_t)len; pos++) {
                    uint64_t hp = (uint64_t)h * (uint64_t)len + pos;
                    if (s->kv_q8) {
                        uint8_t* p = (which ? L->vq : L->kq) + (pos * nkv + h) * hb;
                        for (size_t i = 0; i < hd; i++) p[i] = (uint8_t)(int8_t)((int)(fill_hash(hp, (uint32_t)i, sd, ai) % 255u) - 127);
                        uint16_t* sc = (uint16_t*)(p + hd);
                        for (size_t g = 0; g < (hb - hd) / 2; g++) sc[g] = g < hd / 32 ? (uint16_t)0x2000 : (uint16_t)0;
                    } else {
                        float* p = (which ? L->v : L->k) + (pos * nkv + h) * hd;
                        for (size_t i = 0; i < hd; i++) p[i] = ((float)(fill_hash(hp, (uint32_t)i, sd, ai) % 2001u) - 1000.0f) * 1e-3f;
                    }
                }
        }
        if (c->idx_heads > 0) {   /* the indexer's raw keys of the history; the pooled block keys follow from them at the next step */
            size_t id = (size_t)c->idx_dim;
            for (size_t pos = 0; pos < (size_t)len; pos++)
                for (size_t i = 0; i < id; i++)
                    L->idx_raw[pos * id + i] = ((float)(fill_hash((uint64_t)pos, (uint32_t)i, seed ^ 0x51ed270bu, ai) % 2001u) - 1000.0f) * 1e-3f;
            L->n_blocks = 0;
        }
        ai++;
    }
    s->len = (size_t)len;
    /* the tokens of that history are not known: they read as the end-of-text token to the per-layer embedding, whose conv history is zero */
    if ((size_t)len > s->tok_cap) { s->tok_cap = (size_t)len * 2; s->tokens = (uint32_t*)realloc(s->tokens, s->tok_cap * sizeof(uint32_t)); }
    for (int i = 0; i < len; i++) s->tokens[i] = (uint32_t)s->m->ple.eos;
    if (s->ple_conv) memset(s->ple_conv, 0, ple_hist_floats(s->m) * sizeof(float));
}

/* Where one piece of the session's state lives (what: 0 recurrent state, 1 carried conv rows, 2 K cache, 3 V cache) and its size. */
const void* szo_session_state(const szo_session* s, int what, int l, size_t* bytes) {
    const sz_model_config* c = &s->m->cfg;
    const layer_state* L = &s->st[l];
    size_t kvb = s->len * (size_t)c->n_kv_head * (s->kv_q8 ? szo_kv_q8_head_bytes(c->head_dim) : (size_t)c->head_dim * sizeof(float));
    switch (what) {
        case 0: *bytes = delta_s_floats(c) * sizeof(float); return L->s;
        case 1: *bytes = (size_t)(c->conv_k - 1) * delta_channels(c) * sizeof(float); return L->conv;
        case 2: *bytes = kvb; return s->kv_q8 ? (const void*)L->kq : (const void*)L->k;
        case 3: *bytes = kvb; return s->kv_q8 ? (const void*)L->vq : (const void*)L->v;
    }
    *bytes = 0;
    return NULL;
}

/* The positions layer l attended to in the last step (ascending), and the block scores it selected by (n_scores = 0: it did not
 * select).  The reference records the former as the trace stream `layerL.selected` (forward.rs:997-1004). */
int szo_session_selected(const szo_session* s, int l, int32_t* out, int cap) {
    const layer_state* L = &s->st[l];
    if (!L->sel) return -1;
    for (size_t i = 0; i < L->n_sel && (int)i < cap; i++) out[i] = L->sel[i];
    return (int)L->n_sel;
}
int szo_session_idx_scores(const szo_session* s, int l, float* out, int cap) {
    const layer_state* L = &s->st[l];
    for (size_t i = 0; i < L->n_scores && (int)i < cap; i++) out[i] = L->scores[i];
    return (int)L->n_scores;
}

/* forward.rs:797-817 */
static void hc_read(const szo_session* s, const float* r, const sz_hc* hc, int inject, float* u, float* g) {
    const sz_model_config* c = &s->m->cfg;
    size_t h = (size_t)c->hidden, cs = (size_t)c->streams;
    float* rn = (float*)malloc(cs * h * sizeof(float));
    rmsnorm_groups(r, f32p(&hc->norm), cs * h, h, c->eps, rn);
    float* down = (float*)malloc((size_t)hc->down.rows * sizeof(float));
    mv(&hc->down, rn, down, s->threads);
    for (int64_t i = 0; i < hc->down.rows; i++) down[i] = szo_silu(down[i] / (float)cs);
    float* mix = (float*)malloc(cs * h * sizeof(float));
    mv(&hc->up, down, mix, s->threads);
    for (size_t i = 0; i < cs * h; i++) mix[i] = szo_sigmoid(mix[i]);
    for (size_t i = 0; i < h; i++) u[i] = 0.0f;
    for (size_t st = 0; st < cs; st++)
        for (size_t i = 0; i < h; i++) u[i] += mix[st * h + i] * rn[st * h + i];
    for (size_t i = 0; i < h; i++) u[i] /= (float)cs;
    if (inject) {
        mv(&hc->inject, rn, g, s->threads);
        for (size_t st = 0; st < cs; st++) g[st] = 2.0f * szo_sigmoid(g[st] / (float)cs);
    }
    free(rn); free(down); free(mix);
}

/* forward.rs:1078-1084 */
static void hc_write(float* r, const float* g, const float* y, size_t h, size_t cs) {
    for (size_t st = 0; st < cs; st++)
        for (size_t i = 0; i < h; i++) r[st * h + i] += g[st] * y[i];
}

/* forward.rs:819-896 */
static void delta_net(szo_session* s, int l, const float* u, float* y) {
    const sz_model_config* c = &s->m->cfg;
    const sz_layer* L = &s->m->layers[l];
    size_t kh = (size_t)c->ssm_k_heads, vh = (size_t)c->ssm_v_heads, d = (size_t)c->ssm_head_dim;
    size_t kd = kh * d, vd = vh * d, ch = 2 * kd + vd, k = (size_t)c->conv_k;
    float* qkv = (float*)malloc(ch * sizeof(float));
    float* z = (float*)malloc(vd * sizeof(float));
    float* b = (float*)malloc(vh * sizeof(float));
    float* a = (float*)malloc(vh * sizeof(float));
    mv(&L->attn_qkv, u, qkv, s->threads);
    mv(&L->attn_gate, u, z, s->threads);
    mv(&L->ssm_beta, u, b, s->threads);
    mv(&L->ssm_alpha, u, a, s->threads);
    const float* conv_w = f32p(&L->ssm_conv1d); /* ch x conv_k, tap k multiplies x[t - (conv_k-1) + k] */
    layer_state* st = &s->st[l];
    float* x = (float*)malloc(ch * sizeof(float));
    for (size_t i = 0; i < ch; i++) {
        double acc = (double)conv_w[i * k + (k - 1)] * (double)qkv[i];
        for (size_t t = 0; t + 1 < k; t++) acc += (double)conv_w[i * k + t] * (double)st->conv[t * ch + i];
        x[i] = szo_silu((float)acc);
    }
    memmove(st->conv, st->conv + ch, (k - 2) * ch * sizeof(float));
    memcpy(st->conv + (k - 2) * ch, qkv, ch * sizeof(float));
    float *q = x, *kk = x + kd, *v = x + 2 * kd;
    for (size_t hq = 0; hq < kh; hq++) {
        double ss = 0.0;
        for (size_t i = 0; i < d; i++) ss += (double)q[hq * d + i] * (double)q[hq * d + i];
        double n = 1.0 / sqrt(ss + 1e-6);
        for (size_t i = 0; i < d; i++) { q[hq * d + i] = (float)((double)q[hq * d + i] * n); q[hq * d + i] /= sqrtf((float)d); }
        ss = 0.0;
        for (size_t i = 0; i < d; i++) ss += (double)kk[hq * d + i] * (double)kk[hq * d + i];
        n = 1.0 / sqrt(ss + 1e-6);
        for (size_t i = 0; i < d; i++) kk[hq * d + i] = (float)((double)kk[hq * d + i] * n);
    }
    const float *a_log = f32p(&L->ssm_a), *dt = f32p(&L->ssm_dt_bias), *norm_w = f32p(&L->ssm_norm);
    float* o = (float*)malloc(vd * sizeof(float));
    float* delta = (float*)malloc(d * sizeof(float));
    float* normed = (float*)malloc(d * sizeof(float));
    for (size_t hd = 0; hd < vh; hd++) {
        float beta = szo_sigmoid(b[hd]);
        float decay = (float)exp((double)a_log[hd] * (double)szo_softplus(a[hd] + dt[hd]));
        size_t kx = hd % kh; /* value heads are tiled over the key heads (forward.rs:862-864) */
        const float *qh = q + kx * d, *kh_ = kk + kx * d, *vh_ = v + hd * d;
        float* S = st->s + hd * d * d; /* S[i * d + j]: key index i, value index j */
        for (size_t i = 0; i < d * d; i++) S[i] *= decay;
        for (size_t j = 0; j < d; j++) {
            double mem = 0.0;
            for (size_t i = 0; i < d; i++) mem += (double)S[i * d + j] * (double)kh_[i];
            delta[j] = (float)(((double)vh_[j] - mem) * (double)beta);
        }
        for (size_t i = 0; i < d; i++)
            for (size_t j = 0; j < d; j++) S[i * d + j] += kh_[i] * delta[j];
        float* oh = o + hd * d;
        for (size_t j = 0; j < d; j++) {
            double acc = 0.0;
            for (size_t i = 0; i < d; i++) acc += (double)S[i * d + j] * (double)qh[i];
            oh[j] = (float)acc;
        }
        szo_rmsnorm(oh, norm_w, d, c->eps, normed);
        for (size_t j = 0; j < d; j++) oh[j] = normed[j] * szo_sigmoid(z[hd * d + j]);
    }
    mv(&L->ssm_out, o, y, s->threads);
    free(qkv); free(z); free(b); free(a); free(x); free(o); free(delta); free(normed);
}

/* forward.rs:898-1007 without the indexer (every position is attended to).  With kv_q8 the cache holds the Q8_KV bytes and
 * the scores and the weighted sum use the dequantised values. */
static void attention(szo_session* s, int l, const float* u, float* y) {
    const sz_model_config* c = &s->m->cfg;
    const sz_layer* L = &s->m->layers[l];
    size_t nh = (size_t)c->n_head, nkv = (size_t)c->n_kv_head, hd = (size_t)c->head_dim;
    float* qg = (float*)malloc(2 * nh * hd * sizeof(float));
    float* k = (float*)malloc(nkv * hd * sizeof(float));
    float* v = (float*)malloc(nkv * hd * sizeof(float));
    mv(&L->attn_q, u, qg, s->threads);
    mv(&L->attn_k, u, k, s->threads);
    mv(&L->attn_v, u, v, s->threads);
    const float *qn = f32p(&L->attn_q_norm), *kn = f32p(&L->attn_k_norm);
    double pos = (double)(s->len - 1);
    float* q = (float*)malloc(nh * hd * sizeof(float));
    float* gate = (float*)malloc(nh * hd * sizeof(float));
    for (size_t h = 0; h < nh; h++) {
        szo_rmsnorm(qg + h * 2 * hd, qn, hd, c->eps, q + h * hd);
        rope_apply(q + h * hd, pos, c->rope_dims, c->rope_theta);
        memcpy(gate + h * hd, qg + h * 2 * hd + hd, hd * sizeof(float));
    }
    layer_state* st = &s->st[l];
    size_t n = s->len; /* this token's position is n - 1 */
    kv_reserve(s, st, n);
    size_t hb = szo_kv_q8_head_bytes((int)hd);
    float* kh = (float*)malloc(hd * sizeof(float));
    for (size_t h = 0; h < nkv; h++) {
        szo_rmsnorm(k + h * hd, kn, hd, c->eps, kh);
        rope_apply(kh, pos, c->rope_dims, c->rope_theta);
        if (s->kv_q8) {
            szo_kv_quant_q8(kh, (int)hd, st->kq + ((n - 1) * nkv + h) * hb);
            szo_kv_quant_q8(v + h * hd, (int)hd, st->vq + ((n - 1) * nkv + h) * hb);
        } else {
            memcpy(st->k + ((n - 1) * nkv + h) * hd, kh, hd * sizeof(float));
            memcpy(st->v + ((n - 1) * nkv + h) * hd, v + h * hd, hd * sizeof(float));
        }
    }
    free(kh);
    /* ---- the sparse indexer (forward.rs:930-976): positions in blocks of `ratio`; every COMPLETE block is scored against the query by
     * its pooled key; the best budget / ratio blocks and the incomplete tail are attended to.  With no more complete blocks than
     * that, everything is. */
    size_t nt = n;           /* positions attended to */
    int32_t* toks = NULL;    /* NULL: all of them */
    if (c->idx_heads > 0 && L->idx_q.data) {
        size_t ratio = L->idx_ratio > 0 ? (size_t)L->idx_ratio : 1, id = (size_t)c->idx_dim, ih = (size_t)c->idx_heads;
        float* iq = (float*)malloc(ih * id * sizeof(float));
        float* ik = (float*)malloc(id * sizeof(float));
        mv(&L->idx_q, u, iq, s->threads);
        mv(&L->idx_k, u, ik, s->threads);
        const float *iqn = f32p(&L->idx_q_norm), *ikn = f32p(&L->idx_k_norm);
        memcpy(st->idx_raw + (n - 1) * id, ik, id * sizeof(float));
        size_t nb = n / ratio;
        if (st->n_blocks > nb) st->n_blocks = nb;
        float* pooled = (float*)malloc(id * sizeof(float));
        while (st->n_blocks < nb) {
            size_t b = st->n_blocks;
            for (size_t d = 0; d < id; d++) pooled[d] = 0.0f;
            for (size_t r = 0; r < ratio; r++)
                for (size_t d = 0; d < id; d++) pooled[d] += st->idx_raw[(b * ratio + r) * id + d];
            for (size_t d = 0; d < id; d++) pooled[d] /= (float)ratio;
            szo_rmsnorm(pooled, ikn, id, c->eps, st->blocks + b * id);
            rope_apply(st->blocks + b * id, (double)(b * ratio), c->rope_dims, c->rope_theta);
            st->n_blocks++;
        }
        free(pooled);
        size_t keep = (size_t)c->idx_budget / ratio;
        st->n_scores = 0;
        if (nb > keep) {
            float* qs = (float*)malloc(ih * id * sizeof(float));
            for (size_t h = 0; h < ih; h++) {
                szo_rmsnorm(iq + h * id, iqn, id, c->eps, qs + h * id);
                rope_apply(qs + h * id, pos, c->rope_dims, c->rope_theta);
            }
            float norm = sqrtf((float)id);
            for (size_t b = 0; b < nb; b++) {
                const float* kb = st->blocks + b * id;
                float sc = 0.0f;
                for (size_t h = 0; h < ih; h++) {
                    double dot = 0.0;
                    for (size_t d = 0; d < id; d++) dot += (double)qs[h * id + d] * (double)kb[d];
                    float f = (float)dot;
                    sc += f > 0.0f ? f : 0.0f;   /* f32::max(0.0): a NaN gives 0 */
                }
                st->scores[b] = sc / norm;
            }
            st->n_scores = nb;
            free(qs);
            /* the `keep` best, score descending, block ascending among equals (a stable descending sort) */
            uint8_t* taken = (uint8_t*)calloc(nb, 1);
            for (size_t k = 0; k < keep; k++) {
                size_t best = nb;
                for (size_t b = 0; b < nb; b++)
                    if (!taken[b] && (best == nb || st->scores[b] > st->scores[best])) best = b;
                taken[best] = 1;
            }
            toks = st->sel;
            nt = 0;
            for (size_t b = 0; b < nb; b++)
                if (taken[b])
                    for (size_t r = 0; r < ratio; r++) toks[nt++] = (int32_t)(b * ratio + r);
            for (size_t t = nb * ratio; t < n; t++) toks[nt++] = (int32_t)t;
            free(taken);
        }
        if (!toks) { for (size_t t = 0; t < n; t++) st->sel[t] = (int32_t)t; }
        st->n_sel = nt;
        free(iq); free(ik);
    }
    /* dequantised views for the Q8 cache (one group at a time) */
    float *kview = NULL, *vview = NULL;
    if (s->kv_q8) { kview = (float*)malloc(n * hd * sizeof(float)); vview = (float*)malloc(n * hd * sizeof(float)); }
    float* o = (float*)malloc(nh * hd * sizeof(float));
    double* ex = (double*)malloc(n * sizeof(double));
    double scale = 1.0 / sqrt((double)hd);
    size_t last_g = (size_t)-1;
    for (size_t h = 0; h < nh; h++) {
        size_t g = h / (nh / nkv);
        if (s->kv_q8 && g != last_g) {
            for (size_t t = 0; t < n; t++) {
                szo_kv_dequant_q8(st->kq + (t * nkv + g) * hb, (int)hd, kview + t * hd);
                szo_kv_dequant_q8(st->vq + (t * nkv + g) * hb, (int)hd, vview + t * hd);
            }
            last_g = g;
        }
        const float* qh = q + h * hd;
        double mx = -1.7976931348623157e308; /* f64::MIN */
        for (size_t ti = 0; ti < nt; ti++) {
            size_t t = toks ? (size_t)toks[ti] : ti;
            const float* kt = s->kv_q8 ? kview + t * hd : st->k + (t * nkv + g) * hd;
            double sc = 0.0;
            for (size_t i = 0; i < hd; i++) sc += (double)qh[i] * (double)kt[i];
            sc *= scale;
            ex[ti] = sc;
            mx = sc > mx ? sc : mx;
        }
        double zs = 0.0;
        for (size_t ti = 0; ti < nt; ti++) { ex[ti] = exp(ex[ti] - mx); zs += ex[ti]; }
        for (size_t j = 0; j < hd; j++) {
            double acc = 0.0;
            for (size_t ti = 0; ti < nt; ti++) {
                size_t t = toks ? (size_t)toks[ti] : ti;
                float vv = s->kv_q8 ? vview[t * hd + j] : st->v[(t * nkv + g) * hd + j];
                acc += ex[ti] * (double)vv;
            }
            o[h * hd + j] = (float)(acc / zs) * szo_sigmoid(gate[h * hd + j]);
        }
    }
    mv(&L->attn_output, o, y, s->threads);
    free(qg); free(k); free(v); free(q); free(gate); free(o); free(ex); free(kview); free(vview);
}

/* forward.rs:1177-1198: the rows of the n-gram table the last tokens select */
int szo_ple_rows(const sz_ple* p, const uint32_t* tokens, size_t n, int64_t* rows) {
    long long last_eos = -1;
    for (size_t i = n; i-- > 0;) if (tokens[i] == (uint32_t)p->eos) { last_eos = (long long)i; break; }
    int nr = 0;
    for (int order = 2; order <= p->ngram; order++) {
        uint64_t mixed = 0;
        for (int sft = 0; sft < order; sft++) {
            int64_t tk = (int64_t)(uint32_t)p->eos;
            if ((size_t)(1 + sft) <= n) {
                size_t i = n - 1 - (size_t)sft;
                if (last_eos < 0 || (long long)i >= last_eos) tk = (int64_t)tokens[i];
            }
            uint64_t term = (uint64_t)tk * (uint64_t)p->multipliers[sft];   /* wrapping_mul */
            mixed = sft == 0 ? term : (mixed ^ term);
        }
        for (int j = 0; j < p->heads_per_ngram; j++) {
            int i = (order - 2) * p->heads_per_ngram + j;
            int64_t v = p->vocab[i], rmd = (int64_t)mixed % v;
            if (rmd < 0) rmd += v < 0 ? -v : v;                              /* rem_euclid */
            rows[nr++] = rmd + p->offsets[i];
        }
    }
    return nr;
}

/* forward.rs:1036-1074: the hashed n-gram memory, added to the whole residual stream */
static void ple(szo_session* s, float* r) {
    const sz_model* m = s->m;
    const sz_model_config* c = &m->cfg;
    const sz_ple* p = &m->ple;
    size_t h = (size_t)c->hidden, cs = (size_t)c->streams, ch = cs * h, hd = (size_t)p->head_dim;
    int64_t rows[SZ_PLE_MAX_HEADS];
    int nr = szo_ple_rows(p, s->tokens, s->len, rows);
    float* e = (float*)malloc(h * sizeof(float));
    size_t rb = row_bytes(&p->table);
    for (int i = 0; i < nr; i++)
        szo_dequant(p->table.type, (const uint8_t*)(uintptr_t)p->table.data + (size_t)rows[i] * rb, rb, e + (size_t)i * hd, hd);
    float* key = (float*)malloc(ch * sizeof(float));
    float* keyn = (float*)malloc(ch * sizeof(float));
    float* val = (float*)malloc(h * sizeof(float));
    float* qry = (float*)malloc(ch * sizeof(float));
    float* gv = (float*)malloc(ch * sizeof(float));
    float* gvn = (float*)malloc(ch * sizeof(float));
    mv(&p->key, e, key, s->threads);
    rmsnorm_groups(key, f32p(&p->norm_key), ch, h, c->eps, keyn);
    mv(&p->value, e, val, s->threads);
    rmsnorm_groups(r, f32p(&p->norm_query), ch, h, c->eps, qry);
    for (size_t st = 0; st < cs; st++) {
        double dot = 0.0;
        for (size_t i = 0; i < h; i++) dot += (double)keyn[st * h + i] * (double)qry[st * h + i];
        dot /= sqrt((double)h);
        double ad = fabs(dot) > 1e-6 ? fabs(dot) : 1e-6;
        double gg = sqrt(ad) * (dot > 0.0 ? 1.0 : (dot < 0.0 ? -1.0 : (signbit(dot) ? -1.0 : 1.0)));   /* f64::signum: +-1, also for +-0 */
        float sg = szo_sigmoid((float)gg);
        for (size_t i = 0; i < h; i++) gv[st * h + i] = sg * val[i];
    }
    rmsnorm_groups(gv, f32p(&p->norm_conv), ch, h, c->eps, gvn);
    size_t k = (size_t)p->conv_k, dil = (size_t)p->ngram, hist_len = (k - 1) * dil;
    const float* w = f32p(&p->conv1d);
    for (size_t i = 0; i < ch; i++) {
        double acc = (double)w[i * k + (k - 1)] * (double)gvn[i];
        for (size_t t = 0; t + 1 < k; t++) {
            size_t back = (k - 1 - t) * dil;
            acc += (double)w[i * k + t] * (double)s->ple_conv[(hist_len - back) * ch + i];
        }
        r[i] += gv[i] + szo_silu((float)acc);
    }
    memmove(s->ple_conv, s->ple_conv + ch, (hist_len - 1) * ch * sizeof(float));
    memcpy(s->ple_conv + (hist_len - 1) * ch, gvn, ch * sizeof(float));
    free(e); free(key); free(keyn); free(val); free(qry); free(gv); free(gvn);
}

/* Session::step (forward.rs:751-794).  logits may be NULL (prefill rows whose logits nobody reads); hidden_out, when not NULL,
 * receives the head's input u (the trace stream `final_u`). */
void szo_session_step(szo_session* s, uint32_t token, float* logits, float* final_u) {
    const sz_model* m = s->m;
    const sz_model_config* c = &m->cfg;
    size_t h = (size_t)c->hidden, cs = (size_t)c->streams;
    s->len += 1;
    if (s->len > s->tok_cap) { s->tok_cap = s->tok_cap ? s->tok_cap * 2 : 256; while (s->tok_cap < s->len) s->tok_cap *= 2; s->tokens = (uint32_t*)realloc(s->tokens, s->tok_cap * sizeof(uint32_t)); }
    s->tokens[s->len - 1] = token;
    float* emb = (float*)malloc(h * sizeof(float));
    size_t rb = row_bytes(&m->token_embd);
    szo_dequant(m->token_embd.type, (const uint8_t*)(uintptr_t)m->token_embd.data + (size_t)token * rb, rb, emb, h);
    float* r = (float*)malloc(cs * h * sizeof(float));
    for (size_t st = 0; st < cs; st++) memcpy(r + st * h, emb, h * sizeof(float));
    float* u = (float*)malloc(h * sizeof(float));
    float* y = (float*)malloc(h * sizeof(float));
    float* g = (float*)malloc(cs * sizeof(float));
    for (int l = 0; l < c->n_layer; l++) {
        const sz_layer* L = &m->layers[l];
        if (m->ple.ngram >= 2 && l == m->ple.layer) ple(s, r);
        hc_read(s, r, &L->hc_attn, 1, u, g);
        if (is_attention(c, l)) attention(s, l, u, y); else delta_net(s, l, u, y);
        hc_write(r, g, y, h, cs);
        hc_read(s, r, &L->hc_ffn, 1, u, g);
        szo_moe_layer ml;
        ml.hidden = L->moe.hidden; ml.n_expert = L->moe.n_expert; ml.top_k = L->moe.top_k; ml.expert_ff = L->moe.expert_ff;
        ml.shared_ff = L->moe.shared_ff; ml.expert_type = L->moe.expert_type; ml.shared_type = L->moe.shared_type;
        ml.router = (const float*)(uintptr_t)L->moe.router; ml.shared_router = (const float*)(uintptr_t)L->moe.shared_router;
        ml.gate = (const uint8_t*)(uintptr_t)L->moe.gate; ml.up = (const uint8_t*)(uintptr_t)L->moe.up; ml.down = (const uint8_t*)(uintptr_t)L->moe.down;
        ml.gate_stride = L->moe.gate_stride; ml.up_stride = L->moe.up_stride; ml.down_stride = L->moe.down_stride;
        ml.sh_gate = (const uint8_t*)(uintptr_t)L->moe.sh_gate; ml.sh_up = (const uint8_t*)(uintptr_t)L->moe.sh_up;
        ml.sh_down = (const uint8_t*)(uintptr_t)L->moe.sh_down;
        szo_moe(&ml, u, y, s->routes + (size_t)l * (size_t)c->n_expert_used, s->route_w + (size_t)l * (size_t)c->n_expert_used, NULL, s->threads);
        hc_write(r, g, y, h, cs);
    }
    hc_read(s, r, &m->output_hc, 0, u, NULL);
    if (final_u) memcpy(final_u, u, h * sizeof(float));
    if (logits) mv(&m->output, u, logits, s->threads);
    free(emb); free(r); free(u); free(y); free(g);
}

/* A pass over a draft tree, the slow and obvious way: every row steps its token on a COPY of the session as its parent left it, so
 * row j's logits are those of the sequence root .. j by construction.  No counterpart in the reference (its verify pass is a chain);
 * this is what the library's tree pass - tree mask, per-branch state forks, position by depth - must reproduce.  logits: [m][vocab].
 * keep_path / n_keep (n_keep > 0): afterwards the session becomes the one that read the kept path (row indices, root first); with
 * n_keep = 0 the session is left as it was. */
void szo_session_tree(szo_session* s, const uint32_t* ids, const int32_t* parents, int m, float* logits, const int32_t* keep_path, int n_keep) {
    size_t vocab = (size_t)s->m->cfg.vocab;
    szo_session** after = (szo_session**)calloc((size_t)m, sizeof(szo_session*));
    for (int j = 0; j < m; j++) {
        after[j] = szo_session_clone(parents[j] < 0 ? s : after[parents[j]]);
        szo_session_step(after[j], ids[j], logits + (size_t)j * vocab, NULL);
    }
    if (n_keep > 0) szo_session_assign(s, after[keep_path[n_keep - 1]]);
    for (int j = 0; j < m; j++) szo_session_free(after[j]);
    free(after);
}

/* Greedy acceptance down a tree: from the root, the best token (lowest id among equals, as the device's top-64 orders them) after
 * the current row must be the token of one of its children - the lowest row among equals -, never a drafted end-of-generation token.
 * Returns the rows kept; path[0 .. kept) the kept rows, *next the token after them. */
int szo_tree_accept_greedy(const float* logits, int vocab, const uint32_t* ids, const int32_t* parents, int m, int eog, int32_t* path, uint32_t* next) {
    int cur = 0, keep = 1;
    path[0] = 0;
    for (;;) {
        const float* row = logits + (size_t)cur * (size_t)vocab;
        int best = 0;
        for (int v = 1; v < vocab; v++) if (row[v] > row[best]) best = v;
        *next = (uint32_t)best;
        int nxt = -1;
        for (int c = cur + 1; c < m; c++)
            if (parents[c] == cur && (int)ids[c] == best && best != eog) { nxt = c; break; }
        if (nxt < 0) break;
        cur = nxt;
        path[keep++] = cur;
    }
    return keep;
}

/* Sampled acceptance down a draft tree by rejection sampling against the drafter's probabilities (no counterpart in the reference;
 * the library's sz_tree_accept_sampled states the rule).  tv / ti: [m][64] values and ids of every row's top-64. */
static int tree_candidates(const szo_sampler* sp, const float* tv, int ntop, double* p) {
    float max = tv[0];
    if (!isfinite(max)) { p[0] = 1.0; return 1; }
    float cut = max - 18.0f * sp->temperature;
    int n = 0;
    while (n < ntop && tv[n] >= cut) n++;
    int tk = sp->top_k < 1 ? 1 : sp->top_k;
    if (n > tk) n = tk;
    float inv_t = 1.0f / sp->temperature;
    double z = 0.0;
    for (int i = 0; i < n; i++) { p[i] = exp((double)((tv[i] - max) * inv_t)); z += p[i]; }
    for (int i = 0; i < n; i++) p[i] /= z;
    double floor_p = (double)sp->min_p * p[0];
    int keep = 0;
    while (keep < n && p[keep] >= floor_p) keep++;
    if (keep < 1) keep = 1;
    if (sp->top_p < 1.0f) {
        double acc = 0.0;
        int cnt = 0;
        for (int i = 0; i < keep; i++) { acc += p[i]; cnt++; if (acc >= (double)sp->top_p) break; }
        keep = cnt < 1 ? 1 : cnt;
    }
    double mass = 0.0;
    for (int i = 0; i < keep; i++) mass += p[i];
    for (int i = 0; i < keep; i++) p[i] /= mass;
    return keep;
}

int szo_tree_accept_sampled(const szo_sampler* sp, const float* tv, const uint32_t* ti, const uint32_t* ids, const int32_t* parents, int m,
                            const float* draft_prob, uint64_t pos, int eog, int32_t* path, uint32_t* next) {
    int cur = 0, keep = 1;
    path[0] = 0;
    for (;;) {
        double p[64];
        const float* v = tv + (size_t)cur * 64;
        const uint32_t* id = ti + (size_t)cur * 64;
        int n = tree_candidates(sp, v, 64, p);
        uint64_t P = pos + (uint64_t)(keep - 1);
        int tried = 0, taken = -1;
        for (int c = cur + 1; c < m; c++) {
            if (parents[c] != cur) continue;
            uint32_t x = ids[c];
            int at = -1;
            for (int i = 0; i < n; i++) if (id[i] == x) { at = i; break; }
            double px = at >= 0 ? p[at] : 0.0, q = (double)draft_prob[c];
            if (!(q > 1e-12)) q = 1e-12;
            if (q > 1.0) q = 1.0;
            double u = szo_uniform(sp->seed, 256 * P + 1 + (uint64_t)tried);
            tried++;
            if (eog >= 0 && x == (uint32_t)eog) continue;
            if (u * q < px) { taken = c; break; }
            if (at >= 0) {
                p[at] = px > q ? px - q : 0.0;
                double z = 0.0;
                for (int i = 0; i < n; i++) z += p[i];
                if (z > 0.0) { for (int i = 0; i < n; i++) p[i] /= z; }
                else { p[at] = 0.0; n = tree_candidates(sp, v, 64, p); }
            }
        }
        if (taken >= 0) { cur = taken; path[keep++] = cur; continue; }
        double u = szo_uniform(sp->seed, 256 * P);
        uint32_t tok = id[n - 1];
        for (int i = 0; i < n; i++) {
            if (u < p[i]) { tok = id[i]; break; }
            u -= p[i];
        }
        *next = tok;
        return keep;
    }
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* prompt lookup and the suffix drafter (engine.rs:823-1011)                                                         */

/* engine.rs:829-839: the (up to) k tokens after the latest earlier occurrence of the last n tokens, n from `lens` in order */
int szo_lookup(const uint32_t* hist, int n_hist, int k, const int* lens, int n_lens, uint32_t* out) {
    for (int li = 0; li < n_lens; li++) {
        int n = lens[li];
        if (k == 0 || n_hist <= n) break;
        const uint32_t* tail = hist + n_hist - n;
        for (int i = n_hist - n - 1; i >= 0; i--) {
            if (memcmp(hist + i, tail, (size_t)n * sizeof(uint32_t)) == 0) {
                int cnt = 0;
                for (int q = i + n; q < i + n + k && q < n_hist; q++) out[cnt++] = hist[q];
                return cnt;
            }
        }
    }
    return 0;
}

#define SUFFIX_WAYS 4
typedef struct { uint64_t key; uint32_t pos[SUFFIX_WAYS]; uint8_t n; } suffix_slot;
struct szo_drafter { size_t min_match, max_match; uint32_t* hist; size_t len, hcap; suffix_slot* table; size_t mask; };

static uint64_t sd_mix(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; return x ^ (x >> 33);
}
static uint64_t sd_key(const uint32_t* s, size_t end) {
    uint64_t a = s[end - 2], b = s[end - 1], c = s[end];
    return sd_mix((a * 0x9E3779B97F4A7C15ULL) ^ sd_mix(b + 0x632BE59BD9B4E019ULL) ^ (c << 1)) | 1;
}

szo_drafter* szo_drafter_new(int min_match, int max_match, int capacity_tokens) {
    szo_drafter* d = (szo_drafter*)calloc(1, sizeof(szo_drafter));
    d->min_match = (size_t)(min_match < 3 ? 3 : min_match);
    d->max_match = (size_t)max_match < d->min_match ? d->min_match : (size_t)max_match;
    size_t want = (size_t)(capacity_tokens < 1024 ? 1024 : capacity_tokens) * 2, cap = 1;
    while (cap < want) cap <<= 1;
    d->table = (suffix_slot*)calloc(cap, sizeof(suffix_slot));
    d->mask = cap - 1;
    d->hcap = 1024;
    d->hist = (uint32_t*)malloc(d->hcap * sizeof(uint32_t));
    return d;
}
void szo_drafter_free(szo_drafter* d) { if (d) { free(d->table); free(d->hist); free(d); } }

static void sd_append(szo_drafter* d, uint32_t t) {
    if (d->len == d->hcap) { d->hcap *= 2; d->hist = (uint32_t*)realloc(d->hist, d->hcap * sizeof(uint32_t)); }
    d->hist[d->len++] = t;
}

void szo_drafter_push(szo_drafter* d, uint32_t token) {
    sd_append(d, token);
    size_t end = d->len - 1;
    if (end < 2) return;
    uint64_t key = sd_key(d->hist, end);
    size_t i = (size_t)key & d->mask;
    for (size_t probe = 0; probe <= d->mask; probe++) {
        suffix_slot* s = &d->table[i];
        if (s->key == key || s->key == 0) {
            s->key = key;
            for (int w = SUFFIX_WAYS - 1; w >= 1; w--) s->pos[w] = s->pos[w - 1];
            s->pos[0] = (uint32_t)end;
            if (s->n < SUFFIX_WAYS) s->n++;
            return;
        }
        i = (i + 1) & d->mask;
    }
}

int szo_drafter_propose_with_min(const szo_drafter* d, int max_k, int min_match, uint32_t* out, int* match_len) {
    size_t min_m = (size_t)(min_match < 3 ? 3 : min_match), n = d->len;
    *match_len = 0;
    if (n < min_m + 1 || max_k == 0) return 0;
    size_t cur = n - 1;
    uint64_t key = sd_key(d->hist, cur);
    const suffix_slot* s = NULL;
    size_t i = (size_t)key & d->mask;
    for (size_t probe = 0; probe <= d->mask; probe++) {
        if (d->table[i].key == key) { s = &d->table[i]; break; }
        if (d->table[i].key == 0) break;
        i = (i + 1) & d->mask;
    }
    if (!s) return 0;
    size_t best_end = 0, best_len = 0;
    for (int w = 0; w < s->n; w++) {
        size_t p = s->pos[w];
        if (p >= cur) continue;
        size_t len = 0;
        while (len < d->max_match && len <= p && d->hist[p - len] == d->hist[cur - len]) len++;
        if (len > best_len) { best_len = len; best_end = p; }
    }
    if (best_len < min_m) return 0;
    int cnt = 0;
    for (size_t q = best_end + 1; q <= cur && cnt < max_k; q++) out[cnt++] = d->hist[q];
    *match_len = (int)best_len;
    return cnt;
}

int szo_drafter_propose(const szo_drafter* d, int max_k, uint32_t* out, int* match_len) {
    return szo_drafter_propose_with_min(d, max_k, (int)d->min_match, out, match_len);
}

/* engine.rs:996-1010: propose on hist + extra without touching the index */
int szo_drafter_propose_after(szo_drafter* d, const uint32_t* extra, int n_extra, int max_k, uint32_t* out, int* match_len) {
    if (n_extra == 0) return szo_drafter_propose(d, max_k, out, match_len);
    *match_len = 0;
    if (max_k == 0) return 0;
    size_t n0 = d->len;
    for (int i = 0; i < n_extra; i++) sd_append(d, extra[i]);
    int r = szo_drafter_propose(d, max_k, out, match_len);
    d->len = n0;
    return r;
}
int szo_drafter_len(const szo_drafter* d) { return (int)d->len; }

/* ---------------------------------------------------------------------------------------------------------------- */
/* the sampler (sampler.rs:83-210)                                                                                   */

static uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}
uint64_t szo_splitmix64(uint64_t x) { return splitmix64(x); }

double szo_uniform(uint64_t seed, uint64_t pos) {
    uint64_t bits = splitmix64(splitmix64(seed) ^ (pos * 0xD6E8FEB86659FD93ULL));
    return (double)(bits >> 11) / (double)(1ULL << 53);
}

/* sampler.rs:176-208: cand = (value, id) largest first, already cut to top_k */
static uint32_t sampler_draw(const szo_sampler* sp, const float* cv, const uint32_t* ci, int n, float max, uint64_t pos) {
    float inv_t = 1.0f / sp->temperature;
    double* probs = (double*)malloc((size_t)n * sizeof(double));
    double total = 0.0;
    for (int i = 0; i < n; i++) { probs[i] = exp((double)((cv[i] - max) * inv_t)); total += probs[i]; }
    for (int i = 0; i < n; i++) probs[i] /= total;
    double floor_p = (double)sp->min_p * probs[0];
    int keep = 0;
    while (keep < n && probs[keep] >= floor_p) keep++;
    if (keep < 1) keep = 1;
    if (sp->top_p < 1.0f) {
        double acc = 0.0;
        int cnt = 0;
        for (int i = 0; i < keep; i++) { acc += probs[i]; cnt++; if (acc >= (double)sp->top_p) break; }
        keep = cnt < 1 ? 1 : cnt;
    }
    double mass = 0.0;
    for (int i = 0; i < keep; i++) mass += probs[i];
    double u = szo_uniform(sp->seed, pos) * mass;
    uint32_t pick = ci[keep - 1];
    for (int i = 0; i < keep; i++) {
        if (u < probs[i]) { pick = ci[i]; break; }
        u -= probs[i];
    }
    free(probs);
    return pick;
}

/* sampler.rs:163-174 */
uint32_t szo_sample_top(const szo_sampler* sp, const float* tv, const uint32_t* ti, int ntop, uint64_t pos) {
    float max = tv[0];
    if (!isfinite(max)) return ti[0];
    float cut = max - 18.0f * sp->temperature;
    int n = 0;
    while (n < ntop && tv[n] >= cut) n++;
    int tk = sp->top_k < 1 ? 1 : sp->top_k;
    if (n > tk) n = tk;
    return sampler_draw(sp, tv, ti, n, max, pos);
}

typedef struct { float v; uint32_t i; } cand_t;
static int cand_cmp(const void* a, const void* b) {
    const cand_t *x = (const cand_t*)a, *y = (const cand_t*)b;
    if (x->v > y->v) return -1;
    if (x->v < y->v) return 1;
    return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0);
}

/* sampler.rs:112-157 without penalties (the top-64 path is only taken without them, sampler.rs:161) */
uint32_t szo_sample(const szo_sampler* sp, const float* logits, int vocab, uint64_t pos) {
    float max = -INFINITY;
    for (int i = 0; i < vocab; i++) max = logits[i] > max ? logits[i] : max;
    if (!isfinite(max)) {
        int best = 0;
        for (int i = 0; i < vocab; i++) if (logits[i] > logits[best]) best = i;
        return (uint32_t)best;
    }
    float cut = max - 18.0f * sp->temperature;
    cand_t* c = (cand_t*)malloc((size_t)vocab * sizeof(cand_t));
    int n = 0;
    for (int i = 0; i < vocab; i++) if (logits[i] >= cut) { c[n].v = logits[i]; c[n].i = (uint32_t)i; n++; }
    qsort(c, (size_t)n, sizeof(cand_t), cand_cmp);
    int tk = sp->top_k < 1 ? 1 : sp->top_k;
    if (n > tk) n = tk;
    float* cv = (float*)malloc((size_t)n * sizeof(float));
    uint32_t* ci = (uint32_t*)malloc((size_t)n * sizeof(uint32_t));
    for (int i = 0; i < n; i++) { cv[i] = c[i].v; ci[i] = c[i].i; }
    uint32_t r = sampler_draw(sp, cv, ci, n, max, pos);
    free(c); free(cv); free(ci);
    return r;
}

/* ---------------------------------------------------------------------------------------------------------------- */
/* the draft / verify / accept loop (engine.rs:2149-2454) for the suffix drafter alone: no neural drafter, policy off, so a
 * window is 1 + at most spec_k rows.  The CPU side has no batched verify: a pass is steps one after another from a snapshot,
 * and a rejection restores the snapshot and re-steps the kept rows - the result the reference's rollback is defined to give
 * (crates/shadowzero/tests/reference.rs:291-319).  Picks use the device's top-64 order (lowest id on ties), the path the
 * engine takes whenever speculation is on (engine.rs:2131,2204-2209). */
static uint32_t pick_token(const szo_gen_params* p, const float* logits, int vocab, uint64_t pos) {
    float tv[64];
    uint32_t ti[64];
    szo_top64(logits, vocab, tv, ti);
    if (p->greedy) return ti[0];
    return szo_sample_top(&p->sampler, tv, ti, 64, pos);
}

int szo_generate(szo_session* s, const uint32_t* prompt, int n_prompt, const szo_gen_params* p, uint32_t* out, int32_t* pass_log,
                 int pass_cap, szo_gen_stats* stats) {
    const int vocab = s->m->cfg.vocab;
    float* logits = (float*)malloc((size_t)vocab * sizeof(float));
    float* row = (float*)malloc((size_t)vocab * sizeof(float));
    memset(stats, 0, sizeof(*stats));
    for (int i = 0; i + 1 < n_prompt; i++) szo_session_step(s, prompt[i], NULL, NULL);
    szo_session_step(s, prompt[n_prompt - 1], logits, NULL);
    int lookup_min = p->lookup_min;
    szo_drafter* sd = szo_drafter_new(lookup_min < 3 ? 3 : lookup_min, 32, n_prompt + p->max_new + 64);
    uint32_t* hist = (uint32_t*)malloc((size_t)(n_prompt + p->max_new + 16) * sizeof(uint32_t));
    int n_hist = 0;
    for (int i = 0; i < n_prompt; i++) { hist[n_hist++] = prompt[i]; szo_drafter_push(sd, prompt[i]); }
    int n = 0;
    while (n < p->max_new) {
        uint32_t next = pick_token(p, logits, vocab, (uint64_t)n);
        if (p->eog_token >= 0 && next == (uint32_t)p->eog_token) break;
        out[n++] = next;
        hist[n_hist++] = next;
        szo_drafter_push(sd, next);
        if (p->spec_k <= 0) { szo_session_step(s, next, logits, NULL); continue; }
        int rem = p->max_new - n;
        int k_neural = p->spec_k < rem ? p->spec_k : rem;
        uint32_t draft[8];
        int match_len = 0, nd = 0;
        if (lookup_min > 0) nd = szo_drafter_propose(sd, k_neural, draft, &match_len);
        int by_lookup = nd >= 2;
        if (!by_lookup) {
            nd = szo_drafter_propose_with_min(sd, k_neural, 3, draft, &match_len);
            if (nd == 0) { static const int lens[2] = {3, 2}; nd = szo_lookup(hist, n_hist, k_neural, lens, 2, draft); }
        } else stats->lookup_passes++;
        if (nd == 0) { szo_session_step(s, next, logits, NULL); continue; }
        /* verify: outs[i] is what follows batch[..=i] */
        szo_session_step(s, next, logits, NULL);
        int keep = 1;
        for (int i = 0; i < nd; i++) {
            stats->pos_tried[i < 7 ? i : 7]++;
            uint32_t want = pick_token(p, logits, vocab, (uint64_t)n);
            if (want != draft[i] || (p->eog_token >= 0 && draft[i] == (uint32_t)p->eog_token)) break;
            out[n++] = draft[i];
            keep++;
            stats->pos_right[i < 7 ? i : 7]++;
            hist[n_hist++] = draft[i];
            szo_drafter_push(sd, draft[i]);
            szo_session_step(s, draft[i], logits, NULL); /* the row after this accepted draft */
        }
        /* stepping only the kept rows is the rolled-back state: nothing to undo on this side */
        stats->passes++;
        stats->drafted += nd;
        stats->accepted += keep - 1;
        if (pass_log && stats->passes <= pass_cap) { pass_log[2 * (stats->passes - 1)] = nd; pass_log[2 * (stats->passes - 1) + 1] = keep - 1; }
    }
    stats->n_tokens = n;
    (void)row;
    szo_drafter_free(sd); free(hist); free(logits); free(row);
    return n;
}
