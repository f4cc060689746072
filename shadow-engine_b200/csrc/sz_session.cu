// The verify surface of the GPU session: prefill, verify (1..8 rows in one pass), acceptance, commit / rollback.
// Mirrors GpuSession::{step_batch_verify_top, rollback, note_verify, capacity, tokens} of the reference
// (crates/shadowzero-cuda/src/session.rs:6061-6107, 6217-6276) for a model held entirely in HBM.
//
// State that a rejected draft must not touch is double-buffered instead of snapshotted: a pass reads the DeltaNet states and
// conv rows of buffer `cur` and writes those after all m rows into buffer `cur ^ 1`; a commit of fewer rows re-runs the (cheap)
// recurrences for the kept rows from the pass's saved inputs - the reference's replay (session.rs:6245-6268) - into `cur ^ 1`,
// then the buffers swap.  The KV cache is append-only: rejected positions are overwritten by the next pass.
#include "sz_session_kernels.cuh"
#include "sz_indexer.cuh"
#include "sz_ple.cuh"

#include <cmath>
#include <map>
#include <new>
#include <stdlib.h>
#include <string.h>
#include <vector>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>

struct SzLayerBuf {
    int delta_index;   // index among DeltaNet layers, or -1
    int attn_index;    // index among attention layers, or -1
};

int sz_ep_graph_refs(int delta);      // sz_ep.cu: recorded passes that hold the communicator
int sz_ep_p2p_graph_refs(int delta);  // ... that hold the addresses of the attached peer-memory exchange
int sz_ep_generation(void);           // changes whenever the exchange set-up does
extern "C" int sz_ep_world(void);
extern "C" int sz_ep_p2p_world(void);

struct sz_session {
    sz_model model;
    std::vector<sz_layer> layers;
    std::vector<SzLayerBuf> lb;
    int ctx, flags, n_delta, n_attn;
    int len;          // committed positions
    int cur;          // which state buffer is current
    int last_m;       // rows of the last pass (0: none pending)
    int want_routes;
    // device memory (all inside the caller's block)
    u8* base;
    int64_t bytes;
    float *r, *rn, *hdown, *mix, *u, *g, *y;
    float* r2;            // the second residual buffer of the fused hyper-connection read (reads ping-pong between r and r2)
    long long* hc_acc;    // [3][8][SZ_HC_ACC_ROWS] fixed-point accumulators of the fused read
    int64_t hc_acc_stride;   // entries from one of the three to the next (a batched step points the session into buffers of the batch)
    double* rope_den;     // [rope_dims / 2]: theta^(2 i / rope_dims), computed on the host as the CPU reference computes it
    int hc_fast;          // every hyper-connection of the model fits the fused kernels
    int hc_n;             // reads launched so far in the pass being built (buffer parities are static per launch)
    float *d_xin, *d_z, *d_b, *d_a, *d_xc, *d_beta, *d_decay, *d_og;   // per-layer saved: xin, xc, beta, decay [n_delta][8][...]
    float *S[2], *conv[2];
    float *a_qg, *a_k, *a_v, *a_q, *a_gate, *a_o, *a_part;
    u8 *kc, *vc;
    float* logits;
    u64* tk_tmp;
    u32* top;
    int32_t *ids, *res, *routes, *state;   // state: {committed positions, current state buffer} as the kernels see them
    double* route_w;
    u8* moe_scratch;
    int64_t moe_scratch_bytes;
    int attn_splits, attn_splits2;
    // host staging (pinned, so that a captured graph re-reads it at every launch)
    int32_t* h_pin;   // [0..8): ids of the pass, [8]: keep of a host-decided commit, [10..12]: error words read back, [13..14]: {kept, next}, [16..24): SzSampleArgs
    sz_sampler samp = {};   // sz_session_set_sampler
    int has_samp = 0;
    int tree_pass = 0;      // the pass being built / pending is a tree pass (sz_session_verify_tree)
    float* fork = nullptr;  // [v heads][8][d * d]: recurrent states a tree pass branches off
    // the per-layer embedding (model.ple.ngram >= 2): see sz_ple.cuh
    float *p_e = nullptr, *p_key = nullptr, *p_val = nullptr, *p_gv = nullptr, *p_gvn = nullptr, *p_hist = nullptr;
    int32_t* p_tail = nullptr;
    int64_t p_hist_bytes = 0;
    // the sparse indexer (model.cfg.idx_heads > 0): see sz_indexer.cuh
    float *i_q = nullptr, *i_k = nullptr, *i_qn = nullptr, *i_raw = nullptr, *i_blocks = nullptr, *i_scores = nullptr;
    u32 *i_sel = nullptr, *i_trace = nullptr;
    int32_t *i_list = nullptr, *i_count = nullptr;   // [8][ctx blocks]: each row's ascending list of position groups; [8]: how many
    int64_t i_raw_layer = 0, i_blocks_layer = 0;
    int i_ctx_blocks = 0, i_words = 0;
    int pending_committed;  // the pending pass was already committed on the device (acceptance modes GREEDY / ALL / SAMPLED)
    int device_keep;        // rows the device kept in that pass: known at launch for ALL, read by sz_session_result otherwise (-1: not read yet)
    int inflight;           // a pass was launched and the stream not synchronised since: the id staging buffer may still be read
    int use_graphs;
    std::map<int, cudaGraphExec_t> graphs;
    int ep_graphs = 0;      // how many of them recorded a collective of the expert-parallel communicator
    int p2p_graphs = 0;     // how many of them recorded kernels that address the attached peer-memory exchange
    int graph_gen = 0;      // the exchange set-up (sz_ep_generation) the graphs were recorded under
    sz_head head = {};      // rows > 0: output.weight is an EXL3 blob and the head runs through sz_head_top
    void drop_graphs() {
        for (auto& kv : graphs) cudaGraphExecDestroy(kv.second);
        graphs.clear();
        sz_ep_graph_refs(-ep_graphs);
        sz_ep_p2p_graph_refs(-p2p_graphs);
        ep_graphs = p2p_graphs = 0;
    }
    ~sz_session() {
        drop_graphs();
        if (h_pin) cudaFreeHost(h_pin);
    }
};

static int sz_is_attn(const sz_model_config& c, int l) { return l % c.attn_interval == c.attn_interval - 1; }

struct SzSessLayout {
    int64_t r, r2, hc_acc, rope, rn, hdown, mix, u, g, y, d_xin, d_z, d_b, d_a, d_xc, d_beta, d_decay, d_og, S0, S1, conv0, conv1, a_qg, a_k, a_v, a_q, a_gate,
        a_o, a_part, kc, vc, logits, tk_tmp, top, ids, res, state, routes, route_w, moe, head_q2, head_sc, head_work, fork, i_q, i_k, i_qn, i_raw, i_blocks, i_scores, i_sel, i_list, i_count, i_trace, p_e, p_key, p_val, p_gv, p_gvn, p_hist, p_tail, total;
    int64_t p_hist_bytes;
    int64_t i_raw_layer, i_blocks_layer;   // bytes of one attention layer's raw-key and pooled-key caches
    int i_ctx_blocks, i_words;
    int64_t moe_bytes, S_bytes, conv_bytes, kv_bytes, head_work_bytes;
    int splits, splits2;
};

// output.weight as an EXL3 blob: the head is sz_head_top's (dense, or screened by the 2-bit proxy with SZ_HEAD_PROXY).
static bool sz_head_is_exl3(const sz_model* m) { return m->output.type > 1020 && m->output.type <= 1028; }
static int sz_head_describe(const sz_model* m, int flags, sz_head* h) {
    *h = sz_head();
    if (!sz_head_is_exl3(m)) {
        if (flags & SZ_HEAD_PROXY) return sz_fail(SZ_E_ARG, "SZ_HEAD_PROXY needs an EXL3 output.weight (type %d given)", m->output.type);
        return SZ_OK;
    }
    h->rows = m->cfg.vocab; h->cols = m->cfg.hidden; h->bits = m->output.type - 1020;
    h->weight = m->output.data;
    if (flags & SZ_HEAD_PROXY) {
        const char* e = getenv("SZ_HEAD_KBLK");  // blocks kept a row (the reference's SHADOWZERO_HEAD_KBLK, session.rs:2655)
        h->k_blk = e && atoi(e) > 0 ? atoi(e) : 128;
    }
    return SZ_OK;
}

static int64_t up256(int64_t v) { return (v + 255) & ~(int64_t)255; }

static int sz_sess_layout(const sz_model* m, int ctx, int flags, SzSessLayout* L) {
    const sz_model_config& c = m->cfg;
    const int64_t M = SZ_MAX_VERIFY, H = c.hidden, C = c.streams, CH = C * H;
    int n_delta = 0, n_attn = 0;
    for (int l = 0; l < c.n_layer; l++) (sz_is_attn(c, l) ? n_attn : n_delta)++;
    const int64_t kd = (int64_t)c.ssm_k_heads * c.ssm_head_dim, vd = (int64_t)c.ssm_v_heads * c.ssm_head_dim, ch = 2 * kd + vd, vh = c.ssm_v_heads;
    const int64_t qd = (int64_t)c.n_head * c.head_dim, kvd = (int64_t)c.n_kv_head * c.head_dim;
    int64_t o = 0;
    auto take = [&](int64_t bytes) { int64_t at = o; o = up256(o + bytes); return at; };
    L->r = take(4 * M * CH); L->r2 = take(4 * M * CH); L->hc_acc = take(8 * 3 * M * SZ_HC_ACC_ROWS); L->rope = take(8 * (int64_t)(c.rope_dims > 0 ? c.rope_dims / 2 : 1)); L->rn = take(4 * M * CH); L->hdown = take(4 * M * c.hc_rank); L->mix = take(4 * M * CH);
    L->u = take(4 * M * H); L->g = take(4 * M * C); L->y = take(4 * M * H);
    const int64_t nd = n_delta > 0 ? n_delta : 1;
    L->d_xin = take(4 * nd * M * ch); L->d_xc = take(4 * nd * M * ch); L->d_beta = take(4 * nd * M * vh); L->d_decay = take(4 * nd * M * vh);
    L->d_z = take(4 * M * vd); L->d_b = take(4 * M * vh); L->d_a = take(4 * M * vh); L->d_og = take(4 * M * vd);
    L->S_bytes = 4 * nd * vh * c.ssm_head_dim * c.ssm_head_dim;
    L->conv_bytes = 4 * nd * (c.conv_k - 1) * ch;
    L->S0 = take(L->S_bytes); L->S1 = take(L->S_bytes); L->conv0 = take(L->conv_bytes); L->conv1 = take(L->conv_bytes);
    L->a_qg = take(4 * M * 2 * qd); L->a_k = take(4 * M * kvd); L->a_v = take(4 * M * kvd); L->a_q = take(4 * M * qd);
    L->a_gate = take(4 * M * qd); L->a_o = take(4 * M * qd);
    // enough (head, row, split) blocks to fill the GPU twice over, at least 256 positions a split
    int splits = 1;
    if (c.n_head > 0) {
        splits = (int)((2 * 148 + c.n_head * 4 - 1) / (c.n_head * 4));
        const int by_len = (ctx + 255) / 256;
        if (splits > by_len) splits = by_len;
        if (splits < 1) splits = 1;
    }
    L->splits = splits;
    // the grouped kernel: one block per (kv head, split), about one block a multiprocessor
    int splits2 = 148 / (c.n_kv_head > 0 ? c.n_kv_head : 1);
    if (splits2 > (ctx + 255) / 256) splits2 = (ctx + 255) / 256;
    if (splits2 < 1) splits2 = 1;
    L->splits2 = splits2;
    // (with few queries a head the grouped kernel runs two blocks a multiprocessor and takes twice the splits)
    const int smax = splits > 2 * splits2 ? splits : 2 * splits2;
    L->a_part = take(4 * M * c.n_head * smax * (c.head_dim + 2));
    const int64_t hb = (flags & SZ_KV_Q8) ? (c.head_dim + (((c.head_dim >> 5) * 2 + 15) & ~15)) : 4 * (int64_t)c.head_dim;
    L->kv_bytes = (int64_t)(n_attn > 0 ? n_attn : 1) * ctx * c.n_kv_head * hb;
    L->kc = take(L->kv_bytes); L->vc = take(L->kv_bytes);
    L->logits = take(4 * M * (int64_t)c.vocab);
    const int64_t nb = ((int64_t)c.vocab + SZ_TK_N - 1) / SZ_TK_N;
    L->tk_tmp = take(8 * M * nb * 64); L->top = take(4 * M * 128);
    L->ids = take(512);  // the rows' tokens, then (word 16) the sampler block of a sampled pass, then (word 32) the tables of a tree pass
    L->fork = take(4 * (int64_t)vh * M * c.ssm_head_dim * c.ssm_head_dim);
    // the sparse indexer: projections of the pass, raw and pooled key caches of every attention layer, scores, per-row block sets,
    // the merged list.  Sized by the smallest block (the most blocks) any layer uses.
    L->i_ctx_blocks = 0; L->i_words = 0; L->i_raw_layer = 0; L->i_blocks_layer = 0;
    if (c.idx_heads > 0) {
        int rmin = 1 << 30;
        for (int l = 0; l < c.n_layer; l++)
            if (sz_is_attn(c, l)) { const int r = m->layers[l].idx_ratio > 0 ? m->layers[l].idx_ratio : 1; rmin = r < rmin ? r : rmin; }
        if (rmin == 1 << 30) rmin = 1;
        const int64_t id = c.idx_dim, ih = c.idx_heads, na = n_attn > 0 ? n_attn : 1;
        L->i_ctx_blocks = ctx / rmin + 1;
        L->i_words = (L->i_ctx_blocks + 31) / 32;
        L->i_raw_layer = up256(4 * (int64_t)ctx * id);
        L->i_blocks_layer = up256(4 * (int64_t)L->i_ctx_blocks * id);
        L->i_q = take(4 * M * ih * id); L->i_k = take(4 * M * id); L->i_qn = take(4 * M * ih * id);
        L->i_raw = take(na * L->i_raw_layer); L->i_blocks = take(na * L->i_blocks_layer);
        L->i_scores = take(4 * M * (int64_t)L->i_ctx_blocks); L->i_sel = take(4 * M * (int64_t)L->i_words);
        L->i_list = take(4 * M * (int64_t)L->i_ctx_blocks); L->i_count = take(64);
        L->i_trace = take(4 * na * M * (int64_t)L->i_words);
    }
    L->p_hist_bytes = 0;
    if (m->ple.ngram >= 2) {   // the per-layer embedding: the pass's rows and the carried history (two copies, as the DeltaNet's conv rows)
        L->p_hist_bytes = up256(4 * (int64_t)(m->ple.conv_k - 1) * m->ple.ngram * CH);
        L->p_e = take(4 * M * H); L->p_key = take(4 * M * CH); L->p_val = take(4 * M * H); L->p_gv = take(4 * M * CH); L->p_gvn = take(4 * M * CH);
        L->p_hist = take(2 * L->p_hist_bytes); L->p_tail = take(64);
    }
    L->res = take(64); L->state = take(64);
    L->routes = take(4 * (int64_t)c.n_layer * M * SZ_MAX_TOPK); L->route_w = take(8 * (int64_t)c.n_layer * M * SZ_MAX_TOPK);
    int64_t moe_bytes = 0;
    for (int l = 0; l < c.n_layer; l++) {
        int64_t b = 0;
        const int rc = sz_moe_scratch_bytes(&m->layers[l].moe, SZ_MAX_VERIFY, &b);
        if (rc) return rc;
        if (b > moe_bytes) moe_bytes = b;
    }
    L->moe_bytes = moe_bytes;
    L->moe = take(moe_bytes);
    L->head_q2 = L->head_sc = L->head_work = 0;
    L->head_work_bytes = 0;
    sz_head hd;
    int hrc = sz_head_describe(m, flags, &hd);
    if (hrc) return hrc;
    if (hd.rows > 0) {
        if ((hrc = sz_head_work_bytes(hd.rows, hd.cols, hd.k_blk, &L->head_work_bytes))) return hrc;
        L->head_work = take(L->head_work_bytes);
        if (hd.k_blk > 0) {
            int64_t q2 = 0, sc = 0;
            if ((hrc = sz_head_proxy_bytes(hd.rows, hd.cols, &q2, &sc))) return hrc;
            L->head_q2 = take(q2);
            L->head_sc = take(sc);
        }
    }
    L->total = o;
    return SZ_OK;
}

int sz_dense_check(const sz_tensor* t, const char* what, int64_t rows, int64_t cols) {
    if (!t->data || t->rows != rows || t->cols != cols)
        return sz_fail(SZ_E_ARG, "%s: expected a [%lld -> %lld] tensor, got [%lld -> %lld]%s", what, (long long)cols, (long long)rows,
                       (long long)t->cols, (long long)t->rows, t->data ? "" : " (null)");
    switch (t->type) {
        case SZ_TYPE_F32: case SZ_TYPE_F16: case SZ_TYPE_BF16: if (cols % 4) return sz_fail(SZ_E_ARG, "%s: %lld columns are not a multiple of 4", what, (long long)cols); break;
        case SZ_TYPE_Q8_0: if (cols % 32) return sz_fail(SZ_E_ARG, "%s: Q8_0 rows of %lld weights", what, (long long)cols); break;
        case SZ_TYPE_IQ3_S: if (cols % 256) return sz_fail(SZ_E_ARG, "%s: IQ3_S rows of %lld weights", what, (long long)cols); break;
        default: return sz_fail(SZ_E_TYPE, "%s: no dense kernel for tensor type %d", what, t->type);
    }
    if (t->data & 15) return sz_fail(SZ_E_ARG, "%s: the tensor must start on a 16-byte boundary", what);
    return SZ_OK;
}

static int sz_f32_check(const sz_tensor* t, const char* what, int64_t n) {
    if (!t->data || t->type != SZ_TYPE_F32 || t->rows * t->cols != n || (t->data & 15))
        return sz_fail(SZ_E_ARG, "%s: expected %lld F32 values, 16-byte aligned", what, (long long)n);
    return SZ_OK;
}

static int sz_model_check(const sz_model* m) {
    if (!m || !m->layers) return sz_fail(SZ_E_ARG, "null model");
    const sz_model_config& c = m->cfg;
    if (c.n_layer < 1 || c.hidden < 128 || c.hidden % 128 || c.streams < 1 || c.streams > 8 || c.hc_rank < 4 || c.hc_rank % 4 || c.vocab < 64)
        return sz_fail(SZ_E_ARG, "bad model shape (layers %d, hidden %d, streams %d, rank %d, vocab %d)", c.n_layer, c.hidden, c.streams, c.hc_rank, c.vocab);
    if (c.vocab > 64 * SZ_TK_N) return sz_fail(SZ_E_ARG, "vocab %d exceeds %d", c.vocab, 64 * SZ_TK_N);
    if (c.attn_interval < 1) return sz_fail(SZ_E_ARG, "attn_interval %d", c.attn_interval);
    if (!(c.head_dim == 64 || c.head_dim == 128 || c.head_dim == 256) || c.n_head < 1 || c.n_kv_head < 1 || c.n_head % c.n_kv_head || c.rope_dims % 2 ||
        c.rope_dims > c.head_dim)
        return sz_fail(SZ_E_ARG, "attention shape (heads %d / %d, head_dim %d, rope %d): head_dim must be 64, 128 or 256", c.n_head, c.n_kv_head, c.head_dim, c.rope_dims);
    if (!(c.ssm_head_dim == 64 || c.ssm_head_dim == 128) || c.ssm_k_heads < 1 || c.ssm_v_heads % c.ssm_k_heads || c.conv_k < 2 || c.conv_k > 8)
        return sz_fail(SZ_E_ARG, "DeltaNet shape (heads %d / %d, dim %d, conv %d): head dim must be 64 or 128", c.ssm_k_heads, c.ssm_v_heads, c.ssm_head_dim, c.conv_k);
    const int64_t H = c.hidden, CH = (int64_t)c.streams * H;
    const int64_t kd = (int64_t)c.ssm_k_heads * c.ssm_head_dim, vd = (int64_t)c.ssm_v_heads * c.ssm_head_dim, ch = 2 * kd + vd;
    const int64_t qd = (int64_t)c.n_head * c.head_dim, kvd = (int64_t)c.n_kv_head * c.head_dim;
    if (c.idx_heads < 0 || c.idx_heads > 8 || (c.idx_heads > 0 && (c.idx_dim < 16 || c.idx_dim > SZ_IDX_MAX_DIM || c.idx_dim % 4 || c.idx_dim < c.rope_dims || c.idx_budget < 1)))
        return sz_fail(SZ_E_ARG, "indexer shape (heads %d, width %d, budget %d): up to 8 heads of 16..%d, at least the rotated dimensions", c.idx_heads, c.idx_dim, c.idx_budget, SZ_IDX_MAX_DIM);
    int rc;
    if (m->ple.ngram >= 2) {
        const sz_ple& p = m->ple;
        const int heads = (p.ngram - 1) * p.heads_per_ngram;
        if (p.ngram > SZ_PLE_MAX_NGRAM || heads < 1 || heads > SZ_PLE_MAX_HEADS || p.head_dim < 4 || p.head_dim % 4 || (int64_t)heads * p.head_dim != H ||
            p.layer < 0 || p.layer >= c.n_layer || p.conv_k < 2 || p.conv_k > 8)
            return sz_fail(SZ_E_ARG, "per-layer embedding shape (layer %d, n-grams to %d, %d heads each of %d, conv %d): the heads' rows side by side are one embedding of %d",
                           p.layer, p.ngram, p.heads_per_ngram, p.head_dim, p.conv_k, (int)H);
        for (int i = 0; i < heads; i++)
            if (p.vocab[i] < 1 || p.offsets[i] < 0 || p.offsets[i] + p.vocab[i] > p.table.rows) return sz_fail(SZ_E_ARG, "per-layer embedding: head %d reaches past the table", i);
        if ((rc = sz_dense_check(&p.table, "per_layer_token_embd", p.table.rows, p.head_dim))) return rc;
        if ((rc = sz_dense_check(&p.key, "ple_key", CH, H)) || (rc = sz_dense_check(&p.value, "ple_value", H, H))) return rc;
        if ((rc = sz_f32_check(&p.norm_key, "ple_norm_key", CH)) || (rc = sz_f32_check(&p.norm_query, "ple_norm_query", CH)) ||
            (rc = sz_f32_check(&p.norm_conv, "ple_norm_conv", CH)) || (rc = sz_f32_check(&p.conv1d, "ple_conv1d", CH * p.conv_k)))
            return rc;
    }
    auto hc = [&](const sz_hc& h, const char* what, bool inject) -> int {
        int r2;
        if ((r2 = sz_f32_check(&h.norm, what, CH))) return r2;
        if ((r2 = sz_dense_check(&h.down, what, c.hc_rank, CH))) return r2;
        if ((r2 = sz_dense_check(&h.up, what, CH, c.hc_rank))) return r2;
        if (inject && (r2 = sz_dense_check(&h.inject, what, c.streams, CH))) return r2;
        return SZ_OK;
    };
    if ((rc = sz_dense_check(&m->token_embd, "token_embd", c.vocab, H))) return rc;
    if (sz_head_is_exl3(m)) {
        if (!m->output.data || m->output.rows != c.vocab || m->output.cols != H) return sz_fail(SZ_E_ARG, "output: expected a [%d -> %d] tensor", H, (int)c.vocab);
    } else if ((rc = sz_dense_check(&m->output, "output", c.vocab, H))) return rc;
    if ((rc = hc(m->output_hc, "output_hc", false))) return rc;
    for (int l = 0; l < c.n_layer; l++) {
        const sz_layer& L = m->layers[l];
        if ((rc = hc(L.hc_attn, "hc_attn", true))) return rc;
        if ((rc = hc(L.hc_ffn, "hc_ffn", true))) return rc;
        if (sz_is_attn(c, l)) {
            if ((rc = sz_dense_check(&L.attn_q, "attn_q", 2 * qd, H))) return rc;
            if ((rc = sz_dense_check(&L.attn_k, "attn_k", kvd, H))) return rc;
            if ((rc = sz_dense_check(&L.attn_v, "attn_v", kvd, H))) return rc;
            if ((rc = sz_dense_check(&L.attn_output, "attn_output", H, qd))) return rc;
            if ((rc = sz_f32_check(&L.attn_q_norm, "attn_q_norm", c.head_dim))) return rc;
            if ((rc = sz_f32_check(&L.attn_k_norm, "attn_k_norm", c.head_dim))) return rc;
            if (c.idx_heads > 0) {
                if ((rc = sz_dense_check(&L.idx_q, "indexer.q_proj", (int64_t)c.idx_heads * c.idx_dim, H))) return rc;
                if ((rc = sz_dense_check(&L.idx_k, "indexer.k_proj", c.idx_dim, H))) return rc;
                if ((rc = sz_f32_check(&L.idx_q_norm, "indexer.q_norm", c.idx_dim))) return rc;
                if ((rc = sz_f32_check(&L.idx_k_norm, "indexer.k_norm", c.idx_dim))) return rc;
                const int ratio = L.idx_ratio > 0 ? L.idx_ratio : 1;
                if (ratio > SZ_AT_T || SZ_AT_T % ratio) return sz_fail(SZ_E_ARG, "layer %d: %d positions a block of the indexer (a power of two up to %d)", l, ratio, SZ_AT_T);
            }
        } else {
            if ((rc = sz_dense_check(&L.attn_qkv, "attn_qkv", ch, H))) return rc;
            if ((rc = sz_dense_check(&L.attn_gate, "attn_gate", vd, H))) return rc;
            if ((rc = sz_dense_check(&L.ssm_beta, "ssm_beta", c.ssm_v_heads, H))) return rc;
            if ((rc = sz_dense_check(&L.ssm_alpha, "ssm_alpha", c.ssm_v_heads, H))) return rc;
            if ((rc = sz_dense_check(&L.ssm_out, "ssm_out", H, vd))) return rc;
            if ((rc = sz_f32_check(&L.ssm_conv1d, "ssm_conv1d", ch * c.conv_k))) return rc;
            if ((rc = sz_f32_check(&L.ssm_a, "ssm_a", c.ssm_v_heads))) return rc;
            if ((rc = sz_f32_check(&L.ssm_dt_bias, "ssm_dt.bias", c.ssm_v_heads))) return rc;
            if ((rc = sz_f32_check(&L.ssm_norm, "ssm_norm", c.ssm_head_dim))) return rc;
        }
        if (L.moe.hidden != c.hidden || L.moe.n_expert != c.n_expert || L.moe.top_k != c.n_expert_used)
            return sz_fail(SZ_E_ARG, "layer %d: the MoE description does not match the model shape", l);
    }
    return SZ_OK;
}

extern "C" int sz_session_bytes(const sz_model* m, int ctx, int flags, int64_t* bytes) {
    int rc = sz_model_check(m);
    if (rc) return rc;
    if (ctx < 8 || !bytes) return sz_fail(SZ_E_ARG, "sz_session_bytes: ctx = %d", ctx);
    SzSessLayout L;
    if ((rc = sz_sess_layout(m, ctx, flags, &L))) return rc;
    *bytes = L.total;
    return SZ_OK;
}

extern "C" int sz_session_reset(sz_session* s, uint64_t stream) {
    if (!s) return sz_fail(SZ_E_ARG, "null session");
    SzSessLayout L;
    int rc = sz_sess_layout(&s->model, s->ctx, s->flags, &L);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    SZ_CUDA(cudaMemsetAsync(s->S[0], 0, L.S_bytes, st));
    SZ_CUDA(cudaMemsetAsync(s->S[1], 0, L.S_bytes, st));
    SZ_CUDA(cudaMemsetAsync(s->conv[0], 0, L.conv_bytes, st));
    SZ_CUDA(cudaMemsetAsync(s->conv[1], 0, L.conv_bytes, st));
    SZ_CUDA(cudaMemsetAsync(s->state, 0, 64, st));
    SZ_CUDA(cudaMemsetAsync(s->res, 0, 64, st));
    if (s->i_count) SZ_CUDA(cudaMemsetAsync(s->i_count, 0, 64, st));
    if (s->p_hist) {   // no history; every position before the sequence reads as the end-of-text token (forward.rs:1181-1184)
        SZ_CUDA(cudaMemsetAsync(s->p_hist, 0, (size_t)(2 * s->p_hist_bytes), st));
        if (s->inflight) { SZ_CUDA(cudaStreamSynchronize(st)); s->inflight = 0; }
        for (int i = 0; i < 16; i++) s->h_pin[64 + i] = s->model.ple.eos;
        SZ_CUDA(cudaMemcpyAsync(s->p_tail, s->h_pin + 64, 64, cudaMemcpyHostToDevice, st));
        SZ_CUDA(cudaStreamSynchronize(st));
    }
    if ((rc = sz_moe_scratch_init((uint64_t)s->moe_scratch, s->moe_scratch_bytes, stream))) return rc;
    s->len = 0; s->cur = 0; s->last_m = 0; s->pending_committed = 0; s->inflight = 0;
    return SZ_OK;
}

static bool sz_hc_fits(const sz_model_config& c, const sz_hc& hc, bool inject);

static int sz_sm_count_session() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    }
    return n;
}

extern "C" int sz_session_create(const sz_model* m, int ctx, int flags, uint64_t mem, int64_t bytes, uint64_t stream, sz_session** out) {
    int rc = sz_model_check(m);
    if (rc) return rc;
    if (!out || !mem || (mem & 255)) return sz_fail(SZ_E_ARG, "sz_session_create: memory must be 256-byte aligned");
    if (m->cfg.idx_heads > 0 && (!(flags & SZ_KV_Q8) || m->cfg.n_head / m->cfg.n_kv_head * SZ_MAX_VERIFY > 64))
        return sz_fail(SZ_E_ARG, "sz_session_create: the sparse indexer runs on the packed cache (SZ_KV_Q8) with at most 8 query heads a KV head");
    SzSessLayout L;
    if ((rc = sz_sess_layout(m, ctx, flags, &L))) return rc;
    if (bytes < L.total) return sz_fail(SZ_E_SCRATCH, "sz_session_create: %lld bytes given, %lld needed", (long long)bytes, (long long)L.total);
    sz_session* s = new (std::nothrow) sz_session();
    if (!s) return sz_fail(SZ_E_ARG, "out of host memory");
    s->model = *m;
    s->layers.assign(m->layers, m->layers + m->cfg.n_layer);
    s->model.layers = s->layers.data();
    s->ctx = ctx; s->flags = flags; s->want_routes = 0;
    s->h_pin = nullptr;
    if (cudaHostAlloc((void**)&s->h_pin, 512, cudaHostAllocDefault) != cudaSuccess) { delete s; return sz_fail(SZ_E_CUDA, "cudaHostAlloc of the id staging buffer failed"); }
    memset(s->h_pin, 0, 512);
    {
        const char* e = getenv("SZ_SESSION_GRAPHS");  // A/B switch: 0 = launch every kernel eagerly
        s->use_graphs = !(e && atoi(e) == 0);
    }
    {
        const char* e = getenv("SZ_GENERIC_KERNELS");
        bool fast = !(e && atoi(e) != 0) && sz_hc_fits(m->cfg, m->output_hc, false);
        for (int l = 0; l < m->cfg.n_layer && fast; l++) fast = sz_hc_fits(m->cfg, s->layers[l].hc_attn, true) && sz_hc_fits(m->cfg, s->layers[l].hc_ffn, true);
        s->hc_fast = fast ? 1 : 0;
        s->hc_n = 0;
    }
    s->lb.resize(m->cfg.n_layer);
    s->n_delta = s->n_attn = 0;
    for (int l = 0; l < m->cfg.n_layer; l++) {
        const bool at = sz_is_attn(m->cfg, l);
        s->lb[l].delta_index = at ? -1 : s->n_delta++;
        s->lb[l].attn_index = at ? s->n_attn++ : -1;
    }
    u8* b = (u8*)mem;
    s->base = b; s->bytes = bytes;
    s->r = (float*)(b + L.r); s->r2 = (float*)(b + L.r2); s->hc_acc = (long long*)(b + L.hc_acc); s->hc_acc_stride = (int64_t)SZ_MAX_VERIFY * SZ_HC_ACC_ROWS; s->rope_den = (double*)(b + L.rope); s->rn = (float*)(b + L.rn); s->hdown = (float*)(b + L.hdown); s->mix = (float*)(b + L.mix);
    s->u = (float*)(b + L.u); s->g = (float*)(b + L.g); s->y = (float*)(b + L.y);
    s->d_xin = (float*)(b + L.d_xin); s->d_z = (float*)(b + L.d_z); s->d_b = (float*)(b + L.d_b); s->d_a = (float*)(b + L.d_a);
    s->d_xc = (float*)(b + L.d_xc); s->d_beta = (float*)(b + L.d_beta); s->d_decay = (float*)(b + L.d_decay); s->d_og = (float*)(b + L.d_og);
    s->S[0] = (float*)(b + L.S0); s->S[1] = (float*)(b + L.S1); s->conv[0] = (float*)(b + L.conv0); s->conv[1] = (float*)(b + L.conv1);
    s->a_qg = (float*)(b + L.a_qg); s->a_k = (float*)(b + L.a_k); s->a_v = (float*)(b + L.a_v); s->a_q = (float*)(b + L.a_q);
    s->a_gate = (float*)(b + L.a_gate); s->a_o = (float*)(b + L.a_o); s->a_part = (float*)(b + L.a_part);
    s->kc = b + L.kc; s->vc = b + L.vc;
    s->logits = (float*)(b + L.logits); s->tk_tmp = (u64*)(b + L.tk_tmp); s->top = (u32*)(b + L.top);
    s->ids = (int32_t*)(b + L.ids); s->res = (int32_t*)(b + L.res); s->state = (int32_t*)(b + L.state); s->routes = (int32_t*)(b + L.routes); s->route_w = (double*)(b + L.route_w);
    s->moe_scratch = b + L.moe; s->moe_scratch_bytes = L.moe_bytes;
    s->fork = (float*)(b + L.fork);
    if (m->ple.ngram >= 2) {
        s->p_e = (float*)(b + L.p_e); s->p_key = (float*)(b + L.p_key); s->p_val = (float*)(b + L.p_val); s->p_gv = (float*)(b + L.p_gv);
        s->p_gvn = (float*)(b + L.p_gvn); s->p_hist = (float*)(b + L.p_hist); s->p_tail = (int32_t*)(b + L.p_tail); s->p_hist_bytes = L.p_hist_bytes;
    }
    if (m->cfg.idx_heads > 0) {
        s->i_q = (float*)(b + L.i_q); s->i_k = (float*)(b + L.i_k); s->i_qn = (float*)(b + L.i_qn); s->i_raw = (float*)(b + L.i_raw);
        s->i_blocks = (float*)(b + L.i_blocks); s->i_scores = (float*)(b + L.i_scores); s->i_sel = (u32*)(b + L.i_sel);
        s->i_list = (int32_t*)(b + L.i_list); s->i_count = (int32_t*)(b + L.i_count); s->i_trace = (u32*)(b + L.i_trace);
        s->i_raw_layer = L.i_raw_layer; s->i_blocks_layer = L.i_blocks_layer; s->i_ctx_blocks = L.i_ctx_blocks; s->i_words = L.i_words;
    }
    s->attn_splits = L.splits; s->attn_splits2 = L.splits2;
    if ((rc = sz_head_describe(m, flags, &s->head))) { delete s; return rc; }
    if (s->head.rows > 0) {
        s->head.work = (uint64_t)(b + L.head_work); s->head.work_bytes = L.head_work_bytes;
        if (s->head.k_blk > 0) { s->head.w_q2 = (uint64_t)(b + L.head_q2); s->head.w_sc = (uint64_t)(b + L.head_sc); }
        if ((rc = sz_head_work_init(&s->head, stream)) || (s->head.k_blk > 0 && (rc = sz_head_proxy_build(&s->head, stream)))) { delete s; return rc; }
    }
    if ((rc = sz_session_reset(s, stream))) { delete s; return rc; }
    if (m->cfg.rope_dims > 0) {  // forward.rs:290-299: angle = pos / theta^(2 i / rope_dims); the denominators never change
        std::vector<double> den(m->cfg.rope_dims / 2);
        for (size_t i = 0; i < den.size(); i++) den[i] = pow((double)m->cfg.rope_theta, 2.0 * (double)i / (double)m->cfg.rope_dims);
        if (cudaMemcpy(s->rope_den, den.data(), den.size() * 8, cudaMemcpyHostToDevice) != cudaSuccess) { delete s; return sz_fail(SZ_E_CUDA, "rope table upload failed"); }
    }
    *out = s;
    return SZ_OK;
}

extern "C" void sz_session_destroy(sz_session* s) { delete s; }
extern "C" int sz_session_len(const sz_session* s) { return s ? s->len : -1; }
extern "C" int sz_session_capacity(const sz_session* s) { return s ? s->ctx : -1; }
extern "C" int sz_session_pending(const sz_session* s) { return s ? s->last_m : -1; }
extern "C" int sz_session_trace_routes(sz_session* s, int on) { if (!s) return sz_fail(SZ_E_ARG, "null session"); s->want_routes = on; return SZ_OK; }

// ---- dense launcher -----------------------------------------------------------------------------------------------------------------
static size_t sz_row_bytes_host(int type, int cols) {
    switch (type) {
        case SZ_TYPE_F32: return (size_t)cols * 4;
        case SZ_TYPE_F16: case SZ_TYPE_BF16: return (size_t)cols * 2;
        case SZ_TYPE_Q8_0: return (size_t)(cols / 32) * 34;
        default: return (size_t)(cols / 256) * 110;
    }
}

static int sz_dense_launch_generic(SzDenseArgs& a, cudaStream_t st, const char* name) {
    const size_t limit = 200 * 1024 - 2048;
    int mt = a.m;
    while (mt > 1 && (size_t)mt * a.cols * 4 > limit) mt = (mt + 1) / 2;
    if ((size_t)mt * a.cols * 4 > limit) return sz_fail(SZ_E_ARG, "%s: %d input columns do not fit in shared memory", name, a.cols);
    const size_t smem = 2048 + (size_t)mt * a.cols * 4;
    int blocks = (a.total_rows + 7) / 8;
    const int cap = 148 * 8;
    if (blocks > cap) blocks = cap;
    static bool set[9] = {false};
#define SZ_DENSE_CASE(MT)                                                                                                             \
    case MT:                                                                                                                          \
        if (!set[MT]) { SZ_CUDA(cudaFuncSetAttribute(sz_dense_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); set[MT] = true; } \
        SZ_CUDA(sz_launch(name, sz_dense_kernel<MT>, dim3(blocks), dim3(256), smem, st, true, a));                                   \
        break;
    switch (mt) {
        SZ_DENSE_CASE(1) SZ_DENSE_CASE(2) SZ_DENSE_CASE(3) SZ_DENSE_CASE(4) SZ_DENSE_CASE(5) SZ_DENSE_CASE(6) SZ_DENSE_CASE(7) SZ_DENSE_CASE(8)
    }
#undef SZ_DENSE_CASE
    return SZ_OK;
}

template <int MT, int RW>
static int sz_dense2_go(const SzDenseArgs& a, const SzDense2Cfg& c, int blocks, size_t smem, cudaStream_t st, const char* name) {
    static bool set = false;
    if (!set) { SZ_CUDA(cudaFuncSetAttribute(sz_dense2_kernel<MT, RW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); set = true; }
    SZ_CUDA(sz_launch(name, sz_dense2_kernel<MT, RW>, dim3(blocks), dim3(256), smem, st, true, a, c));
    return SZ_OK;
}

int sz_dense_launch(SzDenseArgs& a, cudaStream_t st, const char* name) {
    int total = 0;
    for (int i = 0; i < a.n_jobs; i++) { a.job[i].row0 = total; total += a.job[i].rows; }
    a.total_rows = total;
    static const bool generic_only = getenv("SZ_GENERIC_KERNELS") && atoi(getenv("SZ_GENERIC_KERNELS")) != 0;
    // the streaming kernel wants one type for all jobs of the launch and rows that are whole 16-byte chunks
    const int type = a.job[0].type;
    const size_t rb = sz_row_bytes_host(type, a.cols);
    bool ok = !generic_only && rb % 16 == 0 && rb <= 96 * 1024;
    for (int i = 1; i < a.n_jobs; i++) ok = ok && a.job[i].type == type;
    if (!ok) return sz_dense_launch_generic(a, st, name);
    if (type == SZ_TYPE_Q8_0 && a.cols % 256 == 0) {
        // tensor-pipe form: 16-row units, the columns split over the 8 warps
        SzDenseQ8Cfg q = {};
        // padded strides: consecutive rows 4 (mod 8) words apart in bank space, rows of the pass 16 words apart
        int rbp = (int)rb;
        while (((rbp / 4) % 32) % 8 != 4) rbp += 16;
        int xsp = a.cols;
        while (((xsp / 2) % 32) != 16) xsp += 8;
        q.rbp = rbp; q.xsp = xsp;
        q.unit_bytes = 16 * rbp;
        size_t fixed = 64 + 4096 + (size_t)a.m * xsp * 4;
        size_t budget = 110 * 1024;                        // two blocks a multiprocessor when that leaves at least two stages
        if (fixed + 2 * (size_t)q.unit_bytes > budget) budget = 216 * 1024;
        if (fixed + 2 * (size_t)q.unit_bytes > budget && a.m > 1 && 64 + 4096 + (size_t)((a.m + 1) / 2) * xsp * 4 + 2 * (size_t)q.unit_bytes <= budget) {
            // wide inputs with many rows do not fit next to two stages: two launches over half the rows each (the matrix is read
            // twice, from L2 the second time where it fits).  A row's result must not depend on how many rows share its pass
            // (batched == one at a time, bit for bit: crates/shadowzero/tests/reference.rs:226-255), so every row count has to
            // go through this one kernel's arithmetic rather than fall through to the f32 kernel below.
            const int m0 = (a.m + 1) / 2;
            SzDenseArgs lo = a, hi = a;
            lo.m = m0;
            hi.m = a.m - m0;
            hi.x = a.x + (size_t)m0 * a.xstride;
            for (int i = 0; i < a.n_jobs; i++) hi.job[i].out = a.job[i].out + (size_t)m0 * a.job[i].ostride;
            const int rc = sz_dense_launch(lo, st, name);
            return rc ? rc : sz_dense_launch(hi, st, name);
        }
        if (fixed + 2 * (size_t)q.unit_bytes <= budget) {
            int NS = (int)((budget - fixed) / q.unit_bytes);
            q.NS = NS > 4 ? 4 : NS;
            int units = 0;
            for (int i = 0; i < a.n_jobs; i++) { q.units[i] = units; units += (a.job[i].rows + 15) / 16; }
            q.units[a.n_jobs] = units;
            const size_t smem = fixed + (size_t)q.NS * q.unit_bytes;
            int blocks = 148 * (smem <= 110 * 1024 ? 2 : 1);
            if (blocks > units) blocks = units;
            static bool set = false;
            if (!set) { SZ_CUDA(cudaFuncSetAttribute(sz_dense_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); set = true; }
            SZ_CUDA(sz_launch(name, sz_dense_q8_kernel, dim3(blocks), dim3(256), smem, st, true, a, q));
            return SZ_OK;
        }
    }
    SzDense2Cfg c = {};
    int R = 32;
    while (R > 2 && (size_t)R * rb > 36 * 1024) R >>= 1;
    c.R = R;
    c.RW = R < 4 ? R : 4;
    const int NG = R / c.RW;
    int KP = 8 / NG;
    const int gran = type == SZ_TYPE_Q8_0 ? 32 : (type == SZ_TYPE_IQ3_S ? 256 : 4);
    while (KP > 1 && (a.cols % (KP * gran) != 0)) KP >>= 1;
    c.KP = KP;
    c.unit_bytes = (int)((size_t)R * rb);
    const size_t budget = 216 * 1024, fixed = 64 + 2048 + 1024;
    int mt = a.m;
    while (mt > 1 && fixed + (size_t)mt * a.cols * 4 + 2 * (size_t)c.unit_bytes > budget) mt = (mt + 1) / 2;
    if (fixed + (size_t)mt * a.cols * 4 + 2 * (size_t)c.unit_bytes > budget) return sz_dense_launch_generic(a, st, name);
    int NS = (int)((budget - fixed - (size_t)mt * a.cols * 4) / c.unit_bytes);
    c.NS = NS > 4 ? 4 : NS;
    int units = 0;
    for (int i = 0; i < a.n_jobs; i++) { c.units[i] = units; units += (a.job[i].rows + R - 1) / R; }
    c.units[a.n_jobs] = units;
    const size_t smem = fixed + (size_t)mt * a.cols * 4 + (size_t)c.NS * c.unit_bytes;
    const int per_sm = (int)((227 * 1024) / (smem + 1024));
    int blocks = 148 * (per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm));
    if (blocks > units) blocks = units;
#define SZ_D2(MT)                                                                                   \
    case MT:                                                                                        \
        return c.RW == 4 ? sz_dense2_go<MT, 4>(a, c, blocks, smem, st, name) : sz_dense2_go<MT, 2>(a, c, blocks, smem, st, name);
    switch (mt) { SZ_D2(1) SZ_D2(2) SZ_D2(3) SZ_D2(4) SZ_D2(5) SZ_D2(6) SZ_D2(7) SZ_D2(8) }
#undef SZ_D2
    return SZ_OK;
}

// Would sz_dense_launch take the Q8_0 tensor-pipe kernel for 8 rows of these jobs (whole, or as two launches of 4)?  Then it takes
// it for every row count up to 8, and the many-row form computes the same bits.
static bool sz_dense_q8_takes(const SzDenseArgs& a) {
    static const bool generic_only = getenv("SZ_GENERIC_KERNELS") && atoi(getenv("SZ_GENERIC_KERNELS")) != 0;
    if (generic_only || a.n_jobs < 1) return false;
    for (int i = 0; i < a.n_jobs; i++) if (a.job[i].type != SZ_TYPE_Q8_0) return false;
    const size_t rb = sz_row_bytes_host(SZ_TYPE_Q8_0, a.cols);
    if (a.cols % 256 || rb % 16 || rb > 96 * 1024) return false;
    int rbp = (int)rb;
    while (((rbp / 4) % 32) % 8 != 4) rbp += 16;
    int xsp = a.cols;
    while (((xsp / 2) % 32) != 16) xsp += 8;
    const size_t two = 2 * (size_t)16 * rbp;
    for (int m : {8, 4}) {
        const size_t fixed = 64 + 4096 + (size_t)m * xsp * 4;
        if (fixed + two <= 110 * 1024 || fixed + two <= 216 * 1024) return true;
    }
    return false;
}

int sz_dense_rows_launch(SzDenseArgs& a, float* partial, int64_t partial_floats, cudaStream_t st, const char* name, int* taken) {
    *taken = 0;
    if (a.m < 8 || a.m % 8 || !sz_dense_q8_takes(a)) return SZ_OK;
    int total = 0;
    for (int i = 0; i < a.n_jobs; i++) { a.job[i].row0 = total; total += a.job[i].rows; }
    a.total_rows = total;
    if ((int64_t)8 * a.m * total > partial_floats) return SZ_OK;
    SzDenseRowsCfg c = {};
    int units = 0;
    for (int i = 0; i < a.n_jobs; i++) { c.units[i] = units; units += (a.job[i].rows + 15) / 16; }
    c.units[a.n_jobs] = units;
    const int part = a.cols / 8;
    c.sb = part / 32 * 34;
    int rs = 0;
    for (int p = 0; p < 8; p++) { const int need = ((((p * c.sb) & 15) + c.sb + 15) >> 4) << 4; rs = need > rs ? need : rs; }
    while (((rs / 4) % 32) % 8 != 4) rs += 16;     // staged slices 4 (mod 8) words apart, rows of the pass 16 words, as the 8-row kernel
    int xs = part;
    while (((xs / 2) % 32) != 16) xs += 8;
    c.rs = rs; c.xs = xs; c.rows = a.m; c.G = a.m / 8; c.partial = partial;
    // row groups a block: what fits beside the two stages, two blocks a multiprocessor where four groups do
    const size_t stages = 2 * (size_t)128 * rs, group = (size_t)8 * xs * 4;
    int gb = 0;
    if (stages + 4 * group <= 110 * 1024) gb = 4;
    else if (c.G >= 8 && stages + 8 * group <= 216 * 1024) gb = 8;
    else if (stages + 4 * group <= 216 * 1024) gb = 4;
    else if (stages + 2 * group <= 216 * 1024) gb = 2;
    else return SZ_OK;
    if (c.G <= 2) gb = 2;
    c.gb = gb;
    c.nz = (c.G + gb - 1) / gb;
    const size_t smem = stages + (size_t)gb * group;
    const int target = sz_sm_count_session() * (smem <= 110 * 1024 ? 2 : 1);
    int nc = target / (8 * c.nz);
    if (nc < 1) nc = 1;
    c.upc = ((units + nc - 1) / nc + 7) / 8 * 8;
    nc = (units + c.upc - 1) / c.upc;
    const dim3 grid(8, nc, c.nz);
    cudaError_t e = cudaErrorInvalidValue;
#define SZ_DR(GG)                                                                                                                            \
    if (gb == GG) {                                                                                                                          \
        static bool set = false;                                                                                                             \
        if (!set) { SZ_CUDA(cudaFuncSetAttribute(sz_dense_rows_q8_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); set = true; } \
        e = sz_launch(name, sz_dense_rows_q8_kernel<GG>, grid, dim3(256), smem, st, true, a, c);                                             \
    }
    SZ_DR(2) SZ_DR(4) SZ_DR(8)
#undef SZ_DR
    SZ_CUDA(e);
    SZ_CUDA(sz_launch("dense_rows_reduce", sz_dense_rows_reduce_kernel, dim3((total + 255) / 256, a.m), dim3(256), 0, st, true, a, (const float*)partial, a.m));
    *taken = 1;
    return SZ_OK;
}

static SzDenseJob sz_job(const sz_tensor& t, float* out, int ostride, int epi = SZ_EPI_NONE, float div = 1.f) {
    SzDenseJob j;
    j.w = (const u8*)t.data; j.out = out; j.rows = (int)t.rows; j.type = t.type; j.ostride = ostride; j.epi = epi; j.div = div; j.row0 = 0;
    return j;
}

// ---- one pass ---------------------------------------------------------------------------------------------------------------------------
// hyper-connection read of `hc` for the m rows: applies the pending write (g_prev, y_prev) first; leaves u (and g when the read injects)
static bool sz_hc_fits(const sz_model_config& c, const sz_hc& hc, bool inject) {
    const int H = c.hidden, C = c.streams, rank = c.hc_rank, cpr = rank / 8;
    if (hc.down.type != SZ_TYPE_BF16 || hc.up.type != SZ_TYPE_BF16 || hc.norm.type != SZ_TYPE_F32) return false;
    if (inject && hc.inject.type != SZ_TYPE_BF16) return false;
    if (H % 64 || H > 2048 || rank % 8 || rank > 256 || rank + C > 320 || rank + C > SZ_HC_ACC_ROWS) return false;
    if (cpr < 1 || (32 % cpr) || (16 * C * cpr) % 32 || 16 * C * cpr > 2048 || 16 * C > 64) return false;
    return true;
}

static int sz_hc_read(sz_session* s, cudaStream_t st, const sz_hc& hc, int m, bool pending, bool inject) {
    const sz_model_config& c = s->model.cfg;
    const int H = c.hidden, C = c.streams, CH = C * H;
    if (s->hc_fast) {
        // read n: residual in buffer n & 1, out the other; accumulator n % 3, the previous read's holds the gates of the pending write
        const int n = s->hc_n++;
        float* rin = (n & 1) ? s->r2 : s->r;
        float* rout = (n & 1) ? s->r : s->r2;
        const int64_t as = s->hc_acc_stride;
        long long* acc = s->hc_acc + (n % 3) * as;
        long long* acc_prev = s->hc_acc + ((n + 2) % 3) * as;
        long long* acc_next = s->hc_acc + ((n + 1) % 3) * as;
        int nt = ((int)c.hc_rank + C + 31) / 32 * 32;
        if (nt < 256) nt = 256;
        cudaError_t e1 = cudaErrorInvalidValue, e2 = cudaSuccess;
        // SZ_HC_FUSED=1: one launch (down half, grid-wide barrier, up half) when all its blocks fit the GPU at once - the barrier
        // needs every block resident.  Measured slower than the two launches (a 4-row pass of the 48-layer model: 6.48 ms against
        // 6.16 ms): a launch boundary with programmatic dependent launch costs less than a barrier whose every step is a round
        // trip to L2, so the two halves stay launches of their own and the fused form is the second implementation.
        const char* fe = getenv("SZ_HC_FUSED");   // (read when a pass is built: a test switches it between two sessions of one process)
        const bool split = !(fe && atoi(fe) != 0);
        const int blocks = CH / 64 > H / 16 ? CH / 64 : H / 16;
        if (!split && blocks <= sz_sm_count_session()) {
#define SZ_HC_CASE(MM)                                                                                                                   \
    case MM:                                                                                                                             \
        e1 = sz_launch("hc_read", sz_hc_read_kernel<MM>, dim3(blocks), dim3(nt), 0, st, true, (const float*)rin, rout,                   \
                       (const long long*)(pending ? acc_prev : nullptr), (const float*)s->y, (const float*)hc.norm.data,                 \
                       (const u8*)hc.down.data, (const u8*)(inject ? hc.inject.data : 0), (const u8*)hc.up.data, H, C, (int)c.hc_rank,   \
                       c.eps, s->rn, acc, acc_next, s->u, (u32*)(s->state + 4), (u32*)(s->state + 2));                                   \
        break;
            switch (m) {
                SZ_HC_CASE(1) SZ_HC_CASE(2) SZ_HC_CASE(3) SZ_HC_CASE(4) SZ_HC_CASE(5) SZ_HC_CASE(6) SZ_HC_CASE(7) SZ_HC_CASE(8)
            }
#undef SZ_HC_CASE
            SZ_CUDA(e1);
            return SZ_OK;
        }
        e2 = cudaErrorInvalidValue;
#define SZ_HC_CASE(MM)                                                                                                                   \
    case MM:                                                                                                                             \
        e1 = sz_launch("hc_down", sz_hc_down_kernel<MM>, dim3(CH / 64), dim3(nt), 0, st, true, (const float*)rin, rout,                  \
                       (const long long*)(pending ? acc_prev : nullptr), (const float*)s->y, (const float*)hc.norm.data,                 \
                       (const u8*)hc.down.data, (const u8*)(inject ? hc.inject.data : 0), H, C, (int)c.hc_rank, c.eps, s->rn, acc,       \
                       acc_next);                                                                                                        \
        e2 = sz_launch("hc_up", sz_hc_up_kernel<MM>, dim3(H / 16), dim3(256), 0, st, true, (const long long*)acc, (const u8*)hc.up.data, \
                       (const float*)s->rn, H, C, (int)c.hc_rank, s->u);                                                                 \
        break;
        switch (m) {
            SZ_HC_CASE(1) SZ_HC_CASE(2) SZ_HC_CASE(3) SZ_HC_CASE(4) SZ_HC_CASE(5) SZ_HC_CASE(6) SZ_HC_CASE(7) SZ_HC_CASE(8)
        }
#undef SZ_HC_CASE
        SZ_CUDA(e1);
        SZ_CUDA(e2);
        return SZ_OK;
    }
    SZ_CUDA(sz_launch("hc_norm", sz_hc_norm_kernel, dim3(C, m), dim3(256), 0, st, true, s->r, (const float*)(pending ? s->g : nullptr),
                      (const float*)(pending ? s->y : nullptr), (const float*)hc.norm.data, H, C, c.eps, s->rn));
    SzDenseArgs a = {};
    a.err = (u32*)(s->state + 2);
    a.x = s->rn; a.xstride = CH; a.cols = CH; a.m = m;
    a.job[0] = sz_job(hc.down, s->hdown, c.hc_rank, SZ_EPI_SILU_DIV, (float)C);
    a.n_jobs = 1;
    if (inject) { a.job[1] = sz_job(hc.inject, s->g, C, SZ_EPI_SIGMOID2_DIV, (float)C); a.n_jobs = 2; }
    int rc = sz_dense_launch(a, st, "hc_down");
    if (rc) return rc;
    SzDenseArgs b = {};
    b.err = (u32*)(s->state + 2);
    b.x = s->hdown; b.xstride = c.hc_rank; b.cols = c.hc_rank; b.m = m;
    b.job[0] = sz_job(hc.up, s->mix, CH, SZ_EPI_SIGMOID);
    b.n_jobs = 1;
    if ((rc = sz_dense_launch(b, st, "hc_up"))) return rc;
    SZ_CUDA(sz_launch("hc_mix", sz_hc_mix_kernel, dim3((H + 255) / 256, m), dim3(256), 0, st, true, (const float*)s->mix, (const float*)s->rn, H, C, s->u));
    return SZ_OK;
}

// The fused read over the rows of a batch: buffers that hold the rows of all sequences one after the other (a multiple of 8 rows,
// the sequences' own buffers pointing into them), eight rows a block row of the two kernels.  n: the read's number in the pass.
struct SzBatchBufs { float *r, *r2, *y, *u, *rn; long long* acc; int64_t acc_stride; };
static int sz_hc_read_rows(const sz_session* s, cudaStream_t st, const sz_hc& hc, int rows, int n, bool pending, bool inject, const SzBatchBufs& B, bool pdl) {
    const sz_model_config& c = s->model.cfg;
    const int H = c.hidden, C = c.streams, CH = C * H;
    float* rin = (n & 1) ? B.r2 : B.r;
    float* rout = (n & 1) ? B.r : B.r2;
    long long* acc = B.acc + (n % 3) * B.acc_stride;
    long long* acc_prev = B.acc + ((n + 2) % 3) * B.acc_stride;
    long long* acc_next = B.acc + ((n + 1) % 3) * B.acc_stride;
    int nt = ((int)c.hc_rank + C + 31) / 32 * 32;
    if (nt < 256) nt = 256;
    // rows a block row: the kernels keep a row's data in registers, so fewer rows a block mean more blocks a multiprocessor (the
    // second half: 8 or 4 rows two blocks, 2 rows four); measured on a step of 160 rows: 57.7 / 57.5 / 56.8 ms at 8 / 4 / 2
    static const int per = [] { const char* e = getenv("SZ_BATCH_HC_ROWS"); const int v = e ? atoi(e) : 2; return v == 8 || v == 4 ? v : 2; }();
    cudaError_t e1 = cudaErrorInvalidValue, e2 = cudaErrorInvalidValue;
    // The first half in its many-row form: the norm once a (row, stream), then the products (SZ_BATCH_HC_SPLIT=0: the pass's own
    // kernel with a block row per `per` rows, where every block of a stream redoes the stream's norm; same bits).
    const char* sp = getenv("SZ_BATCH_HC_SPLIT");   // (read at every call: a test switches it inside one process)
    if (!(sp && atoi(sp) == 0)) {
        SZ_CUDA(sz_launch("hc_rows_norm", sz_hc_rows_norm_kernel, dim3(C, rows), dim3(nt), 0, st, pdl, (const float*)rin, rout,
                          (const long long*)(pending ? acc_prev : nullptr), (const float*)B.y, (const float*)hc.norm.data, H, C, (int)c.hc_rank, c.eps,
                          B.rn, acc_next));
        SZ_CUDA(sz_launch("hc_rows_down", sz_hc_rows_down_kernel<8>, dim3(CH / 64, rows / 8), dim3(nt), 0, st, true, (const float*)B.rn,
                          (const u8*)hc.down.data, (const u8*)(inject ? hc.inject.data : 0), H, C, (int)c.hc_rank, acc));
        if (per == 8) e2 = sz_launch("hc_up", sz_hc_up_kernel<8>, dim3(H / 16, rows / 8), dim3(256), 0, st, true, (const long long*)acc, (const u8*)hc.up.data, (const float*)B.rn, H, C, (int)c.hc_rank, B.u);
        else if (per == 4) e2 = sz_launch("hc_up", sz_hc_up_kernel<4>, dim3(H / 16, rows / 4), dim3(256), 0, st, true, (const long long*)acc, (const u8*)hc.up.data, (const float*)B.rn, H, C, (int)c.hc_rank, B.u);
        else e2 = sz_launch("hc_up", sz_hc_up_kernel<2>, dim3(H / 16, rows / 2), dim3(256), 0, st, true, (const long long*)acc, (const u8*)hc.up.data, (const float*)B.rn, H, C, (int)c.hc_rank, B.u);
        SZ_CUDA(e2);
        return SZ_OK;
    }
#define SZ_HC_ROWS(MM)                                                                                                                          \
    if (per == MM) {                                                                                                                            \
        e1 = sz_launch("hc_down", sz_hc_down_kernel<MM>, dim3(CH / 64, rows / MM), dim3(nt), 0, st, pdl, (const float*)rin, rout,               \
                       (const long long*)(pending ? acc_prev : nullptr), (const float*)B.y, (const float*)hc.norm.data, (const u8*)hc.down.data, \
                       (const u8*)(inject ? hc.inject.data : 0), H, C, (int)c.hc_rank, c.eps, B.rn, acc, acc_next);                             \
        e2 = sz_launch("hc_up", sz_hc_up_kernel<MM>, dim3(H / 16, rows / MM), dim3(256), 0, st, true, (const long long*)acc,                    \
                       (const u8*)hc.up.data, (const float*)B.rn, H, C, (int)c.hc_rank, B.u);                                                   \
    }
    SZ_HC_ROWS(8) SZ_HC_ROWS(4) SZ_HC_ROWS(2)
#undef SZ_HC_ROWS
    SZ_CUDA(e1);
    SZ_CUDA(e2);
    return SZ_OK;
}

// The DeltaNet scan: the pass of one layer (l >= 0: all m rows, with outputs) or the replay of a commit (l < 0: every layer in one
// launch, the kept rows only, decided on the device).
template <int D, int PARTS>
static int sz_scan_launch(sz_session* s, cudaStream_t st, int l, int m, const SzDeltaPrep& pp) {
    const sz_model_config& c = s->model.cfg;
    const int64_t kd = (int64_t)c.ssm_k_heads * D, vd = (int64_t)c.ssm_v_heads * D, ch = 2 * kd + vd;
    const int64_t Sl = (int64_t)c.ssm_v_heads * D * D;
    const int di = l >= 0 ? s->lb[l].delta_index : 0;
    const float* xc = s->d_xc + (int64_t)di * SZ_MAX_VERIFY * ch;
    const float* beta = s->d_beta + (int64_t)di * SZ_MAX_VERIFY * c.ssm_v_heads;
    const float* decay = s->d_decay + (int64_t)di * SZ_MAX_VERIFY * c.ssm_v_heads;
    const float* nw = l >= 0 ? (const float*)s->layers[l].ssm_norm.data : nullptr;
    SZ_CUDA(sz_launch(l >= 0 ? "delta_scan" : "delta_replay", sz_delta_scan_kernel<D, PARTS>, dim3(c.ssm_v_heads, l >= 0 ? 1 : s->n_delta),
                      dim3(D * PARTS), 0, st, true, xc, beta, decay, (const float*)s->d_z, nw, (const float*)(s->S[0] + di * Sl),
                      (const float*)(s->S[1] + di * Sl), s->S[0] + di * Sl, s->S[1] + di * Sl, (const int32_t*)s->state, (const int32_t*)s->res,
                      (int)c.ssm_k_heads, (int)c.ssm_v_heads, m, c.eps, l >= 0 ? s->d_og : (float*)nullptr, pp,
                      (const SzTree*)(s->tree_pass ? s->ids + 32 : nullptr), s->fork));
    return SZ_OK;
}

static int sz_scan(sz_session* s, cudaStream_t st, int l, int m, const SzDeltaPrep& pp) {
    if (s->model.cfg.ssm_head_dim == 128) return sz_scan_launch<128, 2>(s, st, l, m, pp);
    return sz_scan_launch<64, 1>(s, st, l, m, pp);
}

// One sequence's entry of the table the many-sequence scan reads: what sz_delta_layer hands the scan of layer l, fused front end.
static void sz_scan_seq_entry(sz_session* s, int l, int m, SzScanSeq* e) {
    const sz_model_config& c = s->model.cfg;
    const sz_layer& L = s->layers[l];
    const int di = s->lb[l].delta_index;
    const int vh = c.ssm_v_heads, kh = c.ssm_k_heads, d = c.ssm_head_dim;
    const int64_t kd = (int64_t)kh * d, vd = (int64_t)vh * d, ch = 2 * kd + vd;
    const int64_t Sl = (int64_t)vh * d * d, cl = (int64_t)(c.conv_k - 1) * ch;
    *e = SzScanSeq{};
    e->xc = s->d_xc + (int64_t)di * SZ_MAX_VERIFY * ch;
    e->beta = s->d_beta + (int64_t)di * SZ_MAX_VERIFY * vh;
    e->decay = s->d_decay + (int64_t)di * SZ_MAX_VERIFY * vh;
    e->z = s->d_z;
    e->S0 = s->S[0] + di * Sl; e->S1 = s->S[1] + di * Sl;
    e->O0 = s->S[0] + di * Sl; e->O1 = s->S[1] + di * Sl;
    e->state = s->state; e->res = s->res;
    e->og = s->d_og;
    e->pp.xin = s->d_xin + (int64_t)di * SZ_MAX_VERIFY * ch;
    e->pp.conv0 = s->conv[0] + di * cl; e->pp.conv1 = s->conv[1] + di * cl;
    e->pp.cw = (const float*)L.ssm_conv1d.data;
    e->pp.b = s->d_b; e->pp.a = s->d_a;
    e->pp.a_log = (const float*)L.ssm_a.data; e->pp.dt = (const float*)L.ssm_dt_bias.data;
    e->pp.xc = s->d_xc + (int64_t)di * SZ_MAX_VERIFY * ch;
    e->pp.beta = s->d_beta + (int64_t)di * SZ_MAX_VERIFY * vh;
    e->pp.decay = s->d_decay + (int64_t)di * SZ_MAX_VERIFY * vh;
    e->pp.k = (int)c.conv_k;
    e->m = m;
}
// The scans of layer l of n sequences in one launch (tab: their entries on the device).
static int sz_scan_seqs(sz_session* s0, cudaStream_t st, int l, int n, const SzScanSeq* tab, bool pdl) {
    const sz_model_config& c = s0->model.cfg;
    const float* nw = (const float*)s0->layers[l].ssm_norm.data;
    if (c.ssm_head_dim == 128)
        SZ_CUDA(sz_launch("delta_scan_seqs", sz_delta_scan_seqs_kernel<128, 2>, dim3(c.ssm_v_heads, n), dim3(256), 0, st, pdl, tab, nw, (int)c.ssm_k_heads,
                          (int)c.ssm_v_heads, c.eps));
    else
        SZ_CUDA(sz_launch("delta_scan_seqs", sz_delta_scan_seqs_kernel<64, 1>, dim3(c.ssm_v_heads, n), dim3(64), 0, st, pdl, tab, nw, (int)c.ssm_k_heads,
                          (int)c.ssm_v_heads, c.eps));
    return SZ_OK;
}

// Which parts of a mixer a call runs: its input projections, what lies between them and the output projection, the output
// projection.  A batched step runs the projections of all sequences together and only the middle per sequence.
enum { SZ_MIX_IN = 1, SZ_MIX_CORE = 2, SZ_MIX_OUT = 4, SZ_MIX_ALL = 7 };

// The input projections of layer l's mixer as jobs of the dense launcher that write the session's buffers (a: x = s->u), and the
// output projection (b: x = the mixer's result before it, into s->y).
static void sz_mixer_args(sz_session* s, int l, int m, SzDenseArgs* a, SzDenseArgs* b) {
    const sz_model_config& c = s->model.cfg;
    const sz_layer& L = s->layers[l];
    const int H = c.hidden;
    *a = SzDenseArgs{};
    *b = SzDenseArgs{};
    a->err = b->err = (u32*)(s->state + 2);
    a->x = s->u; a->xstride = H; a->cols = H; a->m = m;
    b->m = m; b->n_jobs = 1;
    if (sz_is_attn(c, l)) {
        const int nh = c.n_head, nkv = c.n_kv_head, hd = c.head_dim;
        a->n_jobs = 3;
        a->job[0] = sz_job(L.attn_q, s->a_qg, 2 * nh * hd);
        a->job[1] = sz_job(L.attn_k, s->a_k, nkv * hd);
        a->job[2] = sz_job(L.attn_v, s->a_v, nkv * hd);
        if (c.idx_heads > 0) {
            a->n_jobs = 5;
            a->job[3] = sz_job(L.idx_q, s->i_q, c.idx_heads * c.idx_dim);
            a->job[4] = sz_job(L.idx_k, s->i_k, c.idx_dim);
        }
        b->x = s->a_o; b->xstride = nh * hd; b->cols = nh * hd;
        b->job[0] = sz_job(L.attn_output, s->y, H);
    } else {
        const int di = s->lb[l].delta_index;
        const int vh = c.ssm_v_heads, kh = c.ssm_k_heads, d = c.ssm_head_dim;
        const int64_t kd = (int64_t)kh * d, vd = (int64_t)vh * d, ch = 2 * kd + vd;
        a->n_jobs = 4;
        a->job[0] = sz_job(L.attn_qkv, s->d_xin + (int64_t)di * SZ_MAX_VERIFY * ch, (int)ch);
        a->job[1] = sz_job(L.attn_gate, s->d_z, (int)vd);
        a->job[2] = sz_job(L.ssm_beta, s->d_b, vh);
        a->job[3] = sz_job(L.ssm_alpha, s->d_a, vh);
        b->x = s->d_og; b->xstride = (int)vd; b->cols = (int)vd;
        b->job[0] = sz_job(L.ssm_out, s->y, H);
    }
}

static int sz_delta_layer(sz_session* s, cudaStream_t st, int l, int m, int parts = SZ_MIX_ALL) {
    const sz_model_config& c = s->model.cfg;
    const sz_layer& L = s->layers[l];
    const int di = s->lb[l].delta_index;
    const int vh = c.ssm_v_heads, kh = c.ssm_k_heads, d = c.ssm_head_dim;
    const int64_t kd = (int64_t)kh * d, vd = (int64_t)vh * d, ch = 2 * kd + vd;
    float* xin = s->d_xin + (int64_t)di * SZ_MAX_VERIFY * ch;
    float* xc = s->d_xc + (int64_t)di * SZ_MAX_VERIFY * ch;
    float* beta = s->d_beta + (int64_t)di * SZ_MAX_VERIFY * vh;
    float* decay = s->d_decay + (int64_t)di * SZ_MAX_VERIFY * vh;
    SzDenseArgs a, b;
    sz_mixer_args(s, l, m, &a, &b);
    int rc = SZ_OK;
    if ((parts & SZ_MIX_IN) && (rc = sz_dense_launch(a, st, "delta_proj"))) return rc;
    if (!(parts & SZ_MIX_CORE)) return (parts & SZ_MIX_OUT) ? sz_dense_launch(b, st, "ssm_out") : SZ_OK;
    const int64_t cl = (int64_t)(c.conv_k - 1) * ch;
    static const bool split_prep = getenv("SZ_GENERIC_KERNELS") && atoi(getenv("SZ_GENERIC_KERNELS")) != 0;
    SzDeltaPrep pp = {};
    if (split_prep) {  // the front end as a kernel of its own (the second implementation the fused one is checked against)
        SZ_CUDA(sz_launch("delta_prep", sz_delta_prep_kernel, dim3((unsigned)((ch + 255) / 256), m), dim3(256), 0, st, true, (const float*)xin, (const float*)(s->conv[0] + di * cl),
                          (const float*)(s->conv[1] + di * cl), (const int32_t*)s->state, (const float*)L.ssm_conv1d.data, (const float*)s->d_b,
                          (const float*)s->d_a, (const float*)L.ssm_a.data, (const float*)L.ssm_dt_bias.data, kh, vh, d, (int)c.conv_k, xc, beta, decay));
    } else {
        pp.xin = xin; pp.conv0 = s->conv[0] + di * cl; pp.conv1 = s->conv[1] + di * cl; pp.cw = (const float*)L.ssm_conv1d.data;
        pp.b = s->d_b; pp.a = s->d_a; pp.a_log = (const float*)L.ssm_a.data; pp.dt = (const float*)L.ssm_dt_bias.data;
        pp.xc = xc; pp.beta = beta; pp.decay = decay; pp.k = (int)c.conv_k;
    }
    if ((rc = sz_scan(s, st, l, m, pp))) return rc;
    return (parts & SZ_MIX_OUT) ? sz_dense_launch(b, st, "ssm_out") : SZ_OK;
}

template <int EPL>
static int sz_attn_launch(sz_session* s, cudaStream_t st, const u8* kc, const u8* vc, int m) {
    const sz_model_config& c = s->model.cfg;
    SZ_CUDA(sz_launch("attention", sz_attn_kernel<EPL>, dim3(c.n_head, m, s->attn_splits), dim3(256), 0, st, true, (const float*)s->a_q, kc, vc,
                      (int)c.n_head, (int)c.n_kv_head, s->ctx, (const int32_t*)s->state, (s->flags & SZ_KV_Q8) ? 1 : 0, s->attn_splits, s->a_part,
                      (const SzTree*)(s->tree_pass ? s->ids + 32 : nullptr)));
    return SZ_OK;
}

template <int HD, int NQT>
static int sz_attn2_go(sz_session* s, cudaStream_t st, const u8* kc, const u8* vc, int m, int* splits_used, int ratio) {
    const sz_model_config& c = s->model.cfg;
    static bool set = false;
    const size_t smem = (size_t)SzAttn2<HD>::smem_bytes(NQT);
    if (!set) { SZ_CUDA(cudaFuncSetAttribute(sz_attn2_kernel<HD, NQT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); set = true; }
    // two blocks fit a multiprocessor when the query fragments are small: twice the splits then, so that each block's chain of
    // chunks is half as long and the two blocks hide each other's barriers
    int splits = s->attn_splits2;
    if (smem + 2048 <= 113 * 1024 && 2 * splits <= (s->ctx + 255) / 256) splits *= 2;
    if (ratio) {   // the sparse form: a block a (kv head, split, row); a row's list holds about the budget's positions, 128 or more a split
        const int by_budget = (c.idx_budget + 127) / 128;
        if (splits > by_budget) splits = by_budget < 1 ? 1 : by_budget;
    }
    *splits_used = splits;
    SZ_CUDA(sz_launch("attention_grouped", sz_attn2_kernel<HD, NQT>, dim3(c.n_kv_head, splits, ratio ? m : 1), dim3(256), smem, st, true, (const float*)s->a_q,
                      kc, vc, (int)c.n_head, (int)c.n_kv_head, m, s->ctx, (const int32_t*)s->state, splits, s->a_part, (u32*)(s->state + 2),
                      (const SzTree*)(s->tree_pass ? s->ids + 32 : nullptr), (const int32_t*)(ratio ? s->i_list : nullptr), (const int32_t*)s->i_count,
                      s->i_ctx_blocks, ratio));
    return SZ_OK;
}

template <int HD>
static int sz_attn2_launch(sz_session* s, cudaStream_t st, const u8* kc, const u8* vc, int m, int* splits_used, int ratio) {
    const sz_model_config& c = s->model.cfg;
    const int qv = c.n_head / c.n_kv_head * (ratio ? 1 : m);   // the sparse form serves one row a block
    if (qv <= 16) return sz_attn2_go<HD, 1>(s, st, kc, vc, m, splits_used, ratio);
    if (qv <= 32) return sz_attn2_go<HD, 2>(s, st, kc, vc, m, splits_used, ratio);
    return sz_attn2_go<HD, 4>(s, st, kc, vc, m, splits_used, ratio);
}

static int sz_attn_layer(sz_session* s, cudaStream_t st, int l, int m, int parts = SZ_MIX_ALL) {
    const sz_model_config& c = s->model.cfg;
    const sz_layer& L = s->layers[l];
    const int ai = s->lb[l].attn_index;
    const int nh = c.n_head, nkv = c.n_kv_head, hd = c.head_dim;
    const int q8 = (s->flags & SZ_KV_Q8) ? 1 : 0;
    const int64_t hb = q8 ? (hd + (((hd >> 5) * 2 + 15) & ~15)) : 4 * (int64_t)hd;
    const int64_t layer_bytes = (int64_t)s->ctx * nkv * hb;
    u8 *kc = s->kc + ai * layer_bytes, *vc = s->vc + ai * layer_bytes;
    SzDenseArgs a, b;
    sz_mixer_args(s, l, m, &a, &b);
    const bool idx = c.idx_heads > 0;
    const int ratio = idx ? (L.idx_ratio > 0 ? L.idx_ratio : 1) : 0;
    if (idx && s->tree_pass) return sz_fail(SZ_E_ARG, "a tree pass on a model with the sparse indexer is not supported");
    int rc = SZ_OK;
    if ((parts & SZ_MIX_IN) && (rc = sz_dense_launch(a, st, "attn_proj"))) return rc;
    if (!(parts & SZ_MIX_CORE)) return (parts & SZ_MIX_OUT) ? sz_dense_launch(b, st, "attn_output") : SZ_OK;
    if (idx) {
        SzIdxGeom g;
        g.heads = c.idx_heads; g.dim = c.idx_dim; g.ratio = ratio; g.keep = c.idx_budget / ratio; g.ctx_blocks = s->i_ctx_blocks; g.words = s->i_words;
        float* raw = (float*)((u8*)s->i_raw + ai * s->i_raw_layer);
        float* blocks = (float*)((u8*)s->i_blocks + ai * s->i_blocks_layer);
        SZ_CUDA(sz_launch("idx_prep", sz_idx_prep_kernel, dim3(c.idx_heads + 2, m), dim3(128), 0, st, true, (const float*)s->i_q, (const float*)s->i_k,
                          (const float*)L.idx_q_norm.data, (const float*)L.idx_k_norm.data, g, c.eps, (const int32_t*)s->state, (int)c.rope_dims,
                          (const double*)s->rope_den, raw, blocks, s->i_qn));
        const int nb_cap = s->ctx / ratio + 1;   // a warp a block, eight blocks a thread block, up to four thread blocks a multiprocessor
        const int sblocks = (nb_cap + 7) / 8 < 4 * sz_sm_count_session() ? (nb_cap + 7) / 8 : 4 * sz_sm_count_session();
        SZ_CUDA(sz_launch("idx_score", sz_idx_score_kernel, dim3(sblocks), dim3(256), (size_t)m * c.idx_heads * c.idx_dim * 4, st, true,
                          (const float*)s->i_qn, (const float*)blocks, g, m, (const int32_t*)s->state, s->i_scores));
        SZ_CUDA(sz_launch("idx_select", sz_idx_select_kernel, dim3(m), dim3(1024), (size_t)s->i_words * 4, st, true, (const float*)s->i_scores, g, m,
                          (const int32_t*)s->state, s->i_sel, s->i_list, s->i_count, s->i_trace + (size_t)ai * SZ_MAX_VERIFY * s->i_words));
    }
    SZ_CUDA(sz_launch("attn_prep", sz_attn_prep_kernel, dim3(nh + 2 * nkv, m), dim3(128), 0, st, true, (const float*)s->a_qg, (const float*)s->a_k,
                      (const float*)s->a_v, (const float*)L.attn_q_norm.data, (const float*)L.attn_k_norm.data, nh, nkv, hd, s->ctx, c.eps,
                      (const int32_t*)s->state, (int)c.rope_dims, (const double*)s->rope_den, q8, kc, vc, s->a_q, s->a_gate,
                      (const SzTree*)(s->tree_pass ? s->ids + 32 : nullptr)));
    // the grouped tensor-core kernel serves the packed int8 cache with up to 64 queries a KV head; the simple kernel everything else
    static const bool generic_only = getenv("SZ_GENERIC_KERNELS") && atoi(getenv("SZ_GENERIC_KERNELS")) != 0;
    const bool grouped = q8 && (!generic_only || idx) && (nh / nkv) * m <= 64;
    int splits = grouped ? s->attn_splits2 : s->attn_splits;
    if (grouped) {
        if (hd == 64) rc = sz_attn2_launch<64>(s, st, kc, vc, m, &splits, ratio);
        else if (hd == 128) rc = sz_attn2_launch<128>(s, st, kc, vc, m, &splits, ratio);
        else rc = sz_attn2_launch<256>(s, st, kc, vc, m, &splits, ratio);
    } else {
        if (hd == 64) rc = sz_attn_launch<2>(s, st, kc, vc, m);
        else if (hd == 128) rc = sz_attn_launch<4>(s, st, kc, vc, m);
        else rc = sz_attn_launch<8>(s, st, kc, vc, m);
    }
    if (rc) return rc;
    SZ_CUDA(sz_launch("attn_merge", sz_attn_merge_kernel, dim3(nh, m), dim3(256), 0, st, true, (const float*)s->a_part, (const float*)s->a_gate, nh, hd,
                      splits, s->a_o));
    return (parts & SZ_MIX_OUT) ? sz_dense_launch(b, st, "attn_output") : SZ_OK;
}

// The per-layer embedding before layer model.ple.layer's first read (sz_ple.cuh).  The residual of the moment: with the fused
// hyper-connection read, the buffer the next read takes as its input, and the pending write's gates in the previous read's accumulator.
static int sz_ple_layer(sz_session* s, cudaStream_t st, int m, bool pending) {
    const sz_model_config& c = s->model.cfg;
    const sz_ple& p = s->model.ple;
    const int H = c.hidden, C = c.streams, CH = C * H, heads = (p.ngram - 1) * p.heads_per_ngram;
    if (s->tree_pass) return sz_fail(SZ_E_ARG, "a tree pass on a model with per-layer embeddings is not supported");
    SzPleGeom g = {};
    g.ngram = p.ngram; g.heads_per_ngram = p.heads_per_ngram; g.head_dim = p.head_dim; g.conv_k = p.conv_k; g.eos = p.eos; g.table_type = p.table.type;
    for (int i = 0; i < SZ_PLE_MAX_NGRAM; i++) g.multipliers[i] = p.multipliers[i];
    for (int i = 0; i < SZ_PLE_MAX_HEADS; i++) { g.vocab[i] = p.vocab[i]; g.offsets[i] = p.offsets[i]; }
    SZ_CUDA(sz_launch("ple_embed", sz_ple_embed_kernel, dim3(heads, m), dim3(64), 0, st, true, (const int32_t*)s->ids, (const int32_t*)s->p_tail,
                      (const int32_t*)s->state, g, (const u8*)p.table.data, (long long)p.table.rows, H, s->p_e));
    SzDenseArgs a = {};
    a.err = (u32*)(s->state + 2);
    a.x = s->p_e; a.xstride = H; a.cols = H; a.m = m; a.n_jobs = 2;
    a.job[0] = sz_job(p.key, s->p_key, CH);
    a.job[1] = sz_job(p.value, s->p_val, H);
    int rc = sz_dense_launch(a, st, "ple_proj");
    if (rc) return rc;
    float* r = s->r;
    const long long* g_acc = nullptr;
    const float* g_f = nullptr;
    if (s->hc_fast) {
        const int n = s->hc_n;                       // the read that follows
        r = (n & 1) ? s->r2 : s->r;
        if (pending) g_acc = s->hc_acc + ((n + 2) % 3) * s->hc_acc_stride;
    } else if (pending) {
        g_f = s->g;
    }
    SZ_CUDA(sz_launch("ple_gate", sz_ple_gate_kernel, dim3(C, m), dim3(256), (size_t)2 * H * 4, st, true, r, g_acc, (int)SZ_HC_ACC_ROWS, (int)c.hc_rank, g_f,
                      (const float*)s->y, (const float*)s->p_key, (const float*)s->p_val, (const float*)p.norm_key.data, (const float*)p.norm_query.data,
                      (const float*)p.norm_conv.data, H, C, c.eps, s->p_gv, s->p_gvn));
    SZ_CUDA(sz_launch("ple_conv", sz_ple_conv_kernel, dim3((CH + 255) / 256, m), dim3(256), 0, st, true, r, (const float*)s->p_gv, (const float*)s->p_gvn,
                      (const float*)s->p_hist, (const float*)((const u8*)s->p_hist + s->p_hist_bytes), (const int32_t*)s->state, (const float*)p.conv1d.data, CH,
                      (int)p.conv_k, (int)p.ngram));
    return SZ_OK;
}

// Runs the m rows through every layer and, with `head`, through the output projection and the top-64.
static int sz_forward_begin(sz_session* s, cudaStream_t st, int m, bool clear = true) {
    const sz_model_config& c = s->model.cfg;
    s->hc_n = 0;
    if (s->hc_fast && clear) SZ_CUDA(cudaMemsetAsync(s->hc_acc, 0, sizeof(long long) * SZ_MAX_VERIFY * SZ_HC_ACC_ROWS, st));  // read 0 adds into buffer 0
    SZ_CUDA(sz_launch("embed", sz_embed_kernel, dim3(m), dim3(256), 0, st, false, (const int32_t*)s->ids, (const u8*)s->model.token_embd.data,
                      (int)s->model.token_embd.type, (int)c.hidden, (int)c.streams, (int)c.vocab, s->r));
    return SZ_OK;
}
// Layer l up to the input of its MoE sublayer (s->u): the per-layer embedding where it is, the read, the mixer, the second read.
static int sz_layer_to_moe(sz_session* s, cudaStream_t st, int l, int m, bool pending) {
    const sz_model_config& c = s->model.cfg;
    const sz_layer& L = s->layers[l];
    int rc;
    if (s->p_hist && l == s->model.ple.layer) {   // the per-layer embedding joins the residual stream; it applies the pending write itself
        if ((rc = sz_ple_layer(s, st, m, pending))) return rc;
        pending = false;
    }
    if ((rc = sz_hc_read(s, st, L.hc_attn, m, pending, true))) return rc;
    rc = sz_is_attn(c, l) ? sz_attn_layer(s, st, l, m) : sz_delta_layer(s, st, l, m);
    if (rc) return rc;
    return sz_hc_read(s, st, L.hc_ffn, m, true, true);   // applies the mixer's write first
}
// After the last layer: the output read, the head, the top-64 of every row.
static int sz_forward_head(sz_session* s, cudaStream_t st, int m, bool pending, bool read = true) {
    const sz_model_config& c = s->model.cfg;
    const int H = c.hidden;
    int rc;
    if (read && (rc = sz_hc_read(s, st, s->model.output_hc, m, pending, false))) return rc;
    if (s->head.rows > 0) return sz_head_top(&s->head, (uint64_t)s->u, H, m, 64, (uint64_t)s->logits, (uint64_t)s->top, (uint64_t)st);
    SzDenseArgs a = {};
    a.err = (u32*)(s->state + 2);
    a.x = s->u; a.xstride = H; a.cols = H; a.m = m; a.n_jobs = 1;
    a.job[0] = sz_job(s->model.output, s->logits, c.vocab);
    if ((rc = sz_dense_launch(a, st, "lm_head"))) return rc;
    const int nb = (c.vocab + SZ_TK_N - 1) / SZ_TK_N;
    SZ_CUDA(sz_launch("topk_slices", sz_topk_slices_kernel, dim3(nb, m), dim3(256), 0, st, true, (const float*)s->logits, (int)c.vocab, (int)c.vocab, nb, s->tk_tmp, (const u32*)nullptr));
    SZ_CUDA(sz_launch("topk_merge", sz_topk_merge_kernel, dim3(m), dim3(256), 0, st, true, (const u64*)s->tk_tmp, nb, s->top));
    return SZ_OK;
}
static int sz_forward(sz_session* s, cudaStream_t st, int m, bool head) {
    const sz_model_config& c = s->model.cfg;
    int rc = sz_forward_begin(s, st, m);
    if (rc) return rc;
    bool pending = false;
    for (int l = 0; l < c.n_layer; l++) {
        const sz_layer& L = s->layers[l];
        if ((rc = sz_layer_to_moe(s, st, l, m, pending))) return rc;
        int32_t* ri = s->want_routes ? s->routes + (int64_t)l * SZ_MAX_VERIFY * SZ_MAX_TOPK : nullptr;
        double* rw = s->want_routes ? s->route_w + (int64_t)l * SZ_MAX_VERIFY * SZ_MAX_TOPK : nullptr;
        if ((rc = sz_moe_verify(&L.moe, (uint64_t)s->u, m, (uint64_t)s->y, (uint64_t)ri, (uint64_t)rw, (uint64_t)s->moe_scratch, s->moe_scratch_bytes,
                                (uint64_t)st)))
            return rc;
        pending = true;
    }
    if (!head) return SZ_OK;  // the last write only matters to the output read; the next pass starts from the embedding
    return sz_forward_head(s, st, m, pending);
}

// The commit as the device does it: replay of the kept rows where some were dropped, conv rows, position count and buffer swap.
// All of it reads res[0] (rows kept) from device memory, so it can follow the acceptance kernel inside one graph.
static int sz_commit_device(sz_session* s, cudaStream_t st, int m) {
    const sz_model_config& c = s->model.cfg;
    if (s->n_delta > 0) {
        const int rc = sz_scan(s, st, -1, m, SzDeltaPrep());
        if (rc) return rc;
        const int64_t kd = (int64_t)c.ssm_k_heads * c.ssm_head_dim, vd = (int64_t)c.ssm_v_heads * c.ssm_head_dim, ch = 2 * kd + vd;
        SZ_CUDA(sz_launch("conv_commit", sz_conv_commit_kernel, dim3(c.conv_k - 1, s->n_delta), dim3(256), 0, st, true, (const float*)s->conv[0],
                          (const float*)s->conv[1], (const int32_t*)s->state, (const int32_t*)s->res, (const float*)s->d_xin, (int)ch, (int)c.conv_k,
                          s->conv[0], s->conv[1], s->tree_pass));
    }
    if (s->p_hist)   // the per-layer embedding's history and token tail as the kept rows leave them
        SZ_CUDA(sz_launch("ple_commit", sz_ple_commit_kernel, dim3((s->model.ple.conv_k - 1) * s->model.ple.ngram), dim3(256), 0, st, true, (const float*)s->p_gvn,
                          s->p_hist, (float*)((u8*)s->p_hist + s->p_hist_bytes), s->p_tail, (const int32_t*)s->ids, (const int32_t*)s->state, (const int32_t*)s->res,
                          (int)(c.streams * c.hidden), (int)((s->model.ple.conv_k - 1) * s->model.ple.ngram)));
    if (s->tree_pass && s->n_attn > 0) {   // the kept rows' keys and values from their rows' slots to their depths' slots
        const int hb = (s->flags & SZ_KV_Q8) ? (c.head_dim + (((c.head_dim >> 5) * 2 + 15) & ~15)) : 4 * c.head_dim;
        SZ_CUDA(sz_launch("kv_compact", sz_kv_compact_kernel, dim3(c.n_kv_head, s->n_attn, 2), dim3(128), 0, st, true, s->kc, s->vc, (const int32_t*)s->state,
                          (const int32_t*)s->res, s->ctx, (int)c.n_kv_head, hb));
    }
    SZ_CUDA(sz_launch("state_update", sz_state_update_kernel, dim3(1), dim3(32), 0, st, true, s->state, (const int32_t*)s->res));
    return SZ_OK;
}

// Everything a pass launches after the ids are on the device.
static int sz_pass_tail(sz_session* s, cudaStream_t st, int m, int accept_mode, int eog_token, bool head);
static int sz_pass(sz_session* s, cudaStream_t st, int m, int accept_mode, int eog_token, bool head) {
    int rc = sz_forward(s, st, m, head);
    if (rc) return rc;
    return sz_pass_tail(s, st, m, accept_mode, eog_token, head);
}
// Acceptance and commit on the device, after the rows' top-64 are there.
static int sz_pass_tail(sz_session* s, cudaStream_t st, int m, int accept_mode, int eog_token, bool head) {
    int rc = SZ_OK;
    if (accept_mode == SZ_ACCEPT_SAMPLED) {
        SZ_CUDA(sz_launch("accept_sampled", sz_accept_sampled_kernel, dim3(1), dim3(32 * SZ_MAX_VERIFY), 0, st, true, (const u32*)s->top,
                          (const int32_t*)s->ids, m, eog_token, (const SzSampleArgs*)(s->ids + 16), s->res));
        if ((rc = sz_commit_device(s, st, m))) return rc;
    } else if (accept_mode != SZ_ACCEPT_NONE && s->tree_pass) {
        SZ_CUDA(sz_launch("accept_tree", sz_accept_tree_kernel, dim3(1), dim3(32), 0, st, true, (const u32*)s->top, (const int32_t*)s->ids,
                          (const SzTree*)(s->ids + 32), m, eog_token, s->res));
        if ((rc = sz_commit_device(s, st, m))) return rc;
    } else if (accept_mode != SZ_ACCEPT_NONE) {
        SZ_CUDA(sz_launch("accept", sz_accept_greedy_kernel, dim3(1), dim3(32), 0, st, true, (const u32*)s->top, (const int32_t*)s->ids, m, eog_token,
                          accept_mode == SZ_ACCEPT_ALL ? 1 : 0, head ? 1 : 0, s->res));
        if ((rc = sz_commit_device(s, st, m))) return rc;
    }
    return SZ_OK;
}

static int sz_verify_impl(sz_session* s, const int32_t* ids, int m, int accept_mode, int eog_token, int want_head, uint64_t stream);

extern "C" int sz_session_verify(sz_session* s, const int32_t* ids, int m, int accept_mode, int eog_token, int want_head, uint64_t stream) {
    if (accept_mode < SZ_ACCEPT_NONE || accept_mode > SZ_ACCEPT_ALL) return sz_fail(SZ_E_ARG, "accept_mode %d (sampled acceptance: sz_session_verify_sampled)", accept_mode);
    if (s && !s->last_m) s->tree_pass = 0;
    return sz_verify_impl(s, ids, m, accept_mode, eog_token, want_head, stream);
}

// A pass over a draft tree: row 0 is the root (the pass's own token), row j > 0 a drafted token whose parent is row parents[j] < j.
// Row j attends to the committed positions, its ancestors and itself, sits at position committed + depth, and continues the
// recurrent state of its parent.
extern "C" int sz_session_verify_tree(sz_session* s, const int32_t* ids, const int32_t* parents, int m, int accept_mode, int eog_token, uint64_t stream) {
    if (!s || !ids || !parents) return sz_fail(SZ_E_ARG, "sz_session_verify_tree: null argument");
    if (accept_mode != SZ_ACCEPT_NONE && accept_mode != SZ_ACCEPT_GREEDY) return sz_fail(SZ_E_ARG, "a tree pass is accepted greedily on the device or by the caller (accept_mode %d)", accept_mode);
    if (m < 1 || m > SZ_MAX_VERIFY) return sz_fail(SZ_E_ARG, "a pass has 1..%d rows, got %d", SZ_MAX_VERIFY, m);
    if (s->last_m) return sz_fail(SZ_E_ARG, "the previous pass was not committed");
    if (parents[0] != -1) return sz_fail(SZ_E_ARG, "row 0 of a tree pass is the root: parents[0] must be -1");
    if (getenv("SZ_GENERIC_KERNELS") && atoi(getenv("SZ_GENERIC_KERNELS")) != 0) return sz_fail(SZ_E_ARG, "tree passes run on the fused DeltaNet front end only (SZ_GENERIC_KERNELS is set)");
    SzTree t = {};
    t.mask[0] = 1u;
    for (int j = 1; j < m; j++) {
        const int p = parents[j];
        if (p < 0 || p >= j) return sz_fail(SZ_E_ARG, "parents[%d] = %d: a row's parent comes before it", j, p);
        t.parents[j] = p;
        t.depth[j] = t.depth[p] + 1;
        t.mask[j] = t.mask[p] | (1u << j);
        if (p != j - 1) t.save |= 1u << p;
    }
    t.parents[0] = -1;
    if (s->inflight) { SZ_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); s->inflight = 0; }
    memcpy(s->h_pin + 32, &t, sizeof(t));
    s->tree_pass = 1;
    const int rc = sz_verify_impl(s, ids, m, accept_mode, eog_token, 1, stream);
    if (rc) s->tree_pass = 0;
    return rc;
}

// After sz_session_result of a tree pass that the device accepted: the kept rows, root first.
extern "C" int sz_session_tree_path(sz_session* s, int32_t* path, int* n, uint64_t stream) {
    if (!s || !path || !n) return sz_fail(SZ_E_ARG, "sz_session_tree_path: null argument");
    if (!s->last_m || !s->tree_pass || !s->pending_committed) return sz_fail(SZ_E_ARG, "sz_session_tree_path: no tree pass accepted on the device is pending");
    cudaStream_t st = (cudaStream_t)stream;
    SZ_CUDA(cudaMemcpyAsync(s->h_pin + 96, s->res, 64, cudaMemcpyDeviceToHost, st));
    SZ_CUDA(cudaStreamSynchronize(st));
    s->inflight = 0;
    *n = s->h_pin[96];
    if (*n < 1 || *n > s->last_m) return sz_fail(SZ_E_DEVICE, "the device reports a path of %d rows", *n);
    for (int i = 0; i < *n; i++) path[i] = s->h_pin[98 + i];
    return SZ_OK;
}

// Stop ids of the request: device acceptance never keeps a drafted one (as it never keeps the pass's end-of-generation id).
extern "C" int sz_session_set_stops(sz_session* s, const int32_t* ids, int n, uint64_t stream) {
    if (!s || n < 0 || n > 7 || (n > 0 && !ids)) return sz_fail(SZ_E_ARG, "sz_session_set_stops: 0..7 stop ids");
    if (s->inflight) { SZ_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); s->inflight = 0; }   // the staging block is free again
    s->h_pin[24] = n;
    for (int i = 0; i < 7; i++) s->h_pin[25 + i] = i < n ? ids[i] : -1;
    return SZ_OK;
}

extern "C" int sz_session_stops(const sz_session* s, int32_t* out) {   // the list as set (out: room for 7); returns how many
    if (!s || !out) return 0;
    const int n = s->h_pin[24];
    for (int i = 0; i < n; i++) out[i] = s->h_pin[25 + i];
    return n;
}

extern "C" int sz_session_set_sampler(sz_session* s, const sz_sampler* sp) {
    if (!s || !sp) return sz_fail(SZ_E_ARG, "sz_session_set_sampler: null argument");
    if (!(sp->temperature > 0.0f)) return sz_fail(SZ_E_ARG, "sz_session_set_sampler: temperature %g (greedy decoding is SZ_ACCEPT_GREEDY)", (double)sp->temperature);
    s->samp = *sp;
    s->has_samp = 1;
    return SZ_OK;
}

extern "C" int sz_session_verify_sampled(sz_session* s, const int32_t* ids, int m, uint64_t pos, int eog_token, uint64_t stream) {
    if (!s) return sz_fail(SZ_E_ARG, "null session or ids");
    if (!s->last_m) s->tree_pass = 0;
    if (!s->has_samp) return sz_fail(SZ_E_ARG, "sz_session_verify_sampled: no sampler set (sz_session_set_sampler)");
    if (s->inflight) { SZ_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); s->inflight = 0; }  // the staging block is free again
    SzSampleArgs a = {s->samp.temperature, s->samp.top_k, s->samp.top_p, s->samp.min_p, s->samp.seed, pos};
    static_assert(sizeof(SzSampleArgs) == 32, "the sampler block is eight words of the staging buffer");
    memcpy(s->h_pin + 16, &a, sizeof(a));
    return sz_verify_impl(s, ids, m, SZ_ACCEPT_SAMPLED, eog_token, 1, stream);
}

static int sz_verify_impl(sz_session* s, const int32_t* ids, int m, int accept_mode, int eog_token, int want_head, uint64_t stream) {
    if (!s || !ids) return sz_fail(SZ_E_ARG, "null session or ids");
    if (m < 1 || m > SZ_MAX_VERIFY) return sz_fail(SZ_E_ARG, "a pass has 1..%d rows, got %d", SZ_MAX_VERIFY, m);
    if (s->last_m) return sz_fail(SZ_E_ARG, "the previous pass was not committed");
    if (s->len + m > s->ctx) return sz_fail(SZ_E_ARG, "%d positions + %d rows exceed the session's capacity %d", s->len, m, s->ctx);
    if (accept_mode == SZ_ACCEPT_GREEDY && !want_head) return sz_fail(SZ_E_ARG, "greedy acceptance needs the head");
    cudaStream_t st = (cudaStream_t)stream;
    if (s->inflight) { SZ_CUDA(cudaStreamSynchronize(st)); s->inflight = 0; }
    memcpy(s->h_pin, ids, (size_t)m * 4);
    // the staging block: ids, (word 16) the sampler of a sampled pass, (word 24) the stop ids, (word 32) a tree pass's tables
    const size_t staged = s->tree_pass ? 128 + sizeof(SzTree) : 128;
    int rc = SZ_OK;
    // one graph per (rows, head, acceptance, eog): every launch-time value a kernel needs lives in device memory
    const int key = m | (want_head ? 16 : 0) | (accept_mode << 5) | (s->tree_pass ? 128 : 0) | ((eog_token & 0xfffff) << 8);
    bool traced = sz_trace_active();
    const bool capturable = st != (cudaStream_t)0 && st != cudaStreamLegacy && st != cudaStreamPerThread;  // the default stream cannot record
    if (s->use_graphs && capturable && !traced && !s->want_routes) {
        if (s->graph_gen != sz_ep_generation()) {  // recorded under another exchange set-up (or none): those launches no longer apply
            if (!s->graphs.empty()) SZ_CUDA(cudaStreamSynchronize(st));
            s->drop_graphs();
            s->graph_gen = sz_ep_generation();
        }
        auto it = s->graphs.find(key);
        if (it == s->graphs.end()) {
            // first use: run the pass eagerly (this also does every one-time function-attribute set-up), then record it for the next time
            SZ_CUDA(cudaMemcpyAsync(s->ids, s->h_pin, staged, cudaMemcpyHostToDevice, st));
            if ((rc = sz_pass(s, st, m, accept_mode, eog_token, want_head != 0))) return rc;
            cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone && s->graphs.size() < 64) {
                // record the same launches without running them
                cudaGraph_t g = nullptr;
                SZ_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
                cudaError_t e = cudaMemcpyAsync(s->ids, s->h_pin, staged, cudaMemcpyHostToDevice, st);
                int prc = e == cudaSuccess ? sz_pass(s, st, m, accept_mode, eog_token, want_head != 0) : SZ_E_CUDA;
                cudaError_t e2 = cudaStreamEndCapture(st, &g);
                if (prc == SZ_OK && e2 == cudaSuccess && g) {
                    cudaGraphExec_t ge = nullptr;
                    if (cudaGraphInstantiate(&ge, g, 0) == cudaSuccess) {
                        s->graphs[key] = ge;
                        if (sz_ep_p2p_world() > 0) { s->p2p_graphs++; sz_ep_p2p_graph_refs(1); }
                        else if (sz_ep_world() > 1) { s->ep_graphs++; sz_ep_graph_refs(1); }
                    }
                }
                if (g) cudaGraphDestroy(g);
                (void)cudaGetLastError();
            }
        } else {
            SZ_CUDA(cudaGraphLaunch(it->second, st));
        }
    } else {
        SZ_CUDA(cudaMemcpyAsync(s->ids, s->h_pin, staged, cudaMemcpyHostToDevice, st));
        if ((rc = sz_pass(s, st, m, accept_mode, eog_token, want_head != 0))) return rc;
    }
    s->last_m = m;
    s->pending_committed = accept_mode != SZ_ACCEPT_NONE;
    s->device_keep = accept_mode == SZ_ACCEPT_ALL ? m : -1;
    s->inflight = 1;
    return SZ_OK;
}

extern "C" int sz_session_result(sz_session* s, int32_t* keep_next, uint32_t* top, float* logits, uint64_t stream) {
    if (!s || !s->last_m) return sz_fail(SZ_E_ARG, "no pass to read");
    cudaStream_t st = (cudaStream_t)stream;
    SZ_CUDA(cudaMemcpyAsync(s->h_pin + 13, s->res, 8, cudaMemcpyDeviceToHost, st));
    if (top) SZ_CUDA(cudaMemcpyAsync(top, s->top, (size_t)s->last_m * 128 * 4, cudaMemcpyDeviceToHost, st));
    if (logits && s->head.k_blk > 0)
        return sz_fail(SZ_E_ARG, "sz_session_result: with the screened head (SZ_HEAD_PROXY) only the kept blocks have logits; ask for the top-64");
    if (logits) SZ_CUDA(cudaMemcpyAsync(logits, s->logits, (size_t)s->last_m * s->model.cfg.vocab * 4, cudaMemcpyDeviceToHost, st));
    s->h_pin[12] = 0;
    if (s->head.rows > 0) {
        uint64_t at = 0;
        int64_t nb = 0;
        const int hrc = sz_head_stage(&s->head, SZ_HEAD_ERR, &at, &nb);
        if (hrc) return hrc;
        SZ_CUDA(cudaMemcpyAsync(s->h_pin + 12, (const void*)at, 4, cudaMemcpyDeviceToHost, st));
    }
    // the error words the kernels raise when one of their bounded waits runs out: [10] the session's kernels, [11] the MoE kernels
    SZ_CUDA(cudaMemcpyAsync(s->h_pin + 10, s->state + 2, 4, cudaMemcpyDeviceToHost, st));
    SZ_CUDA(cudaMemcpyAsync(s->h_pin + 11, s->moe_scratch + 4, 4, cudaMemcpyDeviceToHost, st));
    SZ_CUDA(cudaStreamSynchronize(st));
    s->inflight = 0;
    if (keep_next) { keep_next[0] = s->h_pin[13]; keep_next[1] = s->h_pin[14]; }
    if (s->pending_committed) s->device_keep = s->h_pin[13];
    if (s->h_pin[10] || s->h_pin[11] || s->h_pin[12])
        return sz_fail(SZ_E_DEVICE, "a bounded wait on an asynchronous copy ran out (session word %d, MoE word %d, head word %d): the results of this pass are not valid",
                       s->h_pin[10], s->h_pin[11], s->h_pin[12]);
    return SZ_OK;
}

extern "C" int sz_session_routes(sz_session* s, int32_t* idx, double* w, uint64_t stream) {
    if (!s || !s->last_m || !s->want_routes) return sz_fail(SZ_E_ARG, "routes are recorded only after sz_session_trace_routes(1) and a pass");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t n = (size_t)s->model.cfg.n_layer * SZ_MAX_VERIFY * SZ_MAX_TOPK;
    if (idx) SZ_CUDA(cudaMemcpyAsync(idx, s->routes, n * 4, cudaMemcpyDeviceToHost, st));
    if (w) SZ_CUDA(cudaMemcpyAsync(w, s->route_w, n * 8, cudaMemcpyDeviceToHost, st));
    SZ_CUDA(cudaStreamSynchronize(st));
    return SZ_OK;
}

// Keeps the first `keep` rows of the pending pass: recurrent states of exactly those rows, conv rows, position count.  When the
// device already decided (acceptance modes GREEDY / ALL) `keep` must be what it kept, as sz_session_result reported.
extern "C" int sz_session_commit(sz_session* s, int keep, uint64_t stream) {
    if (!s || !s->last_m) return sz_fail(SZ_E_ARG, "no pass to commit");
    const int m = s->last_m;
    if (keep < 0 || keep > m) return sz_fail(SZ_E_ARG, "keep = %d of a pass of %d rows", keep, m);
    cudaStream_t st = (cudaStream_t)stream;
    if (s->tree_pass && !s->pending_committed) return sz_fail(SZ_E_ARG, "a tree pass is committed by its kept path: sz_session_commit_path");
    if (s->pending_committed) {
        // the device already advanced its state by the rows IT kept: the host's bookkeeping must follow that number, not the caller's
        if (s->device_keep < 0) return sz_fail(SZ_E_ARG, "the device decided this pass: read sz_session_result before sz_session_commit");
        if (keep != s->device_keep) return sz_fail(SZ_E_ARG, "keep = %d, but the device kept %d rows of this pass", keep, s->device_keep);
    } else {
        if (s->inflight) { SZ_CUDA(cudaStreamSynchronize(st)); s->inflight = 0; }
        s->h_pin[8] = keep;
        SZ_CUDA(cudaMemcpyAsync(s->res, s->h_pin + 8, 4, cudaMemcpyHostToDevice, st));
        const int rc = sz_commit_device(s, st, m);
        if (rc) return rc;
    }
    s->last_m = 0;
    s->pending_committed = 0;
    s->tree_pass = 0;
    if (keep > 0) { s->cur ^= 1; s->len += keep; }
    return SZ_OK;
}

// The caller's decision for a tree pass: the kept rows are `path` (root first, each the child of the one before).
extern "C" int sz_session_commit_path(sz_session* s, const int32_t* path, int n, uint64_t stream) {
    if (!s || !s->last_m || !s->tree_pass) return sz_fail(SZ_E_ARG, "no tree pass to commit");
    if (s->pending_committed) return sz_fail(SZ_E_ARG, "the device accepted this pass: sz_session_commit with the row count it kept");
    if (!path || n < 1 || n > s->last_m || path[0] != 0) return sz_fail(SZ_E_ARG, "a kept path starts at the root and has 1..%d rows", s->last_m);
    const SzTree* t = (const SzTree*)(s->h_pin + 32);
    for (int i = 1; i < n; i++)
        if (path[i] <= 0 || path[i] >= s->last_m || t->parents[path[i]] != path[i - 1]) return sz_fail(SZ_E_ARG, "path[%d] = %d is not a child of row %d", i, path[i], path[i - 1]);
    cudaStream_t st = (cudaStream_t)stream;
    if (s->inflight) { SZ_CUDA(cudaStreamSynchronize(st)); s->inflight = 0; }
    s->h_pin[96] = n; s->h_pin[97] = 0;
    for (int i = 0; i < n; i++) s->h_pin[98 + i] = path[i];
    SZ_CUDA(cudaMemcpyAsync(s->res, s->h_pin + 96, (size_t)(2 + n) * 4, cudaMemcpyHostToDevice, st));
    const int rc = sz_commit_device(s, st, s->last_m);
    if (rc) return rc;
    s->last_m = 0;
    s->tree_pass = 0;
    s->cur ^= 1; s->len += n;
    return SZ_OK;
}

// Feeds a prompt: passes of up to 8 rows, every row kept; the head runs for the last pass only.  Afterwards sz_session_result gives the
// top-64 (and logits) of the last pass's rows; the last row's are the prompt's.
extern "C" int sz_session_prefill(sz_session* s, const int32_t* ids, int n, uint64_t stream) {
    if (!s || !ids || n < 1) return sz_fail(SZ_E_ARG, "sz_session_prefill: nothing to feed");
    int done = 0;
    while (done < n) {
        const int m = n - done < SZ_MAX_VERIFY ? n - done : SZ_MAX_VERIFY;
        const bool last = done + m == n;
        int rc = sz_session_verify(s, ids + done, m, last ? SZ_ACCEPT_NONE : SZ_ACCEPT_ALL, -1, last ? 1 : 0, stream);
        if (rc) return rc;
        if (last) return SZ_OK;  // left pending so the caller can read the result, then commit all m rows
        if ((rc = sz_session_commit(s, m, stream))) return rc;
        done += m;
    }
    return SZ_OK;
}

// ---- several sequences in one step ---------------------------------------------------------------------------------------------------
// Config 5's batch, built from what is there: every sequence keeps its session (cache, recurrent states, buffers) and the
// sequences go through the layers in lockstep.  What reads the same weights for every sequence - the hyper-connection reads, the
// mixers' projections, the MoE sublayer - runs once over the rows of ALL sequences (an expert that several sequences chose is
// streamed and decoded once), and so do the DeltaNet scans of a layer; attention and the head stay launches of the sequence.  A
// sequence's numbers are those of a pass of its own, so acceptance, commit and the result are read session by session as after
// sz_session_verify.  Launched eagerly (no graph: the rows a step holds change from step to step).
#define SZ_BATCH_MAX 64
// A step of B sequences is up to some 400 launches a sequence (about 50 with the shared forms): issued by one host thread they
// can take longer than the GPU needs to run them.  A few worker threads (SZ_BATCH_THREADS, default 6; 0 = none) issue the sequences' own launches side by side, each on the
// sequences' own streams; what is shared is issued by the calling thread.  The workers live as long as the process.
namespace {
struct SzIssuePool {
    std::vector<std::thread> th;
    std::mutex mu;
    std::condition_variable cv, cv_done;
    std::function<void(int)> job;
    int n = 0, dev = 0;
    std::atomic<int> next{0};
    int done = 0;
    unsigned long long gen = 0;
    bool stop = false;
    explicit SzIssuePool(int workers) {
        for (int i = 0; i < workers; i++) th.emplace_back([this] { run(); });
    }
    ~SzIssuePool() {
        { std::lock_guard<std::mutex> lk(mu); stop = true; }
        cv.notify_all();
        for (auto& t : th) t.join();
    }
    void work() {
        for (;;) {
            const int i = next.fetch_add(1);
            if (i >= n) break;
            job(i);
            std::lock_guard<std::mutex> lk(mu);
            if (++done == n) cv_done.notify_all();
        }
    }
    void run() {
        unsigned long long seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu);
                cv.wait(lk, [&] { return stop || gen != seen; });
                if (stop) return;
                seen = gen;
            }
            cudaSetDevice(dev);
            work();
        }
    }
    // runs fn(0) .. fn(count - 1), the caller taking its share; returns when all are done
    void each(int count, int device, std::function<void(int)> fn) {
        if (th.empty() || count < 2) { for (int i = 0; i < count; i++) fn(i); return; }
        {
            std::lock_guard<std::mutex> lk(mu);
            job = std::move(fn); n = count; dev = device; done = 0; next.store(0); gen++;
        }
        cv.notify_all();
        work();
        std::unique_lock<std::mutex> lk(mu);
        cv_done.wait(lk, [&] { return done == n; });
    }
};
SzIssuePool& sz_issue_pool() {
    static SzIssuePool pool([] { const char* e = getenv("SZ_BATCH_THREADS"); const int w = e ? atoi(e) : 6; return w < 0 ? 0 : (w > 32 ? 32 : w); }());
    return pool;
}
}  // namespace

struct SzBatchTab {
    const float* u[SZ_BATCH_MAX];
    float* y[SZ_BATCH_MAX];
    int32_t m[SZ_BATCH_MAX], off[SZ_BATCH_MAX];
    int32_t n, pad[3];
};
// grid (rows), block 256: dir 0: X[off_b + j] = u_b[j]; dir 1: y_b[j] = Y[off_b + j]
static __global__ void __launch_bounds__(256)
sz_batch_rows_kernel(const SzBatchTab* __restrict__ T, float* __restrict__ X, int H, int dir) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int r = blockIdx.x;
    int b = 0;
    while (b + 1 < T->n && T->off[b + 1] <= r) b++;
    const int j = r - T->off[b];
    if (j >= T->m[b]) return;
    float4* x = (float4*)(X + (size_t)r * H);
    if (dir == 0) { const float4* src = (const float4*)(T->u[b] + (size_t)j * H); for (int i = threadIdx.x; i < H / 4; i += 256) x[i] = __ldcg(src + i); }
    else { float4* dst = (float4*)(T->y[b] + (size_t)j * H); for (int i = threadIdx.x; i < H / 4; i += 256) dst[i] = __ldcg(x + i); }
}

// The rows of a batch to and from buffers of the sequences' own: what[k] says where piece k of a row lives in the batch buffer
// (offset of the piece's block in floats, floats a row) and ptrs[(slot + k) * SZ_BATCH_MAX + b] where sequence b keeps it.
// grid (rows, pieces), block 256.  dir 0: batch <- sequences; dir 1: sequences <- batch.
struct SzBatchMove { long long off[SZ_DENSE_MAX_JOBS]; int32_t width[SZ_DENSE_MAX_JOBS]; };
static __global__ void __launch_bounds__(256)
sz_batch_move_kernel(const SzBatchTab* __restrict__ T, float* const* __restrict__ ptrs, SzBatchMove mv, float* __restrict__ X, int dir) {
    sz_pdl_wait();
    sz_pdl_trigger();
    const int r = blockIdx.x, k = blockIdx.y;
    int b = 0;
    while (b + 1 < T->n && T->off[b + 1] <= r) b++;
    const int j = r - T->off[b];
    if (j >= T->m[b]) return;
    const int w = mv.width[k];
    float* x = X + mv.off[k] + (size_t)r * w;
    float* p = ptrs[(size_t)k * SZ_BATCH_MAX + b] + (size_t)j * w;
    if (!(w & 3)) {
        if (dir == 0) for (int i = threadIdx.x; i < w / 4; i += 256) ((float4*)x)[i] = __ldcg((const float4*)p + i);
        else for (int i = threadIdx.x; i < w / 4; i += 256) ((float4*)p)[i] = __ldcg((const float4*)x + i);
    } else {
        if (dir == 0) for (int i = threadIdx.x; i < w; i += 256) x[i] = __ldcg(p + i);
        else for (int i = threadIdx.x; i < w; i += 256) p[i] = __ldcg(x + i);
    }
}

enum { SZ_BATCH_SLOTS = SZ_DENSE_MAX_JOBS + 1 };   // per layer: the outputs of the input projections, then the input of the output projection
struct SzBatchScratch { int64_t tab, ptrs, ptrs_bytes, scan, scan_bytes, x, y, r, r2, rn, acc, in, in_row, core, core_row, partial, partial_floats, moe, moe_bytes, total; };
static int sz_batch_layout(const sz_model* m, int rows_max, SzBatchScratch* S) {
    if (!m || !m->layers) return sz_fail(SZ_E_ARG, "null model");
    if (rows_max < 8 || rows_max % 8) return sz_fail(SZ_E_ARG, "sz_batch: rows_max = %d (a multiple of 8)", rows_max);
    const sz_model_config& c = m->cfg;
    int64_t o = 0, mb = 0;
    S->tab = o; o = up256(o + (int64_t)sizeof(SzBatchTab));
    S->ptrs_bytes = (int64_t)c.n_layer * SZ_BATCH_SLOTS * SZ_BATCH_MAX * (int64_t)sizeof(float*);
    S->ptrs = o; o = up256(o + S->ptrs_bytes);
    int n_delta = 0;
    for (int l = 0; l < c.n_layer; l++) n_delta += sz_is_attn(c, l) ? 0 : 1;
    S->scan_bytes = (int64_t)n_delta * SZ_BATCH_MAX * (int64_t)sizeof(SzScanSeq);   // the many-sequence scan's table: [DeltaNet layer][sequence]
    S->scan = o; o = up256(o + S->scan_bytes);
    S->x = o; o = up256(o + 4 * (int64_t)rows_max * c.hidden);
    S->y = o; o = up256(o + 4 * (int64_t)rows_max * c.hidden);
    // the residual streams, their normed copy and the accumulators of the fused reads, for the rows of all sequences
    const int64_t CH = (int64_t)c.streams * c.hidden;
    S->r = o; o = up256(o + 4 * rows_max * CH);
    S->r2 = o; o = up256(o + 4 * rows_max * CH);
    S->rn = o; o = up256(o + 4 * rows_max * CH);
    S->acc = o; o = up256(o + 8 * 3 * (int64_t)rows_max * SZ_HC_ACC_ROWS);
    // a row of the mixers' projections: the wider of the two kinds of layer
    const int64_t kd = (int64_t)c.ssm_k_heads * c.ssm_head_dim, vd = (int64_t)c.ssm_v_heads * c.ssm_head_dim;
    const int64_t in_d = 2 * kd + vd + vd + 2 * c.ssm_v_heads;
    const int64_t in_a = 2 * (int64_t)c.n_head * c.head_dim + 2 * (int64_t)c.n_kv_head * c.head_dim + (int64_t)c.idx_heads * c.idx_dim + c.idx_dim;
    S->in_row = (in_d > in_a ? in_d : in_a);
    S->core_row = vd > (int64_t)c.n_head * c.head_dim ? vd : (int64_t)c.n_head * c.head_dim;
    S->in = o; o = up256(o + 4 * rows_max * S->in_row);
    S->core = o; o = up256(o + 4 * rows_max * S->core_row);
    // the many-row projection kernel's sums of the eight column parts, for the widest set of projections
    S->partial_floats = 8 * (int64_t)rows_max * (S->in_row > c.hidden ? S->in_row : c.hidden);
    S->partial = o; o = up256(o + 4 * S->partial_floats);
    for (int l = 0; l < c.n_layer; l++) {
        int64_t b = 0;
        const int rc = sz_moe_rows_scratch_bytes(&m->layers[l].moe, rows_max, &b);
        if (rc) return rc;
        mb = b > mb ? b : mb;
    }
    S->moe = o; S->moe_bytes = mb; o = up256(o + mb);
    S->total = o;
    return SZ_OK;
}
extern "C" int sz_batch_scratch_bytes(const sz_model* m, int rows_max, int64_t* bytes) {
    SzBatchScratch S;
    const int rc = sz_batch_layout(m, rows_max, &S);
    if (rc) return rc;
    if (!bytes) return sz_fail(SZ_E_ARG, "null bytes");
    *bytes = S.total;
    return SZ_OK;
}
// Once after the scratch is allocated (and after a failed step).
extern "C" int sz_batch_scratch_init(const sz_model* m, int rows_max, uint64_t scratch, uint64_t stream) {
    SzBatchScratch S;
    int rc = sz_batch_layout(m, rows_max, &S);
    if (rc) return rc;
    if (!scratch || (scratch & 255)) return sz_fail(SZ_E_ARG, "scratch must be 256-byte aligned");
    SZ_CUDA(cudaMemsetAsync((void*)(scratch + S.x), 0, (size_t)(S.moe - S.x), (cudaStream_t)stream));
    return sz_moe_rows_status(&m->layers[0].moe, rows_max, scratch + S.moe, nullptr, stream);
}

// One step of n sequences: sequence b reads ms[b] rows (ids: the rows of all sequences, one after the other).  accept_mode:
// SZ_ACCEPT_NONE, _GREEDY or _ALL, as sz_session_verify.  Afterwards every session holds a pending pass: sz_session_result and
// sz_session_commit per session, as after a pass of its own.
// (accept[b], heads[b]: sequence b's acceptance mode and whether its rows go through the head - a prompt's passes before its last
// keep all rows and need no logits)
static int sz_batch_step(sz_session* const* ss, int n, const int32_t* ids, const int32_t* ms, const int* accept, const int* heads, int eog_token,
                         int rows_max, uint64_t scratch, int64_t scratch_bytes, uint64_t stream) {
    if (!ss || !ids || !ms || n < 1 || n > SZ_BATCH_MAX) return sz_fail(SZ_E_ARG, "sz_batch_verify: 1..%d sequences", SZ_BATCH_MAX);
    bool any_head = false;
    for (int b = 0; b < n; b++) {
        if (accept[b] < SZ_ACCEPT_NONE || accept[b] > SZ_ACCEPT_ALL) return sz_fail(SZ_E_ARG, "sz_batch_verify: accept_mode %d", accept[b]);
        if (!heads[b] && accept[b] != SZ_ACCEPT_ALL) return sz_fail(SZ_E_ARG, "sz_batch_verify: a pass without the head keeps all its rows");
        any_head = any_head || heads[b];
    }
    sz_session* s0 = ss[0];
    if (!s0) return sz_fail(SZ_E_ARG, "sz_batch_verify: null session");
    SzBatchScratch S;
    int rc = sz_batch_layout(&s0->model, rows_max, &S);
    if (rc) return rc;
    if (!scratch || (scratch & 255) || scratch_bytes < S.total) return sz_fail(SZ_E_SCRATCH, "sz_batch_verify: scratch of %lld bytes, %lld needed", (long long)scratch_bytes, (long long)S.total);
    cudaStream_t st = (cudaStream_t)stream;
    const sz_model_config& c = s0->model.cfg;
    SzBatchTab tab = {};
    int R = 0;
    for (int b = 0; b < n; b++) {
        sz_session* s = ss[b];
        if (!s || s->model.layers[0].moe.gate != s0->model.layers[0].moe.gate || s->model.cfg.n_layer != c.n_layer)
            return sz_fail(SZ_E_ARG, "sz_batch_verify: sequence %d is not a session of the same model", b);
        for (int q = 0; q < b; q++) if (ss[q] == s) return sz_fail(SZ_E_ARG, "sz_batch_verify: a session appears twice");
        const int m = ms[b];
        if (m < 1 || m > SZ_MAX_VERIFY) return sz_fail(SZ_E_ARG, "a pass has 1..%d rows, got %d", SZ_MAX_VERIFY, m);
        if (s->last_m) return sz_fail(SZ_E_ARG, "sequence %d: the previous pass was not committed", b);
        if (s->len + m > s->ctx) return sz_fail(SZ_E_ARG, "sequence %d: %d positions + %d rows exceed the session's capacity %d", b, s->len, m, s->ctx);
        if (s->want_routes) return sz_fail(SZ_E_ARG, "sz_batch_verify: no routing trace in a batched step");
        tab.u[b] = s->u; tab.y[b] = s->y; tab.m[b] = m; tab.off[b] = R;
        R += m;
    }
    tab.n = n;
    const int Rp = (R + 7) & ~7;
    if (Rp > rows_max) return sz_fail(SZ_E_ARG, "sz_batch_verify: %d rows in a scratch for %d", R, rows_max);
    // the ids of every sequence into its session's staging block (pinned: the copy is asynchronous)
    int at = 0;
    for (int b = 0; b < n; b++) {
        sz_session* s = ss[b];
        if (s->inflight) { SZ_CUDA(cudaStreamSynchronize(st)); s->inflight = 0; }
        s->tree_pass = 0;
        memcpy(s->h_pin, ids + at, (size_t)ms[b] * 4);
        at += ms[b];
        SZ_CUDA(cudaMemcpyAsync(s->ids, s->h_pin, 128, cudaMemcpyHostToDevice, st));
    }
    u8* base = (u8*)scratch;
    SZ_CUDA(cudaMemcpyAsync(base + S.tab, &tab, sizeof(tab), cudaMemcpyHostToDevice, st));   // (pageable: staged before the call returns)
    float *X = (float*)(base + S.x), *Y = (float*)(base + S.y), *IN = (float*)(base + S.in), *CORE = (float*)(base + S.core);
    // What reads the same weights for every sequence runs once over the rows of all of them (`shared`): the hyper-connection reads
    // and the mixers' projections, besides the MoE sublayers.  The sequences' residual streams, mixer outputs and sublayer inputs
    // then live side by side in buffers of the batch - for the length of the step every session points into them, so that its own
    // kernels (embedding, per-layer embedding, scan, attention, head) find their rows where they always do - and the shared kernels
    // take eight rows a block row or a launch, the very kernels of a lone pass: a row's result does not depend on the rows beside
    // it.  Only what carries a sequence's own state stays a launch per sequence.  SZ_BATCH_SHARED=0: only the MoE is shared.
    const char* se = getenv("SZ_BATCH_SHARED");   // (read at every step: a test switches it inside one process)
    const bool shared_off = se && atoi(se) == 0;
    const bool shared = !shared_off && n > 1 && s0->hc_fast;
    const int64_t CH = (int64_t)c.streams * c.hidden;
    SzBatchBufs BB = {(float*)(base + S.r), (float*)(base + S.r2), Y, X, (float*)(base + S.rn), (long long*)(base + S.acc), (int64_t)rows_max * SZ_HC_ACC_ROWS};
    struct Repoint {   // the sessions' buffers while they point into the batch's: put back however the step ends
        sz_session* const* ss = nullptr;
        int n = 0;
        struct { float *r, *r2, *y, *u, *rn; long long* acc; int64_t stride; } was[SZ_BATCH_MAX];
        ~Repoint() {
            for (int b = 0; b < n; b++) {
                sz_session* s = ss[b];
                s->r = was[b].r; s->r2 = was[b].r2; s->y = was[b].y; s->u = was[b].u; s->rn = was[b].rn; s->hc_acc = was[b].acc; s->hc_acc_stride = was[b].stride;
            }
        }
    } repoint;
    float* const* ptrs = (float* const*)(base + S.ptrs);
    float* PART = (float*)(base + S.partial);
    const char* re = getenv("SZ_BATCH_DENSE_ROWS");   // 0: the projections 8 rows a launch (the second form; same bits)
    const bool rows_form = !(re && atoi(re) == 0);
    // the DeltaNet scans of a layer, all sequences in one launch from a table of their pointers (0, or the generic kernels: a launch
    // a sequence on its stream; same bits)
    const char* sc = getenv("SZ_BATCH_SCAN_SEQS");
    const char* ge = getenv("SZ_GENERIC_KERNELS");
    const bool scan_seqs = !(sc && atoi(sc) == 0) && !(ge && atoi(ge) != 0);
    if (shared) {
        repoint.ss = ss;
        for (int b = 0; b < n; b++) {
            sz_session* s = ss[b];
            repoint.was[b] = {s->r, s->r2, s->y, s->u, s->rn, s->hc_acc, s->hc_acc_stride};
            repoint.n = b + 1;
            const int64_t o = tab.off[b];
            s->r = BB.r + o * CH; s->r2 = BB.r2 + o * CH; s->y = BB.y + o * c.hidden; s->u = BB.u + o * c.hidden; s->rn = BB.rn + o * CH;
            s->hc_acc = BB.acc + o * SZ_HC_ACC_ROWS; s->hc_acc_stride = BB.acc_stride;
        }
        static thread_local std::vector<float*> host;   // where every sequence keeps the projections' outputs and the output projection's input
        host.assign((size_t)c.n_layer * SZ_BATCH_SLOTS * SZ_BATCH_MAX, nullptr);
        for (int l = 0; l < c.n_layer; l++)
            for (int b = 0; b < n; b++) {
                SzDenseArgs a, o;
                sz_mixer_args(ss[b], l, ms[b], &a, &o);
                float** row = host.data() + (size_t)l * SZ_BATCH_SLOTS * SZ_BATCH_MAX;
                for (int k = 0; k < a.n_jobs; k++) row[(size_t)k * SZ_BATCH_MAX + b] = a.job[k].out;
                row[(size_t)SZ_DENSE_MAX_JOBS * SZ_BATCH_MAX + b] = const_cast<float*>(o.x);
            }
        SZ_CUDA(cudaMemcpyAsync(base + S.ptrs, host.data(), (size_t)S.ptrs_bytes, cudaMemcpyHostToDevice, st));   // (pageable, as the table)
        if (scan_seqs) {
            static thread_local std::vector<SzScanSeq> hs;
            hs.assign((size_t)(S.scan_bytes / sizeof(SzScanSeq)), SzScanSeq{});
            for (int l = 0; l < c.n_layer; l++)
                if (!sz_is_attn(c, l))
                    for (int b = 0; b < n; b++) sz_scan_seq_entry(ss[b], l, ms[b], &hs[(size_t)s0->lb[l].delta_index * SZ_BATCH_MAX + b]);
            SZ_CUDA(cudaMemcpyAsync(base + S.scan, hs.data(), (size_t)S.scan_bytes, cudaMemcpyHostToDevice, st));
        }
        SZ_CUDA(cudaMemsetAsync(BB.acc, 0, sizeof(long long) * (size_t)Rp * SZ_HC_ACC_ROWS, st));   // read 0 adds into accumulator 0
    }
    if (Rp > R && !shared) SZ_CUDA(cudaMemsetAsync(X + (size_t)R * c.hidden, 0, (size_t)(Rp - R) * c.hidden * 4, st));   // the rows that pad the batch to a multiple of 8
    // The sequences' own kernels are chains of short dependent launches: on one stream they would run one sequence after the other
    // and leave the GPU as idle as a lone pass does.  So every sequence gets a stream of its own for them (a pool owned by the
    // calling thread, made at the first call), and the caller's stream carries what is shared: it lets the sequences' streams go
    // where a layer has work of their own (attention; everything but the MoE when nothing else is shared), waits for them, and
    // goes on with the rows of all.  SZ_BATCH_STREAMS=0: everything on the caller's stream.
    static thread_local cudaStream_t pool[SZ_BATCH_MAX] = {};
    static thread_local cudaEvent_t pool_ev[SZ_BATCH_MAX] = {};
    static thread_local cudaEvent_t main_ev = nullptr;
    static const bool streams_off = getenv("SZ_BATCH_STREAMS") && atoi(getenv("SZ_BATCH_STREAMS")) == 0;
    const bool multi = !streams_off && n > 1;
    if (multi) {
        if (!main_ev) SZ_CUDA(cudaEventCreateWithFlags(&main_ev, cudaEventDisableTiming));
        for (int b = 0; b < n; b++)
            if (!pool[b]) {
                SZ_CUDA(cudaStreamCreateWithFlags(&pool[b], cudaStreamNonBlocking));
                SZ_CUDA(cudaEventCreateWithFlags(&pool_ev[b], cudaEventDisableTiming));
            }
    }
    cudaStream_t* const pl = pool;          // (a worker thread that named `pool` would get its own, empty, thread-local array)
    cudaEvent_t* const pe = pool_ev;
    const cudaEvent_t mev = main_ev;
    auto sq = [&, pl](int b) { return multi ? pl[b] : st; };
    auto fork = [&]() -> int {      // the sequences' streams continue after what the caller's stream has done so far
        if (!multi) return SZ_OK;
        SZ_CUDA(cudaEventRecord(mev, st));
        for (int b = 0; b < n; b++) SZ_CUDA(cudaStreamWaitEvent(pl[b], mev, 0));
        return SZ_OK;
    };
    auto join = [&]() -> int {      // the caller's stream continues after every sequence's stream
        if (!multi) return SZ_OK;
        for (int b = 0; b < n; b++) {
            SZ_CUDA(cudaEventRecord(pe[b], pl[b]));
            SZ_CUDA(cudaStreamWaitEvent(st, pe[b], 0));
        }
        return SZ_OK;
    };
    int dev = 0;
    SZ_CUDA(cudaGetDevice(&dev));
    SzIssuePool& workers = sz_issue_pool();
    std::atomic<int> worst{SZ_OK};   // (a failing launch: the first code is kept; its message is the last one written)
    auto each = [&](const std::function<int(int)>& fn) -> int {
        if (!multi) { for (int b = 0; b < n; b++) { const int r = fn(b); if (r) return r; } return SZ_OK; }
        workers.each(n, dev, [&](int b) { const int r = fn(b); if (r) { int z = SZ_OK; worst.compare_exchange_strong(z, r); } });
        return worst.load();
    };
    if ((rc = fork())) return rc;
    if ((rc = each([&](int b) { return sz_forward_begin(ss[b], sq(b), ms[b], !shared); }))) return rc;
    bool pending = false;
    const SzBatchTab* T = (const SzBatchTab*)(base + S.tab);
    if (shared) {
        int hn = 0;   // hyper-connection reads so far (every session's count follows: the per-layer embedding looks at it)
        auto read_rows = [&](const sz_hc& hc, bool pend, bool inject, bool pdl) -> int {
            const int r = sz_hc_read_rows(s0, st, hc, Rp, hn++, pend, inject, BB, pdl);
            for (int b = 0; b < n; b++) ss[b]->hc_n = hn;
            return r;
        };
        for (int l = 0; l < c.n_layer; l++) {
            const sz_layer& L = s0->layers[l];
            const bool ple_here = s0->p_hist && l == s0->model.ple.layer;
            bool pend = pending;
            if (ple_here) {   // (it applies the pending write itself, on the sequence's rows of the shared buffers)
                if (l > 0 && (rc = fork())) return rc;
                if ((rc = each([&](int b) { return sz_ple_layer(ss[b], sq(b), ms[b], pending); }))) return rc;
                pend = false;
            }
            const bool joined = l == 0 || ple_here;
            if (joined && (rc = join())) return rc;
            if ((rc = read_rows(L.hc_attn, pend, true, !(joined && multi)))) return rc;
            float* const* lp = ptrs + (size_t)l * SZ_BATCH_SLOTS * SZ_BATCH_MAX;
            SzDenseArgs a, o;
            sz_mixer_args(s0, l, 8, &a, &o);
            SzBatchMove mi = {}, mo = {};
            long long at_in = 0;
            for (int k = 0; k < a.n_jobs; k++) { mi.off[k] = at_in; mi.width[k] = a.job[k].ostride; at_in += (long long)Rp * a.job[k].ostride; }
            mo.off[0] = 0; mo.width[0] = o.cols;
            {   // all rows through one launch where the many-row form of the kernel exists, else 8 rows a launch
                SzDenseArgs ar = a;
                ar.m = Rp; ar.x = X;
                for (int k = 0; k < a.n_jobs; k++) ar.job[k].out = IN + mi.off[k];
                int taken = 0;
                if (rows_form && (rc = sz_dense_rows_launch(ar, PART, S.partial_floats, st, "batch_proj", &taken))) return rc;
                for (int g = 0; g < Rp / 8 && !taken; g++) {
                    SzDenseArgs ag = a;
                    ag.x = X + (size_t)g * 8 * c.hidden;
                    for (int k = 0; k < a.n_jobs; k++) ag.job[k].out = IN + mi.off[k] + (size_t)g * 8 * mi.width[k];
                    if ((rc = sz_dense_launch(ag, st, "batch_proj"))) return rc;
                }
            }
            SZ_CUDA(sz_launch("batch_move", sz_batch_move_kernel, dim3(R, a.n_jobs), dim3(256), 0, st, true, T, lp, mi, IN, 1));
            const bool one_scan = scan_seqs && !sz_is_attn(c, l);
            if (one_scan) {   // the whole layer stays on the caller's stream
                if ((rc = sz_scan_seqs(s0, st, l, n, (const SzScanSeq*)(base + S.scan) + (size_t)s0->lb[l].delta_index * SZ_BATCH_MAX, true))) return rc;
            } else {
                if ((rc = fork())) return rc;
                if ((rc = each([&](int b) {
                        return sz_is_attn(c, l) ? sz_attn_layer(ss[b], sq(b), l, ms[b], SZ_MIX_CORE) : sz_delta_layer(ss[b], sq(b), l, ms[b], SZ_MIX_CORE);
                    })))
                    return rc;
                if ((rc = join())) return rc;
            }
            SZ_CUDA(sz_launch("batch_move", sz_batch_move_kernel, dim3(R, 1), dim3(256), 0, st, one_scan || !multi, T, lp + (size_t)SZ_DENSE_MAX_JOBS * SZ_BATCH_MAX, mo, CORE, 0));
            {
                SzDenseArgs orr = o;
                orr.m = Rp; orr.x = CORE; orr.job[0].out = Y;
                int taken = 0;
                if (rows_form && (rc = sz_dense_rows_launch(orr, PART, S.partial_floats, st, "batch_out", &taken))) return rc;
                for (int g = 0; g < Rp / 8 && !taken; g++) {
                    SzDenseArgs og = o;
                    og.x = CORE + (size_t)g * 8 * o.cols;
                    og.job[0].out = Y + (size_t)g * 8 * c.hidden;
                    if ((rc = sz_dense_launch(og, st, "batch_out"))) return rc;
                }
            }
            if ((rc = read_rows(L.hc_ffn, true, true, true))) return rc;
            if ((rc = sz_moe_rows(&L.moe, (uint64_t)X, Rp, (uint64_t)Y, 0, 0, scratch + S.moe, S.moe_bytes, stream))) return rc;
            pending = true;
        }
        if (any_head && (rc = read_rows(s0->model.output_hc, pending, false, true))) return rc;
        if ((rc = fork())) return rc;
    } else {
        for (int l = 0; l < c.n_layer; l++) {
            if ((rc = each([&](int b) { return sz_layer_to_moe(ss[b], sq(b), l, ms[b], pending); }))) return rc;
            if ((rc = join())) return rc;
            SZ_CUDA(sz_launch("batch_gather", sz_batch_rows_kernel, dim3(R), dim3(256), 0, st, !multi, T, X, (int)c.hidden, 0));
            if ((rc = sz_moe_rows(&s0->layers[l].moe, (uint64_t)X, Rp, (uint64_t)Y, 0, 0, scratch + S.moe, S.moe_bytes, stream))) return rc;
            SZ_CUDA(sz_launch("batch_scatter", sz_batch_rows_kernel, dim3(R), dim3(256), 0, st, true, T, Y, (int)c.hidden, 1));
            if ((rc = fork())) return rc;
            pending = true;
        }
    }
    if ((rc = each([&](int b) {
            sz_session* s = ss[b];
            int r = heads[b] ? sz_forward_head(s, sq(b), ms[b], pending, !shared) : SZ_OK;
            if (!r) r = sz_pass_tail(s, sq(b), ms[b], accept[b], eog_token, heads[b] != 0);
            return r;
        })))
        return rc;
    for (int b = 0; b < n; b++) {
        sz_session* s = ss[b];
        s->last_m = ms[b];
        s->pending_committed = accept[b] != SZ_ACCEPT_NONE;
        s->device_keep = accept[b] == SZ_ACCEPT_ALL ? ms[b] : -1;
        s->inflight = 1;
    }
    return join();
}

extern "C" int sz_batch_verify(sz_session* const* ss, int n, const int32_t* ids, const int32_t* ms, int accept_mode, int eog_token, int rows_max,
                               uint64_t scratch, int64_t scratch_bytes, uint64_t stream) {
    if (n < 1 || n > SZ_BATCH_MAX) return sz_fail(SZ_E_ARG, "sz_batch_verify: 1..%d sequences", SZ_BATCH_MAX);
    int accept[SZ_BATCH_MAX], heads[SZ_BATCH_MAX];
    for (int b = 0; b < n; b++) { accept[b] = accept_mode; heads[b] = 1; }
    return sz_batch_step(ss, n, ids, ms, accept, heads, eog_token, rows_max, scratch, scratch_bytes, stream);
}

// The prompts of n sequences fed in lockstep: every step takes up to 8 rows of every sequence that still has some (as many
// sequences a step as the scratch's rows hold), keeps them all, and skips the head except for a prompt's last pass - which is left
// pending, as sz_session_prefill leaves it: sz_session_result, then sz_session_commit of its rows (lens[b] - 1) % 8 + 1.
extern "C" int sz_batch_prefill(sz_session* const* ss, int n, const int32_t* const* ids, const int32_t* lens, int rows_max, uint64_t scratch,
                                int64_t scratch_bytes, uint64_t stream) {
    if (!ss || !ids || !lens || n < 1 || n > SZ_BATCH_MAX) return sz_fail(SZ_E_ARG, "sz_batch_prefill: 1..%d sequences", SZ_BATCH_MAX);
    if (rows_max < SZ_MAX_VERIFY) return sz_fail(SZ_E_ARG, "sz_batch_prefill: a scratch for %d rows", rows_max);
    std::vector<int> done((size_t)n, 0);
    for (int b = 0; b < n; b++)
        if (!ss[b] || !ids[b] || lens[b] < 1) return sz_fail(SZ_E_ARG, "sz_batch_prefill: sequence %d has nothing to feed", b);
    for (;;) {
        sz_session* step_s[SZ_BATCH_MAX];
        int32_t step_m[SZ_BATCH_MAX];
        int accept[SZ_BATCH_MAX], heads[SZ_BATCH_MAX], who[SZ_BATCH_MAX];
        std::vector<int32_t> rows;
        int k = 0;
        for (int b = 0; b < n && (k + 1) * SZ_MAX_VERIFY <= rows_max; b++) {
            if (done[b] >= lens[b]) continue;
            const int left = lens[b] - done[b];
            const int m = left < SZ_MAX_VERIFY ? left : SZ_MAX_VERIFY;
            const bool last = m == left;
            step_s[k] = ss[b]; step_m[k] = m; who[k] = b;
            accept[k] = last ? SZ_ACCEPT_NONE : SZ_ACCEPT_ALL;
            heads[k] = last ? 1 : 0;
            rows.insert(rows.end(), ids[b] + done[b], ids[b] + done[b] + m);
            k++;
        }
        if (k == 0) return SZ_OK;
        int rc = sz_batch_step(step_s, k, rows.data(), step_m, accept, heads, -1, rows_max, scratch, scratch_bytes, stream);
        if (rc) return rc;
        for (int i = 0; i < k; i++) {
            const int b = who[i];
            done[b] += step_m[i];
            if (done[b] < lens[b] && (rc = sz_session_commit(step_s[i], step_m[i], stream))) return rc;   // (a prompt's last pass stays pending)
        }
    }
}

// ---- synthetic history (benchmarks) -------------------------------------------------------------------------------------------------
// Fills the first `len` positions of every attention layer's cache with seeded pseudo-random keys and values (and small random
// DeltaNet states), as if `len` tokens had been fed: a long context without running a long prefill.
__global__ void sz_fill_kv_kernel(u8* __restrict__ kc, int len, int ctx, int nkv, int64_t layer_stride, int hd, int q8, u32 seed) {
    const int layer = blockIdx.y;
    u8* base = kc + layer * layer_stride;
    const int hb = q8 ? sz_kv_head_bytes(hd) : hd * 4;
    const int64_t heads = (int64_t)nkv * len;
    for (int64_t hp = blockIdx.x; hp < heads; hp += gridDim.x) {
        const int64_t h = hp / len, pos = hp % len;
        u8* p = base + (h * ctx + pos) * hb;
        for (int i = threadIdx.x; i < hd; i += blockDim.x) {
            u32 x = (u32)(hp * 2654435761u) ^ (u32)(i * 40503u) ^ seed ^ (u32)(layer * 97u);
            x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
            if (q8) p[i] = (u8)(int8_t)((int)(x % 255u) - 127);
            else ((float*)p)[i] = ((float)(x % 2001u) - 1000.0f) * 1e-3f;
        }
        if (q8) {
            u16* sc = (u16*)(p + hd);
            for (int g = threadIdx.x; g < (hb - hd) / 2; g += blockDim.x) sc[g] = g < hd / 32 ? (u16)0x2000 : (u16)0;  // f16 2^-7
        }
    }
}

extern "C" int sz_session_fill_synthetic(sz_session* s, int len, uint32_t seed, uint64_t stream) {
    if (!s || s->last_m) return sz_fail(SZ_E_ARG, "sz_session_fill_synthetic: null session or a pass is pending");
    if (len < 0 || len + SZ_MAX_VERIFY > s->ctx) return sz_fail(SZ_E_ARG, "sz_session_fill_synthetic: %d positions in a session of %d", len, s->ctx);
    cudaStream_t st = (cudaStream_t)stream;
    const sz_model_config& c = s->model.cfg;
    int rc = sz_session_reset(s, stream);
    if (rc) return rc;
    if (s->n_attn > 0 && len > 0) {
        const int q8 = (s->flags & SZ_KV_Q8) ? 1 : 0;
        const int64_t hb = q8 ? (c.head_dim + (((c.head_dim >> 5) * 2 + 15) & ~15)) : 4 * (int64_t)c.head_dim;
        const int64_t stride = (int64_t)s->ctx * c.n_kv_head * hb;
        sz_fill_kv_kernel<<<dim3(1024, s->n_attn), 128, 0, st>>>(s->kc, len, s->ctx, (int)c.n_kv_head, stride, (int)c.head_dim, q8, seed);
        sz_fill_kv_kernel<<<dim3(1024, s->n_attn), 128, 0, st>>>(s->vc, len, s->ctx, (int)c.n_kv_head, stride, (int)c.head_dim, q8, seed ^ 0x9e3779b9u);
        SZ_CUDA(cudaGetLastError());
        if (s->i_raw) {   // the indexer's raw keys of the history and the pooled key of every complete block
            sz_idx_fill_kernel<<<dim3(1024, s->n_attn), 128, 0, st>>>(s->i_raw, (long long)(s->i_raw_layer / 4), len, (int)c.idx_dim, seed ^ 0x51ed270bu);
            for (int l = 0; l < c.n_layer; l++) {
                if (!sz_is_attn(c, l)) continue;
                const int ai = s->lb[l].attn_index, ratio = s->layers[l].idx_ratio > 0 ? s->layers[l].idx_ratio : 1;
                if (len / ratio > 0)
                    sz_idx_rebuild_kernel<<<len / ratio, 128, 0, st>>>((const float*)((u8*)s->i_raw + ai * s->i_raw_layer), (const float*)s->layers[l].idx_k_norm.data,
                                                                       (int)c.idx_dim, ratio, c.eps, (int)c.rope_dims, (const double*)s->rope_den,
                                                                       (float*)((u8*)s->i_blocks + ai * s->i_blocks_layer));
            }
            SZ_CUDA(cudaGetLastError());
        }
    }
    s->h_pin[8] = len;
    SZ_CUDA(cudaMemcpyAsync(s->state, s->h_pin + 8, 4, cudaMemcpyHostToDevice, st));
    SZ_CUDA(cudaStreamSynchronize(st));
    s->len = len;
    return SZ_OK;
}

// ---- committed state to the host ------------------------------------------------------------------------------------------------------
// What GpuSession::snapshot (crates/shadowzero-cuda/src/session.rs:3407-3459) copies, one piece at a time: the recurrent state and the
// carried conv rows of a DeltaNet layer (the current buffer), or the cache rows of an attention layer in the reference's order
// [position][kv head][head bytes] (the library keeps them per KV head).  No pass may be pending.
extern "C" int sz_session_idx_words(const sz_session* s) { return s ? s->i_words : -1; }

extern "C" int sz_session_export(sz_session* s, int what, int layer, void* dst, int64_t bytes, uint64_t stream) {
    if (!s || !dst) return sz_fail(SZ_E_ARG, "sz_session_export: null argument");
    if (s->last_m) return sz_fail(SZ_E_ARG, "sz_session_export: a pass is pending; commit it first");
    const sz_model_config& c = s->model.cfg;
    if (layer < 0 || layer >= c.n_layer) return sz_fail(SZ_E_ARG, "sz_session_export: layer %d of %d", layer, c.n_layer);
    cudaStream_t st = (cudaStream_t)stream;
    const bool attn = sz_is_attn(c, layer);
    if (what == SZ_STATE_DELTA_S || what == SZ_STATE_DELTA_CONV) {
        if (attn) return sz_fail(SZ_E_ARG, "sz_session_export: layer %d is an attention layer", layer);
        const int di = s->lb[layer].delta_index;
        const int64_t d = c.ssm_head_dim, ch = (2 * (int64_t)c.ssm_k_heads + c.ssm_v_heads) * d;
        const int64_t n = what == SZ_STATE_DELTA_S ? 4 * (int64_t)c.ssm_v_heads * d * d : 4 * (int64_t)(c.conv_k - 1) * ch;
        if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_export: %lld bytes given, the piece has %lld", (long long)bytes, (long long)n);
        const u8* src = what == SZ_STATE_DELTA_S ? (const u8*)s->S[s->cur] : (const u8*)s->conv[s->cur];
        SZ_CUDA(cudaMemcpyAsync(dst, src + (int64_t)di * n, (size_t)n, cudaMemcpyDeviceToHost, st));
    } else if (what == SZ_STATE_KV_K || what == SZ_STATE_KV_V) {
        if (!attn) return sz_fail(SZ_E_ARG, "sz_session_export: layer %d is a DeltaNet layer", layer);
        const int ai = s->lb[layer].attn_index;
        const int64_t hb = (s->flags & SZ_KV_Q8) ? (c.head_dim + (((c.head_dim >> 5) * 2 + 15) & ~15)) : 4 * (int64_t)c.head_dim;
        const int64_t n = (int64_t)s->len * c.n_kv_head * hb;
        if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_export: %lld bytes given, %d positions take %lld", (long long)bytes, s->len, (long long)n);
        const u8* base = (what == SZ_STATE_KV_K ? s->kc : s->vc) + (int64_t)ai * s->ctx * c.n_kv_head * hb;
        for (int h = 0; h < c.n_kv_head && s->len > 0; h++)
            SZ_CUDA(cudaMemcpy2DAsync((u8*)dst + h * hb, (size_t)(c.n_kv_head * hb), base + (int64_t)h * s->ctx * hb, (size_t)hb, (size_t)hb, (size_t)s->len,
                                      cudaMemcpyDeviceToHost, st));
    } else if (what == SZ_STATE_PLE_HIST || what == SZ_STATE_PLE_TAIL) {
        if (!s->p_hist) return sz_fail(SZ_E_ARG, "sz_session_export: the model has no per-layer embedding");
        const int64_t n = what == SZ_STATE_PLE_TAIL ? 32 : 4 * (int64_t)(s->model.ple.conv_k - 1) * s->model.ple.ngram * c.streams * c.hidden;
        if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_export: %lld bytes given, the piece has %lld", (long long)bytes, (long long)n);
        const u8* src = what == SZ_STATE_PLE_TAIL ? (const u8*)(s->p_tail + (s->cur ? 8 : 0)) : (const u8*)s->p_hist + (s->cur ? s->p_hist_bytes : 0);
        SZ_CUDA(cudaMemcpyAsync(dst, src, (size_t)n, cudaMemcpyDeviceToHost, st));
    } else if (what == SZ_STATE_IDX_RAW) {
        if (!attn || !s->i_raw) return sz_fail(SZ_E_ARG, "sz_session_export: layer %d has no sparse indexer", layer);
        const int64_t n = 4 * (int64_t)s->len * c.idx_dim;
        if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_export: %lld bytes given, %d positions take %lld", (long long)bytes, s->len, (long long)n);
        if (n) SZ_CUDA(cudaMemcpyAsync(dst, (const u8*)s->i_raw + s->lb[layer].attn_index * s->i_raw_layer, (size_t)n, cudaMemcpyDeviceToHost, st));
    } else if (what == SZ_STATE_IDX_SELECTED || what == SZ_STATE_IDX_SCORES) {
        if (!attn || !s->i_trace) return sz_fail(SZ_E_ARG, "sz_session_export: layer %d has no sparse indexer", layer);
        const int ai = s->lb[layer].attn_index;
        if (what == SZ_STATE_IDX_SELECTED) {
            const int64_t n = 4 * (int64_t)SZ_MAX_VERIFY * s->i_words;
            if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_export: %lld bytes given, the piece has %lld", (long long)bytes, (long long)n);
            SZ_CUDA(cudaMemcpyAsync(dst, s->i_trace + (size_t)ai * SZ_MAX_VERIFY * s->i_words, (size_t)n, cudaMemcpyDeviceToHost, st));
        } else {
            const int64_t n = 4 * (int64_t)SZ_MAX_VERIFY * 32 * s->i_words;
            if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_export: %lld bytes given, the piece has %lld", (long long)bytes, (long long)n);
            for (int j = 0; j < SZ_MAX_VERIFY; j++)   // rows of i_ctx_blocks scores, of which 32 * words >= that many are asked for
                SZ_CUDA(cudaMemcpyAsync((u8*)dst + (size_t)j * 32 * s->i_words * 4, s->i_scores + (size_t)j * s->i_ctx_blocks, (size_t)s->i_ctx_blocks * 4,
                                        cudaMemcpyDeviceToHost, st));
        }
    } else {
        return sz_fail(SZ_E_ARG, "sz_session_export: unknown piece %d", what);
    }
    SZ_CUDA(cudaStreamSynchronize(st));
    s->inflight = 0;
    return SZ_OK;
}

// ---- the way back: a checkpoint's pieces into a fresh session (GpuSession::restore, session.rs:3463-3541) ---------------------------
extern "C" int sz_session_import(sz_session* s, int what, int layer, const void* src, int64_t bytes, int positions, uint64_t stream) {
    if (!s || !src) return sz_fail(SZ_E_ARG, "sz_session_import: null argument");
    if (s->last_m) return sz_fail(SZ_E_ARG, "sz_session_import: a pass is pending; commit it first");
    const sz_model_config& c = s->model.cfg;
    if (layer < 0 || layer >= c.n_layer) return sz_fail(SZ_E_ARG, "sz_session_import: layer %d of %d", layer, c.n_layer);
    if (positions < 0 || positions + SZ_MAX_VERIFY > s->ctx) return sz_fail(SZ_E_ARG, "sz_session_import: %d positions in a session of %d", positions, s->ctx);
    cudaStream_t st = (cudaStream_t)stream;
    const bool attn = sz_is_attn(c, layer);
    if (what == SZ_STATE_DELTA_S || what == SZ_STATE_DELTA_CONV) {
        if (attn) return sz_fail(SZ_E_ARG, "sz_session_import: layer %d is an attention layer", layer);
        const int di = s->lb[layer].delta_index;
        const int64_t d = c.ssm_head_dim, ch = (2 * (int64_t)c.ssm_k_heads + c.ssm_v_heads) * d;
        const int64_t n = what == SZ_STATE_DELTA_S ? 4 * (int64_t)c.ssm_v_heads * d * d : 4 * (int64_t)(c.conv_k - 1) * ch;
        if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_import: %lld bytes given, the piece has %lld", (long long)bytes, (long long)n);
        u8* dst = what == SZ_STATE_DELTA_S ? (u8*)s->S[s->cur] : (u8*)s->conv[s->cur];
        SZ_CUDA(cudaMemcpyAsync(dst + (int64_t)di * n, src, (size_t)n, cudaMemcpyHostToDevice, st));
    } else if (what == SZ_STATE_KV_K || what == SZ_STATE_KV_V) {
        if (!attn) return sz_fail(SZ_E_ARG, "sz_session_import: layer %d is a DeltaNet layer", layer);
        const int ai = s->lb[layer].attn_index;
        const int64_t hb = (s->flags & SZ_KV_Q8) ? (c.head_dim + (((c.head_dim >> 5) * 2 + 15) & ~15)) : 4 * (int64_t)c.head_dim;
        const int64_t n = (int64_t)positions * c.n_kv_head * hb;
        if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_import: %lld bytes given, %d positions take %lld", (long long)bytes, positions, (long long)n);
        u8* base = (what == SZ_STATE_KV_K ? s->kc : s->vc) + (int64_t)ai * s->ctx * c.n_kv_head * hb;
        for (int h = 0; h < c.n_kv_head && positions > 0; h++)   // [position][kv head][head] of the checkpoint into the cache's [kv head][position][head]
            SZ_CUDA(cudaMemcpy2DAsync(base + (int64_t)h * s->ctx * hb, (size_t)hb, (const u8*)src + h * hb, (size_t)(c.n_kv_head * hb), (size_t)hb, (size_t)positions,
                                      cudaMemcpyHostToDevice, st));
    } else if (what == SZ_STATE_PLE_HIST || what == SZ_STATE_PLE_TAIL) {
        if (!s->p_hist) return sz_fail(SZ_E_ARG, "sz_session_import: the model has no per-layer embedding");
        const int64_t n = what == SZ_STATE_PLE_TAIL ? 32 : 4 * (int64_t)(s->model.ple.conv_k - 1) * s->model.ple.ngram * c.streams * c.hidden;
        if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_import: %lld bytes given, the piece has %lld", (long long)bytes, (long long)n);
        u8* dst = what == SZ_STATE_PLE_TAIL ? (u8*)(s->p_tail + (s->cur ? 8 : 0)) : (u8*)s->p_hist + (s->cur ? s->p_hist_bytes : 0);
        SZ_CUDA(cudaMemcpyAsync(dst, src, (size_t)n, cudaMemcpyHostToDevice, st));
    } else if (what == SZ_STATE_IDX_RAW) {
        if (!attn || !s->i_raw) return sz_fail(SZ_E_ARG, "sz_session_import: layer %d has no sparse indexer", layer);
        const int ai = s->lb[layer].attn_index, ratio = s->layers[layer].idx_ratio > 0 ? s->layers[layer].idx_ratio : 1;
        const int64_t n = 4 * (int64_t)positions * c.idx_dim;
        if (bytes != n) return sz_fail(SZ_E_ARG, "sz_session_import: %lld bytes given, %d positions take %lld", (long long)bytes, positions, (long long)n);
        float* raw = (float*)((u8*)s->i_raw + ai * s->i_raw_layer);
        if (n) SZ_CUDA(cudaMemcpyAsync(raw, src, (size_t)n, cudaMemcpyHostToDevice, st));
        if (positions / ratio > 0) {   // the pooled key of every complete block
            sz_idx_rebuild_kernel<<<positions / ratio, 128, 0, st>>>((const float*)raw, (const float*)s->layers[layer].idx_k_norm.data, (int)c.idx_dim, ratio, c.eps,
                                                                     (int)c.rope_dims, (const double*)s->rope_den, (float*)((u8*)s->i_blocks + ai * s->i_blocks_layer));
            SZ_CUDA(cudaGetLastError());
        }
    } else {
        return sz_fail(SZ_E_ARG, "sz_session_import: piece %d cannot be imported", what);
    }
    SZ_CUDA(cudaStreamSynchronize(st));
    s->inflight = 0;
    return SZ_OK;
}

extern "C" int sz_session_set_len(sz_session* s, int positions, uint64_t stream) {
    if (!s || s->last_m) return sz_fail(SZ_E_ARG, "sz_session_set_len: null session or a pass is pending");
    if (positions < 0 || positions + SZ_MAX_VERIFY > s->ctx) return sz_fail(SZ_E_ARG, "sz_session_set_len: %d positions in a session of %d", positions, s->ctx);
    cudaStream_t st = (cudaStream_t)stream;
    if (s->inflight) { SZ_CUDA(cudaStreamSynchronize(st)); s->inflight = 0; }
    s->h_pin[8] = positions;
    SZ_CUDA(cudaMemcpyAsync(s->state, s->h_pin + 8, 4, cudaMemcpyHostToDevice, st));   // word 0 of the device state: the committed positions
    SZ_CUDA(cudaStreamSynchronize(st));
    s->len = positions;
    return SZ_OK;
}

// ---- launching a kernel by name --------------------------------------------------------------------------------------------------
// The kernel-launch seam of the reference (Program::launch, crates/shadowzero-cuda/src/kernels.rs:546-572; the registry :39-57,
// 163-477): an entry point is looked up by name in a static table that spells out its parameter types, every argument travels in an
// 8-byte slot of its own, and a launch whose arguments do not fit the table is refused before the driver sees it.  The table covers
// this translation unit's kernels with plain parameters (no templates, no structs by value); tests/test_kernel_registry.py parses
// the sources and checks the table against them in both directions, as the reference's tests/drift.rs does.
namespace {
struct SzKernelEntry {
    const char* name;
    const void* fn;
    int n;
    int32_t types[20];
};
const SzKernelEntry kKernels[] = {
    {"sz_embed_kernel", (const void*)sz_embed_kernel, 7, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_PTR}},
    {"sz_hc_norm_kernel", (const void*)sz_hc_norm_kernel, 8, {SZ_P_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_F32, SZ_P_PTR}},
    {"sz_hc_rows_norm_kernel", (const void*)sz_hc_rows_norm_kernel, 11, {SZ_P_CONST_PTR, SZ_P_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_F32, SZ_P_PTR, SZ_P_PTR}},
    {"sz_hc_mix_kernel", (const void*)sz_hc_mix_kernel, 5, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_PTR}},
    {"sz_delta_prep_kernel", (const void*)sz_delta_prep_kernel, 16, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_PTR, SZ_P_PTR, SZ_P_PTR}},
    {"sz_conv_commit_kernel", (const void*)sz_conv_commit_kernel, 10, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_PTR, SZ_P_PTR, SZ_P_I32}},
    {"sz_state_update_kernel", (const void*)sz_state_update_kernel, 2, {SZ_P_PTR, SZ_P_CONST_PTR}},
    {"sz_attn_prep_kernel", (const void*)sz_attn_prep_kernel, 19, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_F32, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_PTR, SZ_P_PTR, SZ_P_PTR, SZ_P_PTR, SZ_P_CONST_PTR}},
    {"sz_attn_merge_kernel", (const void*)sz_attn_merge_kernel, 6, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_PTR}},
    {"sz_accept_greedy_kernel", (const void*)sz_accept_greedy_kernel, 7, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_PTR}},
    {"sz_accept_tree_kernel", (const void*)sz_accept_tree_kernel, 6, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_PTR}},
    {"sz_kv_compact_kernel", (const void*)sz_kv_compact_kernel, 7, {SZ_P_PTR, SZ_P_PTR, SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32}},
    {"sz_accept_sampled_kernel", (const void*)sz_accept_sampled_kernel, 6, {SZ_P_CONST_PTR, SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_CONST_PTR, SZ_P_PTR}},
    {"sz_topk_slices_kernel", (const void*)sz_topk_slices_kernel, 6, {SZ_P_CONST_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_PTR, SZ_P_CONST_PTR}},
    {"sz_topk_merge_kernel", (const void*)sz_topk_merge_kernel, 3, {SZ_P_CONST_PTR, SZ_P_I32, SZ_P_PTR}},
    {"sz_batch_rows_kernel", (const void*)sz_batch_rows_kernel, 4, {SZ_P_CONST_PTR, SZ_P_PTR, SZ_P_I32, SZ_P_I32}},
    {"sz_fill_kv_kernel", (const void*)sz_fill_kv_kernel, 8, {SZ_P_PTR, SZ_P_I32, SZ_P_I32, SZ_P_I32, SZ_P_U64, SZ_P_I32, SZ_P_I32, SZ_P_U32}},
};
const int kKernelCount = (int)(sizeof(kKernels) / sizeof(kKernels[0]));
const SzKernelEntry* sz_find_kernel(const char* name) {
    for (int i = 0; i < kKernelCount; i++)
        if (strcmp(kKernels[i].name, name) == 0) return &kKernels[i];
    return nullptr;
}
}  // namespace

extern "C" int sz_kernel_count(void) { return kKernelCount; }
extern "C" const char* sz_kernel_name(int i) { return i >= 0 && i < kKernelCount ? kKernels[i].name : nullptr; }
extern "C" int sz_kernel_params(const char* name, int32_t* types, int cap) {
    const SzKernelEntry* e = name ? sz_find_kernel(name) : nullptr;
    if (!e) return -1;
    for (int i = 0; i < e->n && i < cap && types; i++) types[i] = e->types[i];
    return e->n;
}

extern "C" int sz_kernel_launch(const char* name, const uint32_t grid[3], const uint32_t block[3], uint32_t shared, uint64_t stream, const sz_karg* args,
                                int nargs) {
    if (!name || !grid || !block || (nargs > 0 && !args)) return sz_fail(SZ_E_ARG, "sz_kernel_launch: null argument");
    const SzKernelEntry* e = sz_find_kernel(name);
    if (!e) return sz_fail(SZ_E_ARG, "the registry has no entry point %s", name);
    if (e->n != nargs) return sz_fail(SZ_E_ARG, "%s takes %d arguments, %d given", name, e->n, nargs);
    static const char* tn[] = {"Ptr", "ConstPtr", "U32", "I32", "U64", "F32"};
    for (int i = 0; i < nargs; i++) {
        const int a = args[i].type, p = e->types[i];
        const bool fits = a == p || (a == SZ_P_PTR && p == SZ_P_CONST_PTR);   // a device pointer satisfies both pointer kinds; scalars match exactly
        if (a < 0 || a > SZ_P_F32 || !fits) return sz_fail(SZ_E_ARG, "%s argument %d: a %s does not fit a %s parameter", name, i, a >= 0 && a <= SZ_P_F32 ? tn[a] : "?", tn[p]);
    }
    if (!grid[0] || !grid[1] || !grid[2] || !block[0] || !block[1] || !block[2] || (uint64_t)block[0] * block[1] * block[2] > 1024)
        return sz_fail(SZ_E_ARG, "%s: a grid of %u x %u x %u blocks of %u x %u x %u threads does not fit", name, grid[0], grid[1], grid[2], block[0], block[1], block[2]);
    uint64_t slots[20];
    void* ptrs[20];
    for (int i = 0; i < nargs; i++) { slots[i] = args[i].bits; ptrs[i] = &slots[i]; }   // little-endian: a 4-byte parameter reads the low half of its slot
    SZ_CUDA(cudaLaunchKernel(e->fn, dim3(grid[0], grid[1], grid[2]), dim3(block[0], block[1], block[2]), ptrs, shared, (cudaStream_t)stream));
    return SZ_OK;
}

#ifdef SZ_PHASES
extern "C" int sz_phase_read_session(long long* out) { return cudaMemcpyFromSymbol(out, sz_phase_t, sizeof(long long) * 16 * 16) == cudaSuccess ? 0 : 1; }
#endif

SZ_TIMELINE_READER(session)
