// Host side of the speculation loop: prompt lookup, the suffix drafter, the draft policy, the sampler and the
// draft -> verify -> accept -> commit loop over a sz_session.  C++ where the reference is Rust
// (crates/shadowzero-serve/src/engine.rs:823-1309, 2149-2454; crates/shadowzero-serve/src/sampler.rs:83-210); no CUDA in this file.
#include "sz_common.cuh"

#include <chrono>
#include <cmath>
#include <cstring>
#include <vector>

extern "C" {
int sz_session_prefill(sz_session* s, const int32_t* ids, int n, uint64_t stream);
int sz_session_verify(sz_session* s, const int32_t* ids, int m, int accept_mode, int eog_token, int want_head, uint64_t stream);
int sz_session_result(sz_session* s, int32_t* keep_next, uint32_t* top, float* logits, uint64_t stream);
int sz_session_commit(sz_session* s, int keep, uint64_t stream);
int sz_session_set_stops(sz_session* s, const int32_t* ids, int n, uint64_t stream);
int sz_batch_verify(sz_session* const* sessions, int n, const int32_t* ids, const int32_t* ms, int accept_mode, int eog_token, int rows_max, uint64_t scratch,
                    int64_t scratch_bytes, uint64_t stream);
int sz_batch_prefill(sz_session* const* sessions, int n, const int32_t* const* ids, const int32_t* lens, int rows_max, uint64_t scratch, int64_t scratch_bytes,
                     uint64_t stream);
int sz_session_stops(const sz_session* s, int32_t* out);
int sz_session_len(const sz_session* s);
int sz_session_capacity(const sz_session* s);
int sz_session_pending(const sz_session* s);
}

// ---- prompt lookup (engine.rs:821-839) --------------------------------------------------------------------------------------------
extern "C" int sz_lookup(const uint32_t* hist, int n_hist, int k, const int* lens, int n_lens, uint32_t* out) {
    if (!hist || !lens || !out) return 0;
    for (int li = 0; li < n_lens; li++) {
        const int n = lens[li];
        if (k == 0 || n_hist <= n) break;
        const uint32_t* tail = hist + (n_hist - n);
        for (int i = n_hist - n - 1; i >= 0; i--) {
            if (std::memcmp(hist + i, tail, sizeof(uint32_t) * (size_t)n) != 0) continue;
            int cnt = 0;
            for (int q = i + n; q < n_hist && cnt < k; q++) out[cnt++] = hist[q];
            return cnt;
        }
    }
    return 0;
}

// ---- suffix drafter (engine.rs:841-1011): every trigram's four most recent end positions in an open-addressing table --------------
struct sz_drafter {
    struct Slot { uint64_t key = 0; uint32_t pos[4] = {0, 0, 0, 0}; uint8_t n = 0; };
    size_t min_match, max_match;
    std::vector<uint32_t> hist;
    std::vector<Slot> table;
    size_t mask;

    static uint64_t mix(uint64_t x) {
        x ^= x >> 33; x *= 0xff51afd7ed558ccdULL;
        x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL;
        return x ^ (x >> 33);
    }
    uint64_t key_at(size_t end) const {
        const uint64_t a = hist[end - 2], b = hist[end - 1], c = hist[end];
        return mix((a * 0x9E3779B97F4A7C15ULL) ^ mix(b + 0x632BE59BD9B4E019ULL) ^ (c << 1)) | 1;
    }
    const Slot* find(uint64_t key) const {
        for (size_t i = (size_t)key & mask, probes = 0; probes <= mask; probes++, i = (i + 1) & mask) {
            if (table[i].key == key) return &table[i];
            if (table[i].key == 0) return nullptr;
        }
        return nullptr;
    }
    void push(uint32_t t) {
        hist.push_back(t);
        const size_t end = hist.size() - 1;
        if (end < 2) return;
        const uint64_t key = key_at(end);
        for (size_t i = (size_t)key & mask, probes = 0; probes <= mask; probes++, i = (i + 1) & mask) {
            Slot& s = table[i];
            if (s.key != key && s.key != 0) continue;
            s.key = key;
            s.pos[3] = s.pos[2]; s.pos[2] = s.pos[1]; s.pos[1] = s.pos[0];
            s.pos[0] = (uint32_t)end;
            if (s.n < 4) s.n++;
            return;
        }
    }
    // the tokens after the longest (then most recent) earlier occurrence of the current suffix
    int propose(int max_k, size_t min_m, uint32_t* out, int* match_len) const {
        *match_len = 0;
        if (min_m < 3) min_m = 3;
        const size_t n = hist.size();
        if (n < min_m + 1 || max_k <= 0) return 0;
        const size_t cur = n - 1;
        const Slot* s = find(key_at(cur));
        if (!s) return 0;
        size_t best_end = 0, best_len = 0;
        for (int w = 0; w < s->n; w++) {
            const size_t p = s->pos[w];
            if (p >= cur) continue;
            size_t len = 0;
            while (len < max_match && len <= p && hist[p - len] == hist[cur - len]) len++;
            if (len > best_len) { best_len = len; best_end = p; }
        }
        if (best_len < min_m) return 0;
        int cnt = 0;
        for (size_t q = best_end + 1; q <= cur && cnt < max_k; q++) out[cnt++] = hist[q];
        *match_len = (int)best_len;
        return cnt;
    }
};

extern "C" sz_drafter* sz_drafter_new(int min_match, int max_match, int capacity_tokens) {
    sz_drafter* d = new sz_drafter();
    d->min_match = (size_t)(min_match < 3 ? 3 : min_match);
    d->max_match = (size_t)max_match > d->min_match ? (size_t)max_match : d->min_match;
    size_t want = 2 * (size_t)(capacity_tokens > 1024 ? capacity_tokens : 1024), cap = 1;
    while (cap < want) cap <<= 1;
    d->table.resize(cap);
    d->mask = cap - 1;
    d->hist.reserve((size_t)(capacity_tokens > 0 ? capacity_tokens : 0));
    return d;
}
extern "C" void sz_drafter_free(sz_drafter* d) { delete d; }
extern "C" void sz_drafter_push(sz_drafter* d, uint32_t token) { if (d) d->push(token); }
extern "C" void sz_drafter_extend(sz_drafter* d, const uint32_t* tokens, int n) { if (d) for (int i = 0; i < n; i++) d->push(tokens[i]); }
extern "C" int sz_drafter_len(const sz_drafter* d) { return d ? (int)d->hist.size() : 0; }
extern "C" int sz_drafter_propose(const sz_drafter* d, int max_k, uint32_t* out, int* match_len) {
    return d->propose(max_k, d->min_match, out, match_len);
}
extern "C" int sz_drafter_propose_with_min(const sz_drafter* d, int max_k, int min_match, uint32_t* out, int* match_len) {
    return d->propose(max_k, (size_t)(min_match < 0 ? 0 : min_match), out, match_len);
}
// propose on history + extra (a neural drafter's proposal) without touching the index (engine.rs:996-1010)
extern "C" int sz_drafter_propose_after(sz_drafter* d, const uint32_t* extra, int n_extra, int max_k, uint32_t* out, int* match_len) {
    if (n_extra <= 0) return d->propose(max_k, d->min_match, out, match_len);
    *match_len = 0;
    if (max_k <= 0) return 0;
    const size_t n0 = d->hist.size();
    d->hist.insert(d->hist.end(), extra, extra + n_extra);
    const int r = d->propose(max_k, d->min_match, out, match_len);
    d->hist.resize(n0);
    return r;
}

// ---- draft policy (engine.rs:1013-1309): expected committed tokens per millisecond decide between the neural drafter's window and a
// suffix-lookup window, how far to chain a lookup after a neural draft, and how deep the neural draft goes ---------------------------
namespace {
constexpr int kMaxT = SZ_MAX_VERIFY;
constexpr int kBuckets = 4;
const double kShape[kMaxT + 1] = {0.0, 1.0, 1.35, 1.70, 2.05, 2.45, 2.85, 3.25, 3.60};
const double kPriorQ[kBuckets] = {0.75, 0.88, 0.93, 0.96};
const double kChainPrior[kBuckets] = {0.45, 0.65, 0.80, 0.90};
constexpr double kCostAlpha = 0.10, kTokAlpha = 0.05, kDecay = 0.97, kPriorN = 4.0, kProbes = 3.0, kStaleRounds = 300.0;
int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
int bucket_of(int match_len) { return match_len < 6 ? 0 : (match_len < 12 ? 1 : (match_len < 24 ? 2 : 3)); }
}  // namespace

struct sz_draft_policy {
    int max_t, base_spec;
    double margin;
    double cost[kMaxT + 1] = {}, cost_n[kMaxT + 1] = {}, tok[kMaxT + 1] = {}, tok_n[kMaxT + 1] = {}, last[kMaxT + 1] = {};
    double ok[kBuckets] = {}, bad[kBuckets] = {}, cok[kBuckets] = {}, cbad[kBuckets] = {};
    double rounds = 0.0, accept_ema = 0.65;
    int full_streak = 0, zero_streak = 0;

    double rate(const double* good, const double* miss, const double* prior, int match_len) const {
        const int b = bucket_of(match_len);
        return (good[b] + kPriorN * prior[b]) / (good[b] + miss[b] + kPriorN);
    }
    double cost_ms(int t) const {
        t = clampi(t, 1, kMaxT);
        if (cost_n[t] > 0.0) return cost[t];
        double num = 0.0, den = 0.0;  // unseen width: scale the seen ones by the shape curve
        for (int u = 1; u <= kMaxT; u++)
            if (cost_n[u] > 0.0) {
                const double w = cost_n[u] < 20.0 ? cost_n[u] : 20.0;
                num += w * cost[u] * kShape[t] / kShape[u];
                den += w;
            }
        return den > 0.0 ? num / den : kShape[t];
    }
    bool stale(int t) const { return cost_n[t] > 0.0 && rounds - last[t] > kStaleRounds; }
    double neural_tokens(int t) const {
        t = clampi(t, 1, kMaxT);
        return tok_n[t] > 0.0 ? tok[t] : 1.0 + 0.70 * (double)(t - 1);
    }
    void note_cost(int t, double round_ms) {
        if (round_ms > 0.0) {
            cost[t] = cost_n[t] > 0.0 ? (1.0 - kCostAlpha) * cost[t] + kCostAlpha * round_ms : round_ms;
            cost_n[t] += 1.0;
            last[t] = rounds;
        }
        rounds += 1.0;
    }
    void note_streak(int drafted, int accepted) {
        if (drafted <= 0) return;
        const int acc = accepted < drafted ? accepted : drafted;
        accept_ema = 0.75 * accept_ema + 0.25 * ((double)acc / (double)drafted);
        if (accepted >= drafted) { full_streak++; zero_streak = 0; }
        else if (accepted == 0) { zero_streak++; full_streak = 0; }
        else { full_streak = 0; zero_streak = 0; }
    }
    void note_neural(int t, int accepted) {
        const double got = (double)accepted + 1.0;
        tok[t] = tok_n[t] > 0.0 ? (1.0 - kTokAlpha) * tok[t] + kTokAlpha * got : got;
        tok_n[t] += 1.0;
    }
};

extern "C" sz_draft_policy* sz_policy_new(int max_t, int base_spec, double margin) {
    sz_draft_policy* p = new sz_draft_policy();
    p->max_t = clampi(max_t, 1, kMaxT);
    p->base_spec = clampi(base_spec, 1, kMaxT - 1);
    p->margin = margin;
    return p;
}
extern "C" void sz_policy_free(sz_draft_policy* p) { delete p; }
extern "C" double sz_policy_accept_ema(const sz_draft_policy* p) { return p->accept_ema; }

extern "C" int sz_policy_neural_k(const sz_draft_policy* p, int rem_tokens) {
    const int max_k = p->max_t - 1 < rem_tokens ? p->max_t - 1 : rem_tokens;
    if (max_k <= 0) return 0;
    int k = p->base_spec;
    if (p->full_streak >= 2 && p->accept_ema >= 0.75) k = p->base_spec + 1 < p->max_t - 1 ? p->base_spec + 1 : p->max_t - 1;
    else if (p->zero_streak >= 3 && p->accept_ema < 0.25) k = 2 < p->base_spec ? 2 : p->base_spec;
    return k < max_k ? k : max_k;
}

// Returns the window size t (1 + drafts); *lookup = 1 when the suffix lookup should draft this round.
extern "C" int sz_policy_choose(const sz_draft_policy* p, int t_neural, int lookup_k, int match_len, int* lookup) {
    int t = clampi(t_neural, 1, p->max_t);
    *lookup = 0;
    if (lookup_k <= 0) return t;
    const double base = p->neural_tokens(t) / p->cost_ms(t);
    const double q = p->rate(p->ok, p->bad, kPriorQ, match_len);
    const int k_lim = lookup_k < p->max_t - 1 ? lookup_k : p->max_t - 1;
    double e = 1.0, qi = 1.0, best = 0.0;
    int best_t = 0;
    for (int k = 1; k <= k_lim; k++) {
        qi *= q;
        e += qi;
        const double r = e / p->cost_ms(k + 1);
        if (r > best) { best = r; best_t = k + 1; }
    }
    const int t_full = k_lim + 1;
    if (best_t > 0 && best > base * (1.0 + p->margin)) {
        *lookup = 1;
        t = best_t;
        if (best_t < t_full && q >= 0.85 && p->stale(t_full)) t = t_full;
        return t;
    }
    if (t_full > t && (p->cost_n[t_full] < kProbes || p->stale(t_full)) && q >= 0.85) { *lookup = 1; t = t_full; }
    return t;
}

extern "C" int sz_policy_chain(const sz_draft_policy* p, int t_neural, double p_neural, int k_avail, int match_len) {
    t_neural = clampi(t_neural, 1, p->max_t);
    const int room = p->max_t - t_neural > 0 ? p->max_t - t_neural : 0;
    const int kmax = k_avail < room ? k_avail : room;
    if (kmax <= 0) return 0;
    const double e0 = p->neural_tokens(t_neural), base = e0 / p->cost_ms(t_neural);
    const double c = p->rate(p->cok, p->cbad, kChainPrior, match_len);
    p_neural = p_neural < 0.0 ? 0.0 : (p_neural > 1.0 ? 1.0 : p_neural);
    double gain = 0.0, ci = 1.0, best = 0.0;
    int best_k = 0;
    for (int k = 1; k <= kmax; k++) {
        ci *= c;
        gain += ci;
        const double r = (e0 + p_neural * gain) / p->cost_ms(t_neural + k);
        if (r > best) { best = r; best_k = k; }
    }
    const int t_full = t_neural + kmax;
    if (best_k > 0 && best > base * (1.0 + p->margin)) {
        if (best_k < kmax && p_neural * c >= 0.60 && p->stale(t_full)) return kmax;
        return best_k;
    }
    if ((p->cost_n[t_full] < kProbes || p->stale(t_full)) && p_neural * c >= 0.60) return kmax;
    return 0;
}

extern "C" void sz_policy_observe(sz_draft_policy* p, int lookup, int t, int accepted, int match_len, double round_ms) {
    t = clampi(t, 1, kMaxT);
    p->note_cost(t, round_ms);
    if (lookup) {
        const int b = bucket_of(match_len);
        p->ok[b] = kDecay * p->ok[b] + (double)accepted;
        p->bad[b] = kDecay * p->bad[b] + (accepted < t - 1 ? 1.0 : 0.0);
    } else {
        p->note_streak(t - 1, accepted);
        p->note_neural(t, accepted);
    }
}

extern "C" void sz_policy_observe_chain(sz_draft_policy* p, int t_neural, int k_chain, int accepted, int match_len, double round_ms) {
    t_neural = clampi(t_neural, 1, kMaxT);
    const int t = clampi(t_neural + k_chain, 1, kMaxT);
    p->note_cost(t, round_ms);
    const int drafted = t_neural - 1;
    const int acc = accepted < drafted ? accepted : drafted;
    p->note_streak(drafted, acc);
    p->note_neural(t_neural, acc);
    if (accepted < drafted) return;
    const int b = bucket_of(match_len), okc = accepted - drafted;
    p->cok[b] = kDecay * p->cok[b] + (double)okc;
    p->cbad[b] = kDecay * p->cbad[b] + (okc < k_chain ? 1.0 : 0.0);
}

// ---- sampler (sampler.rs:83-210): the draw at an output position is a pure function of (candidates, seed, position) -------------
static uint64_t sz_splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}
extern "C" double sz_uniform(uint64_t seed, uint64_t pos) {
    const uint64_t bits = sz_splitmix64(sz_splitmix64(seed) ^ (pos * 0xD6E8FEB86659FD93ULL));
    return (double)(bits >> 11) / 9007199254740992.0;
}

// Draws from a row's 64 largest logits as the device hands them over: top[0..64) value bit patterns (largest first), top[64..128) ids.
extern "C" uint32_t sz_sample_top(const sz_sampler* sp, const uint32_t* top, uint64_t pos) {
    float v[64];
    std::memcpy(v, top, sizeof(v));
    const uint32_t* id = top + 64;
    const float max = v[0];
    if (!std::isfinite(max)) return id[0];
    const float cut = max - 18.0f * sp->temperature;
    int n = 0;
    while (n < 64 && v[n] >= cut) n++;
    const int tk = sp->top_k < 1 ? 1 : sp->top_k;
    if (n > tk) n = tk;
    const float inv_t = 1.0f / sp->temperature;
    double probs[64], total = 0.0;
    for (int i = 0; i < n; i++) { probs[i] = std::exp((double)((v[i] - max) * inv_t)); total += probs[i]; }
    for (int i = 0; i < n; i++) probs[i] /= total;
    const double floor_p = (double)sp->min_p * probs[0];
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
    double u = sz_uniform(sp->seed, pos) * mass;
    for (int i = 0; i < keep; i++) {
        if (u < probs[i]) return id[i];
        u -= probs[i];
    }
    return id[keep - 1];
}

// ---- sampled acceptance down a draft tree (no counterpart in the reference: its sampled acceptance is the chain's "the token the
// target would have drawn", crates/shadowzero-serve/src/sampler.rs:3-9).  Rejection sampling against the drafter's probabilities,
// one level at a time: at the current row the target distribution p is the sampler's (temperature, top-k, min-p, top-p over the row's
// top-64, exactly the candidates and weights sz_sample_top draws from); its children are tried in row order - child c with token x
// and draft probability q is kept with probability min(1, p(x) / q); on a refusal p loses q at x (never below zero) and is
// renormalised.  When no child is kept the next token is drawn from what is left of p.  Under a drafter that proposes fixed tokens
// (q = 1: lookup, suffix drafter) what is emitted is distributed exactly as p; a spread-out drafter's residual would need its whole
// distribution, which the call does not have (only the drafted tokens' probabilities): an approximation then.  Every decision uses the counter-based uniform number of (seed, stream): the stream of the
// token at output position P is 256 P for the final draw and 256 P + 1 + i for the i-th child tried there.
// top: [m][128] as sz_session_result gives it; draft_prob[j]: the drafter's probability of ids[j] under its parent (row 0 unused).
// Returns the rows kept; path[0 .. kept) the kept rows (root first), *next the token after them.
static int sz_candidates(const sz_sampler* sp, const uint32_t* top, double* probs, const uint32_t** ids) {
    float v[64];
    std::memcpy(v, top, sizeof(v));
    *ids = top + 64;
    const float max = v[0];
    if (!std::isfinite(max)) { probs[0] = 1.0; return 1; }
    const float cut = max - 18.0f * sp->temperature;
    int n = 0;
    while (n < 64 && v[n] >= cut) n++;
    const int tk = sp->top_k < 1 ? 1 : sp->top_k;
    if (n > tk) n = tk;
    const float inv_t = 1.0f / sp->temperature;
    double total = 0.0;
    for (int i = 0; i < n; i++) { probs[i] = std::exp((double)((v[i] - max) * inv_t)); total += probs[i]; }
    for (int i = 0; i < n; i++) probs[i] /= total;
    const double floor_p = (double)sp->min_p * probs[0];
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
    for (int i = 0; i < keep; i++) probs[i] /= mass;
    return keep;
}

extern "C" int sz_tree_accept_sampled(const sz_sampler* sp, const uint32_t* top, const uint32_t* ids, const int32_t* parents, int m, const float* draft_prob,
                                      uint64_t pos, int eog_token, int32_t* path, uint32_t* next) {
    if (!sp || !top || !ids || !parents || !draft_prob || !path || !next || m < 1 || m > SZ_MAX_VERIFY) return -1;
    int cur = 0, keep = 1;
    path[0] = 0;
    for (;;) {
        double p[64];
        const uint32_t* cid = nullptr;
        int n = sz_candidates(sp, top + (size_t)cur * 128, p, &cid);
        const uint64_t P = pos + (uint64_t)(keep - 1);       // output position of the token after the current row
        int tried = 0, taken = -1;
        for (int c = cur + 1; c < m && taken < 0; c++) {
            if (parents[c] != cur) continue;
            const uint32_t x = ids[c];
            int at = -1;
            for (int i = 0; i < n; i++) if (cid[i] == x) { at = i; break; }
            const double px = at >= 0 ? p[at] : 0.0;
            double q = (double)draft_prob[c];
            if (!(q > 1e-12)) q = 1e-12;
            if (q > 1.0) q = 1.0;
            const double u = sz_uniform(sp->seed, 256 * P + 1 + (uint64_t)tried);
            tried++;
            if (eog_token >= 0 && x == (uint32_t)eog_token) continue;   // a drafted end-of-generation token is left for the loop's top
            if (u * q < px) { taken = c; break; }
            if (at >= 0) {                                               // refused: the residual distribution
                p[at] = px > q ? px - q : 0.0;
                double total = 0.0;
                for (int i = 0; i < n; i++) total += p[i];
                if (total > 0.0) for (int i = 0; i < n; i++) p[i] /= total;
                else { p[at] = 0.0; n = sz_candidates(sp, top + (size_t)cur * 128, p, &cid); }   // (only when p was all on x and q >= p: start over)
            }
        }
        if (taken >= 0) { cur = taken; path[keep++] = cur; continue; }
        double u = sz_uniform(sp->seed, 256 * P);
        uint32_t tok = cid[n - 1];
        for (int i = 0; i < n; i++) {
            if (u < p[i]) { tok = cid[i]; break; }
            u -= p[i];
        }
        *next = tok;
        return keep;
    }
}

// ---- the loop (engine.rs:2149-2454 with the suffix drafter alone: no neural drafter, so the policy is not consulted and a window
// is 1 + at most spec_k rows) ---------------------------------------------------------------------------------------------------------
static double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct sz_gen {
    sz_session* s;
    sz_gen_params p;
    sz_drafter* sd = nullptr;
    std::vector<uint32_t> hist, top, last;
    int n = 0;            // tokens emitted so far
    bool done = false;    // an end-of-generation token was drawn
    std::vector<uint32_t> stops;   // the request's stop ids (sz_gen_set_stops): end generation like the end-of-generation id
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;  // bracket a pass on its stream: the device's share of a round
    ~sz_gen() {
        sz_drafter_free(sd);
        if (ev0) cudaEventDestroy(ev0);
        if (ev1) cudaEventDestroy(ev1);
    }
};

// sz_gen_begin in its two halves, around the feeding of the prompt (one sequence's own passes, or steps shared with others)
static int gen_create(sz_session* s, const uint32_t* prompt, int n_prompt, const sz_gen_params* p, uint64_t stream, sz_gen** out) {
    if (!s || !prompt || n_prompt < 1 || !p || !out) return sz_fail(SZ_E_ARG, "sz_gen_begin: null argument or empty prompt");
    if (p->spec_k < 0 || p->spec_k > SZ_MAX_VERIFY - 1) return sz_fail(SZ_E_ARG, "sz_gen_begin: spec_k = %d (0..%d)", p->spec_k, SZ_MAX_VERIFY - 1);
    if (sz_session_len(s) + n_prompt + p->max_new + SZ_MAX_VERIFY > sz_session_capacity(s))
        return sz_fail(SZ_E_ARG, "sz_gen_begin: prompt %d + %d new tokens do not fit the session", n_prompt, p->max_new);
    sz_gen* g = new sz_gen();
    g->s = s; g->p = *p;
    { int32_t st[7]; const int ns = sz_session_stops(s, st); g->stops.assign(st, st + ns); }   // the session's stop ids hold for the loop too
    g->top.resize(SZ_MAX_VERIFY * 128); g->last.resize(128);
    if (cudaEventCreate(&g->ev0) != cudaSuccess || cudaEventCreate(&g->ev1) != cudaSuccess) { delete g; return sz_fail(SZ_E_CUDA, "sz_gen_begin: no events"); }
    const int rc = !p->greedy && p->device_accept ? sz_session_set_sampler(s, &p->sampler) : SZ_OK;
    if (rc) { delete g; return rc; }
    *out = g;
    return SZ_OK;
}
// after the prompt's last pass (pending): its top-64, the commit, the drafter's index of the prompt
static int gen_fed(sz_gen* g, const uint32_t* prompt, int n_prompt, uint64_t stream) {
    const sz_gen_params* p = &g->p;
    const int tail = (n_prompt - 1) % SZ_MAX_VERIFY + 1;  // rows of the last prompt pass
    int rc = sz_session_result(g->s, nullptr, g->top.data(), nullptr, stream);
    if (!rc) rc = sz_session_commit(g->s, tail, stream);
    if (rc) return rc;
    std::memcpy(g->last.data(), g->top.data() + (size_t)(tail - 1) * 128, 128 * 4);
    g->sd = sz_drafter_new(p->lookup_min < 3 ? 3 : p->lookup_min, 32, n_prompt + p->max_new + 64);
    g->hist.assign(prompt, prompt + n_prompt);
    sz_drafter_extend(g->sd, prompt, n_prompt);
    return SZ_OK;
}

extern "C" int sz_gen_begin(sz_session* s, const uint32_t* prompt, int n_prompt, const sz_gen_params* p, uint64_t stream, sz_gen** out) {
    sz_gen* g = nullptr;
    int rc = gen_create(s, prompt, n_prompt, p, stream, &g);
    if (rc) return rc;
    rc = sz_session_prefill(s, (const int32_t*)prompt, n_prompt, stream);
    if (!rc) rc = gen_fed(g, prompt, n_prompt, stream);
    if (rc) { delete g; return rc; }
    *out = g;
    return SZ_OK;
}

// sz_gen_begin for n sequences at once: the prompts are fed in lockstep (sz_batch_prefill: steps of up to 8 rows of every
// sequence, what reads weights once over the rows of all of them).  gens[b] is sequence b's generator, as sz_gen_begin makes it.
extern "C" int sz_batch_gen_begin(sz_session* const* ss, int n, const uint32_t* const* prompts, const int32_t* n_prompts, const sz_gen_params* p, int rows_max,
                                  uint64_t scratch, int64_t scratch_bytes, uint64_t stream, sz_gen** gens) {
    if (!ss || !prompts || !n_prompts || !p || !gens || n < 1 || n > 64) return sz_fail(SZ_E_ARG, "sz_batch_gen_begin: 1..64 sequences");
    int rc = SZ_OK, made = 0;
    for (; made < n && !rc; made++) rc = gen_create(ss[made], prompts[made], n_prompts[made], p, stream, &gens[made]);
    if (rc) made--;   // (the one that failed made nothing)
    if (!rc) rc = sz_batch_prefill(ss, n, (const int32_t* const*)prompts, n_prompts, rows_max, scratch, scratch_bytes, stream);
    for (int b = 0; b < n && !rc; b++) rc = gen_fed(gens[b], prompts[b], n_prompts[b], stream);
    if (rc) { for (int b = 0; b < made; b++) { delete gens[b]; gens[b] = nullptr; } }
    return rc;
}

// The request's stop tokens (engine.rs:2386 `stops.contains(&d)`; the tokenizer's further end-of-generation ids go here too): the
// loop ends at one as at the end-of-generation id, and a drafted one is never accepted - on the host and on the device alike.
extern "C" int sz_gen_set_stops(sz_gen* g, const uint32_t* ids, int n, uint64_t stream) {
    if (!g || n < 0 || n > 7 || (n > 0 && !ids)) return sz_fail(SZ_E_ARG, "sz_gen_set_stops: 0..7 stop ids");
    g->stops.assign(ids, ids + n);
    int32_t tmp[7];
    for (int i = 0; i < n; i++) tmp[i] = (int32_t)ids[i];
    return sz_session_set_stops(g->s, tmp, n, stream);
}

extern "C" void sz_gen_free(sz_gen* g) { delete g; }

// One round of the loop in two halves, so that the pass between them can be one sequence's own (sz_gen_run) or a step shared
// with other sequences (sz_batch_gen_run).
struct SzRound {
    int32_t batch[SZ_MAX_VERIFY];
    uint32_t draft[SZ_MAX_VERIFY];
    int nd = 0, m = 0;
    double t1 = 0.0;
};
static uint32_t gen_pick(const sz_gen* g, const uint32_t* row, uint64_t pos) { return g->p.greedy ? row[64] : sz_sample_top(&g->p.sampler, row, pos); }
static bool gen_is_eog(const sz_gen* g, uint32_t t) {
    if (g->p.eog_token >= 0 && t == (uint32_t)g->p.eog_token) return true;
    for (uint32_t st : g->stops) if (st == t) return true;
    return false;
}
// The round's own token and its drafts.  false: the sequence has ended (nothing to verify).
static bool gen_propose(sz_gen* g, uint32_t* out, sz_gen_stats* stats, SzRound* r) {
    const sz_gen_params* p = &g->p;
    int& n = g->n;
    if (g->done || n >= p->max_new) return false;
    const uint32_t next = gen_pick(g, g->last.data(), (uint64_t)n);
    if (gen_is_eog(g, next)) { g->done = true; return false; }
    out[n++] = next;
    g->hist.push_back(next);
    sz_drafter_push(g->sd, next);
    r->batch[0] = (int32_t)next;
    int nd = 0, match_len = 0;
    const double t0 = now_ms();
    if (p->spec_k > 0) {
        const int rem = p->max_new - n;
        const int k = p->spec_k < rem ? p->spec_k : rem;
        if (p->lookup_min > 0) nd = sz_drafter_propose(g->sd, k, r->draft, &match_len);
        if (nd >= 2) stats->lookup_passes++;
        else {
            nd = sz_drafter_propose_with_min(g->sd, k, 3, r->draft, &match_len);
            if (nd == 0) { const int lens[2] = {3, 2}; nd = sz_lookup(g->hist.data(), (int)g->hist.size(), k, lens, 2, r->draft); }
        }
    }
    r->t1 = now_ms();
    stats->draft_ms += r->t1 - t0;
    for (int i = 0; i < nd; i++) r->batch[1 + i] = (int32_t)r->draft[i];
    r->nd = nd;
    r->m = 1 + nd;
    return true;
}
// After the pass: the result, acceptance as the host sees it (checked against the device's), the commit, the books.
static int gen_settle(sz_gen* g, uint32_t* out, int32_t* pass_log, int pass_cap, sz_gen_stats* stats, const SzRound* r, uint64_t stream) {
    sz_session* s = g->s;
    const bool dev_accept = g->p.device_accept != 0;
    int& n = g->n;
    int32_t kn[2] = {1, 0};
    int rc = sz_session_result(s, dev_accept ? kn : nullptr, g->top.data(), nullptr, stream);
    if (rc) return rc;
    const double t2 = now_ms();
    stats->verify_ms += t2 - r->t1;
    int keep = 1;
    for (int i = 0; i < r->nd; i++) {
        stats->pos_tried[i < 7 ? i : 7]++;
        const uint32_t want = gen_pick(g, g->top.data() + (size_t)i * 128, (uint64_t)n);
        if (want != r->draft[i] || gen_is_eog(g, r->draft[i])) break;
        out[n++] = r->draft[i];
        keep++;
        stats->pos_right[i < 7 ? i : 7]++;
        g->hist.push_back(r->draft[i]);
        sz_drafter_push(g->sd, r->draft[i]);
    }
    if (dev_accept && kn[0] != keep) return sz_fail(SZ_E_DEVICE, "device acceptance kept %d rows, the host loop %d", kn[0], keep);
    if ((rc = sz_session_commit(s, keep, stream))) return rc;
    stats->commit_ms += now_ms() - t2;
    stats->rounds++;
    if (r->nd > 0) {
        stats->passes++;
        stats->drafted += r->nd;
        stats->accepted += keep - 1;
        if (pass_log && stats->passes <= pass_cap) { pass_log[2 * (stats->passes - 1)] = r->nd; pass_log[2 * (stats->passes - 1) + 1] = keep - 1; }
    }
    std::memcpy(g->last.data(), g->top.data() + (size_t)(keep - 1) * 128, 128 * 4);
    stats->n_tokens = n;
    return SZ_OK;
}

// Runs up to `rounds` rounds of the loop (0: until max_new tokens or an end-of-generation token).  A round emits one token plus the
// drafts it accepts.  `out` receives every token emitted so far at its position; stats accumulate over calls that pass the same struct.
extern "C" int sz_gen_run(sz_gen* g, int rounds, uint32_t* out, int32_t* pass_log, int pass_cap, sz_gen_stats* stats, uint64_t stream) {
    if (!g || !out || !stats) return sz_fail(SZ_E_ARG, "sz_gen_run: null argument");
    sz_session* s = g->s;
    const sz_gen_params* p = &g->p;
    int rc = SZ_OK, done_rounds = 0;
    while (rounds <= 0 || done_rounds < rounds) {
        SzRound r;
        if (!gen_propose(g, out, stats, &r)) break;
        const bool dev_accept = p->device_accept != 0;
        cudaEventRecord(g->ev0, (cudaStream_t)stream);
        // sampled: row i is the draw at output position n + i (n already counts this round's first token)
        rc = dev_accept && !p->greedy ? sz_session_verify_sampled(s, r.batch, r.m, (uint64_t)g->n, p->eog_token, stream)
                                      : sz_session_verify(s, r.batch, r.m, dev_accept ? SZ_ACCEPT_GREEDY : SZ_ACCEPT_NONE, p->eog_token, 1, stream);
        if (rc) break;
        cudaEventRecord(g->ev1, (cudaStream_t)stream);
        if ((rc = gen_settle(g, out, pass_log, pass_cap, stats, &r, stream))) break;
        float dev = 0.f;
        if (cudaEventElapsedTime(&dev, g->ev0, g->ev1) == cudaSuccess) stats->device_ms += dev;
        done_rounds++;
    }
    stats->n_tokens = g->n;
    return rc;
}

// The loop of n sequences in lockstep: every round, each live sequence proposes its rows, ONE step verifies them all
// (sz_batch_verify: the sequences' sessions, the MoE sublayers shared), and each settles its own.  Greedy acceptance on the device.
// outs[b], stats[b]: as sz_gen_run's for sequence b.  device_ms (when not null) accumulates the steps' time on the device.
extern "C" int sz_batch_gen_run(sz_gen* const* gs, int n, int rounds, uint32_t* const* outs, sz_gen_stats* const* stats, int rows_max, uint64_t scratch,
                                int64_t scratch_bytes, double* device_ms, uint64_t stream) {
    if (!gs || !outs || !stats || n < 1 || n > 64) return sz_fail(SZ_E_ARG, "sz_batch_gen_run: 1..64 sequences");
    for (int b = 0; b < n; b++) {
        if (!gs[b] || !outs[b] || !stats[b]) return sz_fail(SZ_E_ARG, "sz_batch_gen_run: null argument");
        if (!gs[b]->p.greedy || !gs[b]->p.device_accept) return sz_fail(SZ_E_ARG, "sz_batch_gen_run: greedy acceptance on the device (sequence %d asks otherwise)", b);
        if (gs[b]->p.eog_token != gs[0]->p.eog_token) return sz_fail(SZ_E_ARG, "sz_batch_gen_run: one end-of-generation id for the batch");
    }
    cudaEvent_t e0 = gs[0]->ev0, e1 = gs[0]->ev1;
    int rc = SZ_OK, done_rounds = 0;
    std::vector<SzRound> rs((size_t)n);
    std::vector<sz_session*> ss;
    std::vector<int32_t> ids, ms;
    std::vector<int> who;
    while (rounds <= 0 || done_rounds < rounds) {
        ss.clear(); ids.clear(); ms.clear(); who.clear();
        for (int b = 0; b < n; b++) {
            if (!gen_propose(gs[b], outs[b], stats[b], &rs[b])) continue;
            who.push_back(b);
            ss.push_back(gs[b]->s);
            ms.push_back(rs[b].m);
            ids.insert(ids.end(), rs[b].batch, rs[b].batch + rs[b].m);
        }
        if (who.empty()) break;
        cudaEventRecord(e0, (cudaStream_t)stream);
        if ((rc = sz_batch_verify(ss.data(), (int)ss.size(), ids.data(), ms.data(), SZ_ACCEPT_GREEDY, gs[0]->p.eog_token, rows_max, scratch, scratch_bytes, stream))) break;
        cudaEventRecord(e1, (cudaStream_t)stream);
        for (int b : who)
            if ((rc = gen_settle(gs[b], outs[b], nullptr, 0, stats[b], &rs[b], stream))) break;
        if (rc) break;
        float dev = 0.f;
        if (device_ms && cudaEventElapsedTime(&dev, e0, e1) == cudaSuccess) *device_ms += dev;
        done_rounds++;
    }
    for (int b = 0; b < n; b++) stats[b]->n_tokens = gs[b]->n;
    return rc;
}

extern "C" int sz_generate(sz_session* s, const uint32_t* prompt, int n_prompt, const sz_gen_params* p, uint32_t* out, int32_t* pass_log,
                           int pass_cap, sz_gen_stats* stats, uint64_t stream) {
    if (!stats || !out) return sz_fail(SZ_E_ARG, "sz_generate: null argument");
    std::memset(stats, 0, sizeof(*stats));
    sz_gen* g = nullptr;
    int rc = sz_gen_begin(s, prompt, n_prompt, p, stream, &g);
    if (rc) return rc;
    rc = sz_gen_run(g, p->max_rounds, out, pass_log, pass_cap, stats, stream);
    sz_gen_free(g);
    return rc;
}
