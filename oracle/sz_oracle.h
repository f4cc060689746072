/* CPU oracle for the ShadowZero verify-step hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's scalar CPU path
 * (crates/shadowzero-model/src/{half,quant,exl3,forward}.rs, crates/shadowzero-serve/src/{engine,sampler}.rs)
 * and of the arithmetic of the reference's non-exact GPU pieces (kernels/forward.cu Q8_KV, top-64).  It is the
 * checker for the CUDA library; nothing the library ships may call into it.  Every function names the reference
 * lines it follows.
 *
 * Pins (see tests/test_oracle_*.py): the reference's IQ3_S / F16 / BF16 / F32 known-answer blocks
 * (eval/fixtures/dequant.txt), the gguf-py 0.19.0 dequantiser for Q8_0 and IQ3_S, the reference's own unit-test
 * vectors (f16 rounding table, tile_pos bijection, WHT involution, codebook moments, route-vs-full-sort with its
 * xorshift seed, the suffix drafter and sampler vectors) and a slice of the real EXL3 tensors of
 * eval/fixtures/exl3_sample.safetensors through the reconstruct()·x == matvec(x) identity.
 * Tree verification, rejection sampling against draft probabilities, expert-parallel exchange and device-side
 * acceptance have no reference semantics: those parts are "parity unpinned".
 */
#ifndef SZ_ORACLE_H
#define SZ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#include "../include/shadowzero_b200.h" /* the model description structs (sz_model, sz_layer, sz_tensor): data = host addresses here */

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids as the reference's table has them (crates/shadowzero-model/src/gguf.rs:99-150). */
enum {
    SZO_F32 = 0, SZO_F16 = 1, SZO_Q8_0 = 8, SZO_IQ3_S = 21, SZO_BF16 = 30,
    SZO_EXL3_BASE = 1020 /* 1020 + K: codebook "mul1", K = 1..8 bits a weight */
};

/* ---- half.rs ---------------------------------------------------------------------------------------------------- */
float szo_f16_to_f32(uint16_t h);
uint16_t szo_f32_to_f16(float f);
float szo_bf16_to_f32(uint16_t b);
uint16_t szo_f32_to_bf16(float f);
uint16_t szo_f64_to_f16_bits(double x); /* exl3.rs:27-60 */

/* ---- quant.rs --------------------------------------------------------------------------------------------------- */
/* (elements, bytes) of a block of `type`; returns 0 on an unknown or block-less type. */
int szo_block(int type, int* elems, int* bytes);
/* Dequantises whole blocks; returns 0 on success, -1 on a size mismatch or unknown type (quant.rs:229-259). */
int szo_dequant(int type, const uint8_t* data, size_t nbytes, float* out, size_t nout);

/* ---- exl3.rs ---------------------------------------------------------------------------------------------------- */
float szo_exl3_cb(int cb, uint32_t state);
void szo_exl3_tile_pos(int p, int* row, int* col);
uint32_t szo_exl3_state(const uint16_t* tile, int bits, int half, int t);
void szo_exl3_decode_tile(const uint16_t* tile, int bits, int half, int cb, float* out256);
void szo_exl3_decode_tile_fast(const uint16_t* tile, int bits, int half, int cb, float* out256);
void szo_wht128(float* v);
size_t szo_exl3_blob_len(size_t in, size_t out, int bits, int half);
/* W[in][out] = diag(suh) H W_hat H diag(svh)  (exl3.rs:246-286). */
void szo_exl3_reconstruct(size_t in, size_t out, int bits, int half, int cb, const uint8_t* blob, float* w);
/* y = x W straight from the blob (exl3.rs:520-581). */
void szo_exl3_matvec_blob(size_t in, size_t out, int bits, int half, int cb, const uint8_t* blob, const float* x,
                          float* y, int threads);

/* ---- forward.rs ------------------------------------------------------------------------------------------------- */
/* y = W x: W stored ggml [cols, rows], whole rows contiguous; each row dequantised and dotted in f64
 * (forward.rs:210-228).  EXL3 types take the blob route (forward.rs:241-246). */
int szo_matvec(int type, const uint8_t* bytes, size_t rows, size_t cols, const float* x, float* y, int threads);
/* route_into (forward.rs:1088-1153): returns the number of experts written (min(k, n)). */
int szo_route(const float* logits, int n, int k, int32_t* idx, double* w);
void szo_rmsnorm(const float* x, const float* w, size_t n, float eps, float* y);
float szo_sigmoid(float x);
float szo_silu(float x);
float szo_softplus(float x);

/* One MoE layer's tensors.  gate/up/down experts: expert e starts at base + e * stride bytes. */
typedef struct {
    int32_t hidden, n_expert, top_k, expert_ff, shared_ff;
    int32_t expert_type, shared_type; /* ggml type ids */
    const float* router;              /* [n_expert][hidden] f32 (ffn_gate_inp) */
    const float* shared_router;       /* [hidden] f32 (ffn_gate_inp_shexp) */
    const uint8_t* gate; const uint8_t* up; const uint8_t* down;
    uint64_t gate_stride, up_stride, down_stride;
    const uint8_t* sh_gate; const uint8_t* sh_up; const uint8_t* sh_down;
} szo_moe_layer;

/* Session::moe for one token (forward.rs:1009-1034).  route_idx/route_w (top_k each) and logits (n_expert) are
 * optional outputs. */
void szo_moe(const szo_moe_layer* L, const float* u, float* y, int32_t* route_idx, double* route_w, float* logits,
             int threads);

/* ---- part 2 (sz_oracle_model.c): the forward step, the cache formats, drafting, sampling, the speculation loop ---------- */
size_t szo_kv_q8_head_bytes(int hd);
void szo_kv_quant_q8(const float* src, int hd, uint8_t* dst);     /* kernels/forward.cu:3664-3687 */
void szo_kv_dequant_q8(const uint8_t* src, int hd, float* dst);
void szo_top64(const float* logits, int vocab, float* vals64, uint32_t* ids64); /* kernels/forward.cu:3565-3625 */

typedef struct szo_session szo_session;
szo_session* szo_session_new(const sz_model* m, int kv_q8, int threads);
void szo_session_free(szo_session* s);
int szo_session_len(const szo_session* s);
const int32_t* szo_session_routes(const szo_session* s);          /* [n_layer][top_k] of the last step */
const double* szo_session_route_weights(const szo_session* s);
void szo_session_assign(szo_session* dst, const szo_session* src); /* snapshot / restore */
szo_session* szo_session_clone(const szo_session* src);
void szo_session_step(szo_session* s, uint32_t token, float* logits, float* final_u); /* forward.rs:751-794 */
/* a pass over a draft tree, row by row on copies of the session (no counterpart in the reference); greedy acceptance down the tree */
void szo_session_tree(szo_session* s, const uint32_t* ids, const int32_t* parents, int m, float* logits, const int32_t* keep_path, int n_keep);
int szo_tree_accept_greedy(const float* logits, int vocab, const uint32_t* ids, const int32_t* parents, int m, int eog, int32_t* path, uint32_t* next);
/* the library's synthetic history (sz_session_fill_synthetic), value for value: no counterpart in the reference */
void szo_session_fill_synthetic(szo_session* s, int len, uint32_t seed);
/* one piece of the state: 0 recurrent state [v heads][d][d], 1 carried conv rows, 2 / 3 K / V cache [position][kv head][head] */
const void* szo_session_state(const szo_session* s, int what, int l, size_t* bytes);
/* the sparse indexer of attention layer l in the last step: the positions attended to (ascending; returns how many), and the
 * block scores the selection was made by (0 when everything was attended to) */
int szo_session_selected(const szo_session* s, int l, int32_t* out, int cap);
int szo_session_idx_scores(const szo_session* s, int l, float* out, int cap);

int szo_lookup(const uint32_t* hist, int n_hist, int k, const int* lens, int n_lens, uint32_t* out); /* engine.rs:829-839 */
typedef struct szo_drafter szo_drafter;
szo_drafter* szo_drafter_new(int min_match, int max_match, int capacity_tokens);                     /* engine.rs:862-874 */
void szo_drafter_free(szo_drafter* d);
void szo_drafter_push(szo_drafter* d, uint32_t token);
int szo_drafter_len(const szo_drafter* d);
int szo_drafter_propose(const szo_drafter* d, int max_k, uint32_t* out, int* match_len);
int szo_drafter_propose_with_min(const szo_drafter* d, int max_k, int min_match, uint32_t* out, int* match_len);
int szo_drafter_propose_after(szo_drafter* d, const uint32_t* extra, int n_extra, int max_k, uint32_t* out, int* match_len);

typedef struct { float temperature; int32_t top_k; float top_p; float min_p; uint64_t seed; } szo_sampler; /* a resolved Sampler */
uint64_t szo_splitmix64(uint64_t x);
double szo_uniform(uint64_t seed, uint64_t pos);                                                       /* sampler.rs:90-94 */
uint32_t szo_sample(const szo_sampler* sp, const float* logits, int vocab, uint64_t pos);              /* sampler.rs:112-157 */
uint32_t szo_sample_top(const szo_sampler* sp, const float* tv, const uint32_t* ti, int ntop, uint64_t pos);

typedef struct { int32_t spec_k, max_new, lookup_min, greedy, eog_token, reserved; szo_sampler sampler; } szo_gen_params;
typedef struct { int32_t n_tokens, passes, drafted, accepted, lookup_passes; int32_t pos_tried[8], pos_right[8]; } szo_gen_stats;
int szo_tree_accept_sampled(const szo_sampler* sp, const float* tv, const uint32_t* ti, const uint32_t* ids, const int32_t* parents, int m,
                            const float* draft_prob, uint64_t pos, int eog, int32_t* path, uint32_t* next);
/* Generates up to max_new tokens after the prompt with the engine's loop; pass_log gets (drafted, accepted) per verify pass. */
int szo_generate(szo_session* s, const uint32_t* prompt, int n_prompt, const szo_gen_params* p, uint32_t* out, int32_t* pass_log,
                 int pass_cap, szo_gen_stats* stats);

/* ---- part 3 (sz_oracle_head.c): the lm_head's 2-bit screening proxy and block selection (GPU-only in the reference) ---- */
void szo_head_rotate(const uint8_t* blob, const float* x, size_t cols, float* xr);                       /* kernels/exl3.cu:609-625 */
void szo_head_proxy_build(size_t rows, size_t cols, int bits, const uint8_t* blob, uint8_t* w_q2, uint16_t* w_sc); /* exl3.cu:915-987 */
void szo_proxy_quant_x(const float* xr, size_t cols, int8_t* xq, float* x_sc, float* x_corr);            /* kernels/forward.cu:4369-4420 */
void szo_proxy_bmax(size_t rows, size_t cols, const uint8_t* w_q2, const uint16_t* w_sc, const int8_t* xq, const float* x_sc,
                    const float* x_corr, float* bmax);                                                   /* kernels/forward.cu:4428-4495 */
int szo_head_k_use(int k_blk, int need_k);                                                               /* session.rs:5964 */
int szo_proxy_pick(const float* bmax, int m, int n_ob, int k_use, int max_sel, uint32_t* sel);           /* kernels/forward.cu:4536-4632 */

#ifdef __cplusplus
}
#endif
#endif
