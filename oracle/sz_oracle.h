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

#ifdef __cplusplus
}
#endif
#endif
