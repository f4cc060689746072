/* shadowzero_b200: sm_100a kernels for the speculative-decoding verify step of ShadowZero, behind a C ABI.
 *
 * Conventions (those of the reference's own native libraries, native/mmq/shadowzero_mmq.cu:1-33 and
 * native/fused/shadowzero_fused.cu:1-9, bound by crates/shadowzero-cuda/src/{mmq,fused}.rs:9-16):
 *   - plain C; device addresses are uint64_t, sizes int64_t, tensor types are ggml type ids (int);
 *   - the stream is an opaque uint64_t (a CUstream / cudaStream_t; 0 = the default stream);
 *   - every call is asynchronous on the caller's stream and uses the context current on the calling thread
 *     (the `*_host` calls are the exception: they copy from and to host memory and synchronise the stream);
 *   - scratch memory is sized by a pure `*_scratch_bytes` query and provided by the caller; hot calls never allocate;
 *   - the return value is 0 on success, otherwise an SZ_E_* code; sz_last_error() has the message for this thread.
 *     A bad argument list is refused before anything is launched (crates/shadowzero-cuda/src/kernels.rs:546-572).
 * There is no CPU fallback: without a CUDA device every compute call returns SZ_E_CUDA.
 */
#ifndef SHADOWZERO_B200_H
#define SHADOWZERO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SZ_OK 0
#define SZ_E_ARG 1      /* an argument is out of range, misaligned or inconsistent */
#define SZ_E_TYPE 2     /* a tensor type this build has no kernel for */
#define SZ_E_CUDA 3     /* a CUDA call failed; sz_last_error() has the driver's text */
#define SZ_E_SCRATCH 4  /* the scratch buffer is smaller than *_scratch_bytes says */
#define SZ_E_DEVICE 5   /* a kernel reported a failed internal check (bounded wait ran out, bad plan) */

/* ggml type ids, as crates/shadowzero-model/src/gguf.rs:99-150 numbers them. */
#define SZ_TYPE_F32 0
#define SZ_TYPE_F16 1
#define SZ_TYPE_Q8_0 8
#define SZ_TYPE_IQ3_S 21
#define SZ_TYPE_BF16 30
#define SZ_TYPE_EXL3(K) (1020 + (K)) /* trellis, codebook "mul1", K = 1..8 bits a weight (gguf.rs:141-143) */

#define SZ_MAX_VERIFY 8   /* rows of a verify pass: MAX_VERIFY, crates/shadowzero-cuda/src/session.rs:271 */
#define SZ_MAX_TOPK 16    /* experts a token routes to (route_into's fixed arrays, forward.rs:1096) */

/* Library version and the text of this thread's last error. */
const char* sz_version(void);
const char* sz_last_error(void);

/* ---- per-kernel timing ------------------------------------------------------------------------------------------
 * The role of the reference's SHADOWZERO_KTIME switch (crates/shadowzero-cuda/src/kernels.rs:527-536,604).  Between
 * sz_trace_begin and sz_trace_end every kernel this thread launches through the library is followed by a record of the next
 * event of `events` (cudaEvent_t handles created by the caller, timing enabled) on the kernel's stream; events[0] is recorded
 * by sz_trace_begin itself on `stream`.  sz_trace_end returns how many events were recorded; sz_trace_name(i) names the kernel
 * that ended at events[i].  Events between kernels serialise them, so trace for attribution and time the untraced call. */
int sz_trace_begin(uint64_t* events, int capacity, uint64_t stream);
int sz_trace_end(void);
const char* sz_trace_name(int i);

/* ---- test kernels: the format decoders on their own --------------------------------------------------------------
 * Replace kernels/dequant.cu (dequant_*), kernels/convert.cu and the `exl3_codebook` entry of kernels/exl3.cu, which the
 * reference's GPU tests compare bit for bit with its Rust decoders (crates/shadowzero-cuda/tests/dequant.rs:40-70,
 * convert.rs:41-93, exl3.rs:64-77). */

/* dst[i] = weight i of `nbytes` bytes of whole blocks of `type` (F32, F16, BF16, Q8_0, IQ3_S), as f32. */
int sz_dequant(int type, uint64_t src, int64_t nbytes, uint64_t dst_f32, int64_t n_weights, uint64_t stream);
/* dst[s] = the value of codebook "mul1" for each 16-bit state s in [0, 65536). */
int sz_exl3_codebook(uint64_t dst_f32, uint64_t stream);
/* W_hat[in][out] (rotated basis, row-major f32) of an EXL3 blob: crates/shadowzero-model/src/exl3.rs:230-244. */
int sz_exl3_reconstruct_inner(int bits, uint64_t blob, int64_t n_in, int64_t n_out, uint64_t dst_f32, uint64_t stream);

/* ---- the MoE sublayer of a verify pass ---------------------------------------------------------------------------
 * One call = Session::moe (crates/shadowzero-model/src/forward.rs:1009-1034) for each of the m rows of a verify pass:
 * router logits, f64 softmax + top-k + renormalised weights (route_into, forward.rs:1088-1153), the routed experts'
 * SwiGLU FFN grouped by expert so a matrix is read once for all the rows that chose it, the shared expert, and the
 * weighted sum in rank order.  It replaces GpuSession::moe_router_batch + moe_batch_resident
 * (crates/shadowzero-cuda/src/session.rs:7868-7871, 8222-8285, 8871-8953) and the kernels they launch:
 * matvec_cols_f32, route_plan_res_small, matvec_grouped_{q8_0,iq3_s}, matvec_grouped_exl3_*, swiglu,
 * moe_combine_qwen_rows (kernels/matvec.cu:756,1668-1677; kernels/exl3.cu:679-681; kernels/forward.cu:2512,2568,3392). */
typedef struct sz_moe_layer {
    int32_t hidden;        /* H: width of the residual stream */
    int32_t n_expert;      /* routed experts in the layer */
    int32_t top_k;         /* experts a token routes to (<= SZ_MAX_TOPK) */
    int32_t expert_ff;     /* FF of a routed expert */
    int32_t shared_ff;     /* FF of the shared expert (0: the layer has none) */
    int32_t expert_type;   /* type of gate/up/down of the routed experts */
    int32_t shared_type;   /* type of the shared expert's matrices */
    int32_t reserved;
    uint64_t router;        /* f32 [n_expert][hidden]: ffn_gate_inp */
    uint64_t shared_router; /* f32 [hidden]: ffn_gate_inp_shexp */
    uint64_t gate, up, down;                        /* expert e's matrix starts at base + e * stride bytes */
    uint64_t gate_stride, up_stride, down_stride;
    uint64_t sh_gate, sh_up, sh_down;
    /* Expert parallelism: this GPU holds experts [ep_first, ep_first + ep_count) of the layer; gate / up / down then point at the
     * first LOCAL expert.  ep_count = 0: all of them (no sharding).  ep_shared = 1 on the one rank that adds the shared expert. */
    int32_t ep_first, ep_count, ep_shared, ep_reserved;
} sz_moe_layer;
/* Matrices are stored as the reference stores them: ggml [cols = in, rows = out], whole rows contiguous, for the block
 * types; one blob (f16 suh | f16 svh | 4-byte marker | trellis) for EXL3 (crates/shadowzero-model/src/exl3.rs:388-398).
 * A block-type tensor starts on a 16-byte boundary; an EXL3 blob is placed so that its TRELLIS does (blob address = 12 mod 16
 * when in + out is even, since suh, svh and the marker take 2 in + 2 out + 4 bytes).  Strides are multiples of 16. */

/* Bytes of scratch sz_moe_verify needs for up to `m` rows of this layer shape. */
int sz_moe_scratch_bytes(const sz_moe_layer* layer, int m, int64_t* bytes);
/* Clears the scratch's counters.  Once after allocation (and after a failed call), before the first sz_moe_verify. */
int sz_moe_scratch_init(uint64_t scratch, int64_t scratch_bytes, uint64_t stream);
/* y[j] = moe(x[j]) for j < m (1 <= m <= SZ_MAX_VERIFY); x, y: f32 [m][hidden], row-major, 16-byte aligned.
 * route_idx (int32 [m][top_k]) and route_w (f64 [m][top_k]) receive the routing when non-zero: the named streams
 * `layerL.route_idx` / `layerL.route_w` of the reference's trace (forward.rs:1015-1018). */
int sz_moe_verify(const sz_moe_layer* layer, uint64_t x, int m, uint64_t y, uint64_t route_idx, uint64_t route_w,
                  uint64_t scratch, int64_t scratch_bytes, uint64_t stream);
/* The same through host memory: x_host is copied to the device buffer x_dev, the step runs, y_dev (and the routing, when
 * the host pointers are non-null) is copied back, and the stream is synchronised.  Pinned host memory makes the copies
 * asynchronous.  This is the call an engine whose activations live on the host would make. */
int sz_moe_verify_host(const sz_moe_layer* layer, const float* x_host, int m, float* y_host, int32_t* route_idx_host,
                       double* route_w_host, uint64_t x_dev, uint64_t y_dev, uint64_t scratch, int64_t scratch_bytes,
                       uint64_t stream);
/* The same sublayer over MANY rows at once (a prompt chunk; the verify rows of many sequences): y[j] = moe(x[j]) for j < rows, rows a
 * multiple of 8 up to 256, every distinct expert decoded once for all the rows that chose it.  The role of the reference's grouped
 * experts of a long prompt (plan_scan_w / plan_fill_w, kernels/forward.cu:3234-3319; mma_grouped*, kernels/matvec.cu:1190-1260;
 * exl3_mma, kernels/exl3.cu:500-590), with the verify pass's exact kernels: a row's output is bit for bit sz_moe_verify's.  EXL3
 * experts, no expert sharding.  sz_moe_rows_status(layer, rows, scratch, NULL, stream) once after the scratch is allocated (and
 * after a failed call); with a code pointer it synchronises and reports (bit 0: a bounded wait ran out, bit 1: the routing needed
 * more windows than the scratch has, bit 2: an expert id out of range reached the plan).  The scratch has one size and one layout
 * whatever the rows of a call. */
int sz_moe_rows_scratch_bytes(const sz_moe_layer* layer, int rows, int64_t* bytes);
int sz_moe_rows(const sz_moe_layer* layer, uint64_t x, int rows, uint64_t y, uint64_t route_idx, uint64_t route_w, uint64_t scratch,
                int64_t scratch_bytes, uint64_t stream);
int sz_moe_rows_status(const sz_moe_layer* layer, int rows, uint64_t scratch, int* code, uint64_t stream);
/* Number of kernel launches one sz_moe_verify call makes for this layer (for launch accounting). */
int sz_moe_launches(const sz_moe_layer* layer);

/* ---- the model: one description for the whole verify step ------------------------------------------------------------
 * Shapes and tensors as Config::from_gguf and Model read them (crates/shadowzero-model/src/forward.rs:25-142, tensor names in
 * crates/shadowzero-model/src/exl3_model.rs:223-243).  Every tensor is stored as the reference stores it: ggml [cols = in,
 * rows = out] with whole rows contiguous, or one EXL3 blob.  `data` is a device address for the library (a host address for
 * the CPU oracle, which reads the same structs).  The per-layer embedding (sz_ple) and the sparse indexer (cfg.idx_heads) are
 * optional. */
typedef struct sz_tensor {
    int32_t type;      /* ggml type id; 0 rows = absent */
    int32_t reserved;
    uint64_t data;
    int64_t rows;      /* outputs */
    int64_t cols;      /* inputs */
} sz_tensor;

typedef struct sz_model_config {
    int32_t n_layer, hidden, streams, hc_rank, vocab;
    int32_t n_head, n_kv_head, head_dim, rope_dims;
    int32_t n_expert, n_expert_used, expert_ff, shared_ff;
    int32_t ssm_k_heads, ssm_v_heads, ssm_head_dim, conv_k;
    int32_t attn_interval;      /* layer l is gated attention iff l % attn_interval == attn_interval - 1, else DeltaNet */
    float eps;
    float reserved;
    double rope_theta;
    /* The sparse indexer of the attention layers (forward.rs:63-68, 137-140: attention.indexer.head_count, .key_length, .top_k):
     * heads, head width, and the budget of positions a query attends to.  idx_heads = 0: the model has no indexer and every
     * query attends to every position (what the reference computes while no more than idx_budget positions are complete). */
    int32_t idx_heads, idx_dim, idx_budget, idx_reserved;
} sz_model_config;

typedef struct sz_hc {          /* a hyper-connection read: forward.rs:797-817 */
    sz_tensor norm;             /* F32 [streams * hidden] */
    sz_tensor down;             /* [streams * hidden -> rank] */
    sz_tensor up;               /* [rank -> streams * hidden] */
    sz_tensor inject;           /* [streams * hidden -> streams]; absent for the output read */
} sz_hc;

typedef struct sz_layer {
    sz_hc hc_attn, hc_ffn;
    /* DeltaNet (forward.rs:819-896) */
    sz_tensor attn_qkv, attn_gate, ssm_beta, ssm_alpha, ssm_conv1d, ssm_a, ssm_dt_bias, ssm_norm, ssm_out;
    /* gated attention (forward.rs:898-1007) */
    sz_tensor attn_q, attn_k, attn_v, attn_q_norm, attn_k_norm, attn_output;
    /* the sparse indexer of a gated-attention layer (forward.rs:906-976): indexer.q_proj [hidden -> idx_heads * idx_dim],
     * indexer.k_proj [hidden -> idx_dim], indexer.q_norm / k_norm F32 [idx_dim]; idx_ratio = positions a pooled block
     * (attention.compress_ratios; 0 is read as 1, as the reference reads it).  Absent (rows 0) when cfg.idx_heads = 0. */
    sz_tensor idx_q, idx_k, idx_q_norm, idx_k_norm;
    int32_t idx_ratio, idx_reserved;
    sz_moe_layer moe;
} sz_layer;

/* The per-layer embedding of ONE layer: a hashed n-gram memory added to the whole residual stream before that layer's first read
 * (forward.rs:1036-1074 `ple`, :1177-1198 `ple_rows`, configuration :54-62 and :93-136; the reference implements one such layer).
 * For every n-gram order 2 .. ngram the last `order` tokens (tokens before the last `eos` count as `eos`) are mixed -
 * XOR of token * multipliers[distance], 64-bit wrapping - and each of heads_per_ngram heads takes row
 * (mixed mod vocab[i]) + offsets[i] (the non-negative remainder) of `table`; the (ngram - 1) * heads_per_ngram rows of head_dim
 * weights, side by side, are the embedding e [hidden].  key = norm_key(key . e) per stream, val = value . e, qry = norm_query(r) per
 * stream; a stream's gate is sigmoid(sign(d) sqrt(max(|d|, 1e-6))) with d = key . qry / sqrt(hidden); gv = gate * val;
 * out = gv + silu(depthwise causal conv over norm_conv(gv), kernel conv_k, dilation ngram); r += out.
 * ngram < 2: the model has none (a zeroed struct). */
#define SZ_PLE_MAX_NGRAM 8
#define SZ_PLE_MAX_HEADS 32
typedef struct sz_ple {
    int32_t layer, ngram, heads_per_ngram, head_dim, conv_k, eos;
    int64_t multipliers[SZ_PLE_MAX_NGRAM];
    int64_t vocab[SZ_PLE_MAX_HEADS], offsets[SZ_PLE_MAX_HEADS];
    sz_tensor table;        /* per_layer_token_embd [head_dim -> rows] */
    sz_tensor key;          /* ple_key [hidden -> streams * hidden] */
    sz_tensor value;        /* ple_value [hidden -> hidden] */
    sz_tensor norm_key, norm_query, norm_conv;   /* F32 [streams * hidden] */
    sz_tensor conv1d;       /* F32 [streams * hidden][conv_k]: tap t of a channel multiplies the input (conv_k - 1 - t) * ngram steps back */
} sz_ple;

typedef struct sz_model {
    sz_model_config cfg;
    sz_tensor token_embd;       /* [hidden -> vocab]: row t is token t's embedding */
    sz_tensor output;           /* [hidden -> vocab] */
    sz_hc output_hc;
    const sz_layer* layers;     /* host array of n_layer entries */
    sz_ple ple;                 /* ple.ngram < 2: none */
} sz_model;

/* ---- model files ------------------------------------------------------------------------------------------------------------------
 * A GGUF file into struct sz_model.  Replaces Gguf::open (crates/shadowzero-model/src/gguf.rs:468; header, key-values and tensor table
 * :330-420, type table :99-150 with the EXL3 blob types 1021..1028 sized by the span to the next tensor), Config::from_gguf
 * (crates/shadowzero-model/src/forward.rs:72-142: the `<architecture>.<key>` values behind every field of sz_model_config; vocab from
 * output.weight, :106) and the tensor lookup by name (names and ggml dimension order as crates/shadowzero-model/src/exl3_model.rs:223-243
 * lists them; expert e of a three-dimensional expert tensor at byte e * bytes / n_expert, forward.rs:477-485).
 * placement SZ_PLACE_HOST: the file stays mapped and tensor addresses point into the mapping (for a CPU consumer of the struct).
 * SZ_PLACE_DEVICE: one device allocation made here (loading is not a hot call), every tensor copied to an aligned place of its own -
 * EXL3 blobs so that their trellis starts on a 16-byte boundary, EXL3 expert slices re-strided to a multiple of 16 bytes.
 * The per-layer-embedding branch and the sparse indexer are not part of this build: a file that switches one on (a layer below
 * block_count in ple.layers, a non-zero entry of attention.compress_ratios) is refused with SZ_E_TYPE; their tensors are ignored.
 * sz_weights_model: the description, valid until sz_weights_free.  sz_weights_tensor_info: type, dimensions (ggml order, padded with
 * 1) and byte size of a tensor by name (Gguf::tensor, gguf.rs:512).
 * sz_gguf_open reads the header alone (any GGUF, not only a model of this architecture): the tensor table through
 * sz_weights_tensor_info, integer key-values (an array gives its length) through sz_weights_key_u64; sz_weights_model is null then. */
#define SZ_PLACE_HOST 0
#define SZ_PLACE_DEVICE 1
typedef struct sz_weights sz_weights;
int sz_model_load_gguf(const char* path, int placement, uint64_t stream, sz_weights** out);
int sz_gguf_open(const char* path, sz_weights** out);
int sz_weights_key_u64(const sz_weights* w, const char* key, uint64_t* out);
const sz_model* sz_weights_model(const sz_weights* w);
int64_t sz_weights_bytes(const sz_weights* w);
int sz_weights_tensor_count(const sz_weights* w);
int sz_weights_tensor_info(const sz_weights* w, const char* name, int32_t* type, int64_t dims[4], int64_t* bytes);
void sz_weights_free(sz_weights* w);

/* ---- many-row dense projections on the tensor pipe (tcgen05 + tensor memory) ----------------------------------------------------------
 * y[t * ys + r] = sum_k w[r][k] * x[t * xs + k] for t < m token rows and every row r of w (strides in floats).  The prompt / batched
 * form of a projection: replaces the reference's tensor-core family for a long prompt, kernels/matvec.cu:758-1260 (mma_core,
 * mma_cols_<type>, mma_cols64_<type>; same argument meaning: w, x, xs, y, ys, rows, cols, m) as crates/shadowzero-cuda/src/session.rs:7276
 * launches it, with that family's arithmetic: weights decoded as the reference decodes them (d * q in f32) and rounded to f16,
 * inputs rounded to f16, f32 accumulation, the order of the sum left to the tensor core.  The reference calls the mode inexact and
 * keeps it for prompts; results agree with the exact kernels to about 1e-3 relative, not bit for bit.
 * w: Q8_0, cols a multiple of 256, data 16-byte aligned.  x rows 16-byte aligned.  scratch: sz_mma_cols_scratch_bytes, 256-byte
 * aligned, cleared once by sz_mma_cols_status(scratch, 1, NULL, stream); sz_mma_cols_status(scratch, 0, &code, stream) synchronises
 * and reports whether a bounded wait of the kernel ever ran out (code != 0: results of that call are not valid). */
int sz_mma_cols_scratch_bytes(int cols, int m, int64_t* bytes);
int sz_mma_cols(const sz_tensor* w, uint64_t x, int64_t xs, uint64_t y, int64_t ys, int m, uint64_t scratch, int64_t scratch_bytes, uint64_t stream);
int sz_mma_cols_status(uint64_t scratch, int init, int* code, uint64_t stream);

/* ---- the session: the verify surface ------------------------------------------------------------------------------------
 * Replaces the verify subset of GpuSession (crates/shadowzero-cuda/src/session.rs): step_batch_verify_top (6061-6072), rollback
 * (6217-6276), note_verify, capacity, tokens, and prefill by passes.  One engine thread owns a session (engine.rs:340-420).
 * All device memory comes from the caller: sz_session_bytes sizes one block that holds the KV cache (ctx positions), the DeltaNet
 * states (two copies: a pass never overwrites the state it started from, so a rejection needs no snapshot), and every scratch
 * buffer.  flags: SZ_KV_Q8 keeps K and V as packed per-32 int8 + f16 scales (kernels/forward.cu:3652-3687); 0 keeps f32. */
#define SZ_KV_Q8 1
#define SZ_HEAD_PROXY 2     /* output.weight is an EXL3 blob and the head is screened by its 2-bit proxy (see sz_head below); without the
                             * flag an EXL3 output.weight is evaluated in full.  Blocks kept a row: 128, or the environment's SZ_HEAD_KBLK */
#define SZ_ACCEPT_NONE 0    /* the caller decides: read the top-64 of every row, then sz_session_commit(keep) */
#define SZ_ACCEPT_GREEDY 1  /* on the device: keep row i + 1 while row i's best token is the drafted ids[i + 1] (engine.rs:2377-2408) */
#define SZ_ACCEPT_ALL 2     /* prompt rows: all kept */
#define SZ_ACCEPT_SAMPLED 3 /* on the device, through sz_session_verify_sampled: row i's token is the sampler's draw at output position
                             * pos + i from the row's top-64 (sampler.rs:159-210); row i + 1 is kept while that draw is the drafted ids[i + 1] */
typedef struct sz_session sz_session;
int sz_session_bytes(const sz_model* model, int ctx, int flags, int64_t* bytes);
int sz_session_create(const sz_model* model, int ctx, int flags, uint64_t mem, int64_t bytes, uint64_t stream, sz_session** out);
void sz_session_destroy(sz_session* s);
int sz_session_reset(sz_session* s, uint64_t stream);
int sz_session_len(const sz_session* s);        /* committed positions: GpuSession::tokens().len() */
int sz_session_capacity(const sz_session* s);   /* GpuSession::capacity() */
int sz_session_pending(const sz_session* s);    /* rows of the pass that awaits sz_session_commit (0: none) */
/* Feeds a prompt in passes of up to SZ_MAX_VERIFY rows.  The last pass is left pending: read it with sz_session_result (its last
 * row is the prompt's last token), then sz_session_commit(s, rows of that pass). */
int sz_session_prefill(sz_session* s, const int32_t* ids, int n, uint64_t stream);
/* One pass over ids[0..m): row i's output is what follows ids[..=i] (step_batch_verify).  want_head = 0 skips the output
 * projection (prompt passes).  Asynchronous; the pass stays pending until sz_session_commit. */
int sz_session_verify(sz_session* s, const int32_t* ids, int m, int accept_mode, int eog_token, int want_head, uint64_t stream);
/* Sampled acceptance on the device.  The sampler (a resolved one without penalties, `struct sz_sampler` below) is set once; a pass
 * then names the output position of its first row: row i draws with the counter-based uniform number of (seed, pos + i), exactly
 * as the host loop does (engine.rs:2377-2408 with Sampler::sample_top).  keep_next of sz_session_result = {rows kept, the draw of
 * the last kept row}.  The draw matches sz_sample_top except where the uniform number falls within an ulp of a boundary of the
 * cumulative distribution (the device's double-precision exp is not the host library's). */
struct sz_sampler;
int sz_session_set_sampler(sz_session* s, const struct sz_sampler* sp);
/* Up to 7 further ids that end generation (the tokenizer's other end-of-generation ids, the request's stop tokens: engine.rs:2386
 * `tok.is_eog(d) || stops.contains(&d)`): device acceptance - greedy, sampled, down a tree - never keeps a drafted one, exactly as
 * it never keeps the pass's eog_token.  n = 0 clears the list.  Takes effect with the next pass. */
int sz_session_set_stops(sz_session* s, const int32_t* ids, int n, uint64_t stream);
int sz_session_stops(const sz_session* s, int32_t* out /* room for 7 */);   /* returns how many are set */
int sz_session_verify_sampled(sz_session* s, const int32_t* ids, int m, uint64_t pos, int eog_token, uint64_t stream);
/* Tree verification (no counterpart in the reference, whose verify pass is a chain: session.rs:7698-7723, kernels/forward.cu:1481-1487).
 * One pass over a draft TREE of up to SZ_MAX_VERIFY rows: row 0 is the root (the pass's own token, parents[0] = -1), row j > 0 a drafted
 * token whose parent is row parents[j] < j.  Row j attends to the committed positions, to its ancestors and to itself (a tree mask over
 * the pass's own cache slots), sits at sequence position committed + depth(j), and continues the DeltaNet state and the conv window of
 * its parent (the state after a row that a later row branches off is kept aside during the scan).  Row j's output is what follows the
 * path root .. j.  accept_mode SZ_ACCEPT_GREEDY walks down from the root on the device: the target's best token after the current row
 * must be the token of one of its children (the lowest row among equals), never a drafted end-of-generation token; SZ_ACCEPT_NONE
 * leaves the decision to the caller (sampled acceptance: sz_tree_accept_sampled below, then sz_session_commit_path).
 * Committing keeps a PATH: the recurrent state is replayed along it from the pass's saved inputs, and the kept rows' keys and values
 * move from their rows' cache slots to their depths' positions.  sz_session_result gives {rows kept, next token} and every row's
 * top-64 as for a chain; sz_session_tree_path the kept rows (root first) of a pass the device accepted, which is then closed with
 * sz_session_commit(s, rows kept). */
int sz_session_verify_tree(sz_session* s, const int32_t* ids, const int32_t* parents, int m, int accept_mode, int eog_token, uint64_t stream);
int sz_session_tree_path(sz_session* s, int32_t* path, int* n, uint64_t stream);
int sz_session_commit_path(sz_session* s, const int32_t* path, int n, uint64_t stream);
/* Copies the pending pass's results to the host and synchronises: keep_next[2] = {rows kept by the device's acceptance, the
 * token that follows them}; top = [m][128] u32, 64 logit bit patterns (largest first, ties to the lower id) then 64 token ids
 * (session.rs:6034-6039); logits = [m][vocab] f32.  Any pointer may be null. */
int sz_session_result(sz_session* s, int32_t* keep_next, uint32_t* top, float* logits, uint64_t stream);
/* Keeps the first `keep` rows of the pending pass and drops the rest (rollback(&snap, &batch[..keep])). */
int sz_session_commit(sz_session* s, int keep, uint64_t stream);
/* Several sequences in one step (the batch of config 5, from the pieces above): every sequence keeps its session and runs what
 * carries its own state (embedding, attention, head) in lockstep with the others; the hyper-connection reads, the mixers'
 * projections and the MoE sublayer of every layer take the rows of ALL sequences as one batch, so their weights are streamed once
 * a step and an expert several sequences chose is decoded once (sz_moe_rows); the DeltaNet scans of a layer are one launch.  While the call runs, the sessions' per-pass buffers
 * point into the batch's scratch: no other thread may use those sessions.  n <= 64 sessions of one model (EXL3 experts,
 * no expert sharding) on one stream; ms[b] rows of sequence b, ids = the rows of all sequences one after the other; the rows of
 * a step, padded to a multiple of 8, must fit rows_max (<= 256), the size the scratch was made for.  Afterwards every session
 * holds a pending pass: sz_session_result / sz_session_commit per session.  A sequence's results are bit for bit those of a pass
 * of its own.  sz_batch_scratch_init once after the scratch is allocated. */
int sz_batch_scratch_bytes(const sz_model* model, int rows_max, int64_t* bytes);
int sz_batch_scratch_init(const sz_model* model, int rows_max, uint64_t scratch, uint64_t stream);
int sz_batch_verify(sz_session* const* sessions, int n, const int32_t* ids, const int32_t* ms, int accept_mode, int eog_token, int rows_max,
                    uint64_t scratch, int64_t scratch_bytes, uint64_t stream);
/* sz_session_prefill for n sequences in lockstep: every step takes up to 8 rows of every sequence that still has prompt left (as
 * many sequences a step as rows_max holds; the rest wait their turn), keeps them all, and runs the head only for a prompt's last
 * pass - which is left pending, as sz_session_prefill leaves it: sz_session_result, then sz_session_commit of its
 * (lens[b] - 1) % 8 + 1 rows.  Every sequence's state and results are bit for bit those of its own sz_session_prefill. */
int sz_batch_prefill(sz_session* const* sessions, int n, const int32_t* const* ids, const int32_t* lens, int rows_max, uint64_t scratch,
                     int64_t scratch_bytes, uint64_t stream);
/* Routing trace (the `layerL.route_idx` / `route_w` streams, forward.rs:1015-1018): switch it on, run a pass, read
 * idx [n_layer][SZ_MAX_VERIFY][SZ_MAX_TOPK] and w (same shape, f64). */
/* Benchmarks: pretend `len` tokens were fed - seeded pseudo-random keys and values in the first `len` cache positions of every
 * attention layer, zero recurrent state - so a long context needs no long prefill.  Resets the session first. */
int sz_session_fill_synthetic(sz_session* s, int len, uint32_t seed, uint64_t stream);
/* Copies one piece of the committed state to host memory and synchronises - what GpuSession::snapshot (session.rs:3407-3459) saves,
 * for tests and checkpoints.  DELTA_S: f32 [v heads][d][d] (key index, then value index) and DELTA_CONV: f32 [conv_k - 1][channels],
 * oldest row first, of DeltaNet layer `layer`; KV_K / KV_V: the first sz_session_len positions of attention layer `layer` in the
 * reference's order [position][kv head][head bytes] (head bytes: 4 head_dim, or the packed Q8_KV head).  `bytes` must be the exact
 * size of the piece; no pass may be pending.
 * IDX_SELECTED: what the sparse indexer of attention layer `layer` chose in the last pass (the reference's trace stream
 * `layerL.selected`, forward.rs:997-1004, as block sets): u32 [SZ_MAX_VERIFY][words], words = sz_session_idx_words, bit b of row j
 * = row j attended to complete block b (every complete block, while there are no more than budget / ratio of them).
 * IDX_SCORES: f32 [SZ_MAX_VERIFY][32 * words]: the block scores of the last attention layer the last pass ran (rows that selected). */
#define SZ_STATE_IDX_SELECTED 4
#define SZ_STATE_IDX_SCORES 5
int sz_session_idx_words(const sz_session* s);
#define SZ_STATE_DELTA_S 0
#define SZ_STATE_DELTA_CONV 1
#define SZ_STATE_KV_K 2
#define SZ_STATE_KV_V 3
int sz_session_export(sz_session* s, int what, int layer, void* dst, int64_t bytes, uint64_t stream);
/* The way back (GpuSession::restore, session.rs:3463-3541): sz_session_reset, then every piece a checkpoint holds through
 * sz_session_import - DELTA_S and DELTA_CONV of every DeltaNet layer, KV_K and KV_V of every attention layer with the `positions`
 * they cover (in sz_session_export's layout), for a model with the sparse indexer IDX_RAW: the raw indexer keys, f32
 * [positions][idx_dim] (the pooled block keys are rebuilt from them), for a model with per-layer embeddings PLE_HIST and PLE_TAIL -
 * and last sz_session_set_len(positions).  The session then
 * continues, bit for bit, as the one the pieces were taken from.  No pass may be pending; each call synchronises the stream. */
#define SZ_STATE_IDX_RAW 6
/* the per-layer embedding's carried state (any `layer`): PLE_HIST f32 [(conv_k - 1) * ngram][streams * hidden], oldest row first;
 * PLE_TAIL int32 [8]: the last committed tokens, most recent first (the end-of-text id where the sequence has none) */
#define SZ_STATE_PLE_HIST 7
#define SZ_STATE_PLE_TAIL 8
int sz_session_import(sz_session* s, int what, int layer, const void* src, int64_t bytes, int positions, uint64_t stream);
int sz_session_set_len(sz_session* s, int positions, uint64_t stream);
int sz_session_trace_routes(sz_session* s, int on);
int sz_session_routes(sz_session* s, int32_t* idx, double* w, uint64_t stream);

/* ---- launching a kernel by name -------------------------------------------------------------------------------------------------------
 * The lowest seam of the reference: Program::launch(name, grid, block, shared, stream, args) (crates/shadowzero-cuda/src/kernels.rs:
 * 546-572) over a static registry that spells out every entry point's parameter types (:9-57, 163-477).  Arguments are typed
 * (pointer, const pointer, u32, i32, u64, f32) and travel in 8-byte slots; a device pointer satisfies both pointer kinds, scalars must
 * match exactly; a launch whose count or types do not fit the registry is refused with SZ_E_ARG before anything reaches the driver
 * ("takes 4 arguments", "does not fit": crates/shadowzero-cuda/tests/gpu.rs).  What remains the caller's promise is that every
 * pointer is large enough for what the kernel reads and writes at that grid.  The registry holds the session's kernels with plain
 * parameters; sz_kernel_count / sz_kernel_name / sz_kernel_params enumerate it (the drift test compares it with the sources). */
#define SZ_P_PTR 0
#define SZ_P_CONST_PTR 1
#define SZ_P_U32 2
#define SZ_P_I32 3
#define SZ_P_U64 4
#define SZ_P_F32 5
typedef struct sz_karg { int32_t type; int32_t reserved; uint64_t bits; } sz_karg;   /* bits: the value, zero-extended (f32: its bit pattern) */
int sz_kernel_count(void);
const char* sz_kernel_name(int i);
int sz_kernel_params(const char* name, int32_t* types, int cap);   /* the number of parameters (-1: unknown name); types[0 .. min(n, cap)) */
int sz_kernel_launch(const char* name, const uint32_t grid[3], const uint32_t block[3], uint32_t shared, uint64_t stream, const sz_karg* args,
                     int nargs);

/* ---- the host side of speculation: drafting, the draft policy, sampling, the loop ------------------------------------------------
 * Pure host code (no CUDA): C++ where the reference is Rust.  Token ids are uint32_t, as there. */
/* Prompt lookup: the (up to) k tokens after the latest earlier occurrence of the history's last n tokens, n tried from `lens` in
 * order (lookup_from, crates/shadowzero-serve/src/engine.rs:829-839).  Returns how many were written. */
int sz_lookup(const uint32_t* hist, int n_hist, int k, const int* lens, int n_lens, uint32_t* out);
/* SuffixDrafter (engine.rs:841-1011): trigram index of the history, longest then most recent match, propose_after chaining. */
typedef struct sz_drafter sz_drafter;
sz_drafter* sz_drafter_new(int min_match, int max_match, int capacity_tokens);
void sz_drafter_free(sz_drafter* d);
void sz_drafter_push(sz_drafter* d, uint32_t token);
void sz_drafter_extend(sz_drafter* d, const uint32_t* tokens, int n);
int sz_drafter_len(const sz_drafter* d);
int sz_drafter_propose(const sz_drafter* d, int max_k, uint32_t* out, int* match_len);
int sz_drafter_propose_with_min(const sz_drafter* d, int max_k, int min_match, uint32_t* out, int* match_len);
int sz_drafter_propose_after(sz_drafter* d, const uint32_t* extra, int n_extra, int max_k, uint32_t* out, int* match_len);
/* DraftPolicy (engine.rs:1013-1309): cost-per-millisecond choice between a neural window and a lookup window, chain length, and
 * the adaptive neural depth.  It is consulted only when a neural drafter exists (engine.rs:2253-2264). */
typedef struct sz_draft_policy sz_draft_policy;
sz_draft_policy* sz_policy_new(int max_t, int base_spec, double margin);
void sz_policy_free(sz_draft_policy* p);
double sz_policy_accept_ema(const sz_draft_policy* p);
int sz_policy_neural_k(const sz_draft_policy* p, int rem_tokens);
int sz_policy_choose(const sz_draft_policy* p, int t_neural, int lookup_k, int match_len, int* lookup);
int sz_policy_chain(const sz_draft_policy* p, int t_neural, double p_neural, int k_avail, int match_len);
void sz_policy_observe(sz_draft_policy* p, int lookup, int t, int accepted, int match_len, double round_ms);
void sz_policy_observe_chain(sz_draft_policy* p, int t_neural, int k_chain, int accepted, int match_len, double round_ms);
/* Sampler (crates/shadowzero-serve/src/sampler.rs:83-210), the part that works from a row's top-64: a resolved sampler without
 * penalties (Sampler::top_ok).  sz_uniform is the counter-based number of (seed, position). */
typedef struct sz_sampler { float temperature; int32_t top_k; float top_p; float min_p; uint64_t seed; } sz_sampler;
double sz_uniform(uint64_t seed, uint64_t pos);
uint32_t sz_sample_top(const sz_sampler* sp, const uint32_t* top128, uint64_t pos);
/* Sampled acceptance down a draft tree (no counterpart in the reference): rejection sampling against the drafter's probabilities, level
 * by level.  At the current row the target distribution p is the sampler's over the row's top-64 (the candidates and weights
 * sz_sample_top draws from); its children are tried in row order: child c with token x and draft probability draft_prob[c] = q is kept
 * with probability min(1, p(x) / q); after a refusal p loses q at x (not below zero) and is renormalised; when no child is kept the next
 * token is drawn from what is left of p.  With a drafter that proposes fixed tokens (q = 1: a lookup or suffix drafter) the emitted
 * tokens are distributed exactly as the target's; for a drafter with a spread-out distribution exactness would need its whole
 * distribution in the residual, and the call only knows the drafted tokens' probabilities: an approximation then.  Decisions use
 * sz_uniform(seed, stream): stream 256 P for the draw of the token at output position P, 256 P + 1 + i for the i-th child tried there;
 * `pos` is the output position of the token after the root.  top: [m][128] as sz_session_result gives it.  Returns the rows kept (-1: a
 * bad argument); path: the kept rows, root first (for sz_session_commit_path); *next: the token after them. */
int sz_tree_accept_sampled(const sz_sampler* sp, const uint32_t* top, const uint32_t* ids, const int32_t* parents, int m, const float* draft_prob,
                           uint64_t pos, int eog_token, int32_t* path, uint32_t* next);
/* The draft / verify / accept / commit loop of engine.rs:2149-2454 for `--spec spec_k` with the suffix drafter (no neural
 * drafter, draft policy not consulted): generates up to max_new tokens after the prompt into `out`; pass_log receives
 * (drafted, accepted) per verify pass.  device_accept = 1 lets the device decide acceptance, greedy or sampled (checked against the host's own decision). */
typedef struct sz_gen_params {
    int32_t spec_k, max_new, lookup_min, greedy, eog_token, device_accept;
    sz_sampler sampler;
    int32_t max_rounds;   /* sz_generate: stop after this many rounds of the loop (0: no limit); a round is one pass, drafted or not */
    int32_t reserved;
} sz_gen_params;
typedef struct sz_gen_stats {
    int32_t n_tokens, passes, drafted, accepted, lookup_passes, rounds;
    int32_t pos_tried[8], pos_right[8];
    double draft_ms, verify_ms, commit_ms;   /* host wall clock of the three parts of a round */
    double device_ms;                          /* the passes alone, by events on their stream */
} sz_gen_stats;
int sz_generate(sz_session* s, const uint32_t* prompt, int n_prompt, const sz_gen_params* p, uint32_t* out, int32_t* pass_log, int pass_cap,
                sz_gen_stats* stats, uint64_t stream);
/* The same loop in pieces, so that a caller can run some rounds, look, and run more: sz_gen_begin feeds the prompt, sz_gen_run runs
 * up to `rounds` rounds (0: to the end) appending to `out` and accumulating into `stats` (zero it before the first call). */
typedef struct sz_gen sz_gen;
int sz_gen_begin(sz_session* s, const uint32_t* prompt, int n_prompt, const sz_gen_params* p, uint64_t stream, sz_gen** out);
int sz_gen_run(sz_gen* g, int rounds, uint32_t* out, int32_t* pass_log, int pass_cap, sz_gen_stats* stats, uint64_t stream);
/* The loop of n sequences in lockstep (generators made by sz_gen_begin on sessions of one model): every round each live sequence
 * proposes its rows, one sz_batch_verify step verifies them all, each sequence settles its own.  Greedy acceptance on the device.
 * outs[b] / stats[b] as sz_gen_run's; *device_ms accumulates the steps' device time.  A sequence's tokens are those of its own loop. */
int sz_batch_gen_run(sz_gen* const* gens, int n, int rounds, uint32_t* const* outs, sz_gen_stats* const* stats, int rows_max, uint64_t scratch,
                     int64_t scratch_bytes, double* device_ms, uint64_t stream);
/* sz_gen_begin for n sequences at once: the prompts go through sz_batch_prefill; gens[b] is sequence b's generator, as sz_gen_begin
 * on its own would have made it (one parameter block for all). */
int sz_batch_gen_begin(sz_session* const* sessions, int n, const uint32_t* const* prompts, const int32_t* n_prompts, const sz_gen_params* p, int rows_max,
                       uint64_t scratch, int64_t scratch_bytes, uint64_t stream, sz_gen** gens);
/* the request's stop ids for the loop: it ends at one as at eog_token, and never accepts a drafted one (host and device alike) */
int sz_gen_set_stops(sz_gen* g, const uint32_t* ids, int n, uint64_t stream);
void sz_gen_free(sz_gen* g);

/* ---- expert parallelism over NCCL ------------------------------------------------------------------------------------------
 * No counterpart in the reference (its only multi-GPU mode is a two-stage layer split through host memory,
 * crates/shadowzero-cuda/src/session.rs:6945-7015; expert parallelism was estimated and not built, docs/STATUS.md:1922).
 * Experts are sharded by contiguous id range; router, attention, DeltaNet and the head are replicated, so every rank routes
 * the same rows by itself and runs only the experts it holds: the dispatch exchange is empty.  The combine is one all-reduce
 * per MoE layer of the weighted expert outputs as 64-bit fixed point (scale 2^40): integer addition is exact, so the result is
 * the same bits for any number of ranks.  sz_ep_unique_id makes the NCCL id on one rank; the host carries it to the others
 * (torch.distributed, MPI, a file); sz_ep_init joins.  One communicator per process; NCCL is loaded with dlopen at this point. */
int sz_ep_unique_id(uint8_t id[128]);
int sz_ep_init(int rank, int world, const uint8_t id[128]);
int sz_ep_world(void);
/* Refused (SZ_E_ARG) while a session that recorded passes over the communicator is alive: destroy the sessions first. */
int sz_ep_destroy(void);
/* The two halves of an expert-parallel MoE pass, for hosts that exchange the partial sums themselves (and for testing several
 * ranks on one GPU): the partial (int64 [m][hidden], this rank's experts only), and the conversion of a summed buffer to f32. */
int sz_moe_verify_partial(const sz_moe_layer* layer, uint64_t x, int m, uint64_t y_fix, uint64_t scratch, int64_t scratch_bytes,
                          uint64_t stream);
int sz_moe_finish(uint64_t y_fix, int m, int hidden, uint64_t y, uint64_t stream);

/* The same exchange without a collective library on the data path: every rank owns an exchange buffer that its peers map (CUDA
 * IPC over NVLink).  The combine kernel of a layer stores the rank's fixed-point share straight into every rank's buffer and bumps
 * an arrival counter there; the finish kernel waits - a bounded number of polls - for all sources and adds the shares.  When an
 * exchange is attached, expert-parallel layers use it instead of NCCL (sz_ep_init is then not needed).
 *   sz_ep_p2p_bytes / _alloc / _free: the buffer (an allocation of its own, zeroed: IPC exports whole allocations);
 *   sz_ep_ipc_export / _import / _close: the 64-byte handle the host carries to the peers, and the mapping on their side;
 *   sz_ep_p2p_attach(rank, world, hidden, bufs): bufs[r] = rank r's buffer as this process addresses it; _detach;
 *   sz_ep_p2p_status: 1 in *error once a wait of this rank ran out (a peer died or fell behind by more than the poll budget):
 *   the pass still ends, its output is wrong, and every later wait of this rank returns at once.
 * All ranks must attach zeroed buffers and then run the same sequence of passes.
 * A session's recorded passes (CUDA graphs) carry the attached addresses: while such a session is alive sz_ep_p2p_attach and
 * sz_ep_p2p_detach return SZ_E_ARG, and sz_ep_p2p_free / sz_ep_ipc_close refuse a buffer that is attached.  Destroy the sessions,
 * detach, then close and free.  Passes recorded before an attach (or an sz_ep_init) are dropped and recorded again.
 * sz_moe_verify_partial with y_fix = 0 pushes the share; sz_moe_finish_exchange adds up (the two halves, for tests that run several
 * ranks on one GPU one after the other). */
int sz_ep_p2p_bytes(int world, int hidden, int64_t* bytes);
int sz_ep_p2p_alloc(int64_t bytes, uint64_t* ptr);
int sz_ep_p2p_free(uint64_t ptr);
int sz_ep_ipc_export(uint64_t ptr, uint8_t handle[64]);
int sz_ep_ipc_import(const uint8_t handle[64], uint64_t* ptr);
int sz_ep_ipc_close(uint64_t ptr);
int sz_ep_p2p_attach(int rank, int world, int hidden, const uint64_t* bufs);
int sz_ep_p2p_detach(void);
int sz_ep_p2p_world(void);
int sz_ep_p2p_status(int* error);
int sz_moe_finish_exchange(const sz_moe_layer* layer, int m, uint64_t y, uint64_t stream);

/* sz_moe_verify without a scratch argument.  (No counterpart in the reference: its session always owns a scratch buffer.)
 * For hosts that cannot allocate device memory once they are running - an engine that gave all of it to its own arena at start-up,
 * a plugin in a process that forbids the CUDA allocator after initialisation (a cudaMalloc would stall every stream of the GPU) -
 * and so have no buffer to pass.  The scratch is a fixed array of sz_moe_static_scratch_max() bytes (4 MiB) that the library keeps
 * in the memory of every GPU that loads it, until the process exits.  The call allocates nothing.
 *   - A layer shape and row count whose sz_moe_scratch_bytes exceeds the array is refused with SZ_E_SCRATCH.
 *   - The first call on a device looks the array up and clears its counters (a synchronous clear: it is ordered before work on
 *     every stream); make that call before any stream capture begins.
 *   - The array's address is private, so the error word that a kernel raises when one of its bounded waits runs out is read with
 *     sz_moe_static_status (it synchronises the stream); nonzero means the y of that call is not valid.  sz_moe_static_reset clears
 *     the control words again - the static twin of sz_moe_scratch_init - and looks the array up anew: call it after a failed call,
 *     and after a cudaDeviceReset (the address the library remembered is stale then).
 *   - All calls on a device share the one array, and it keeps what the last call left: two calls that can overlap on the GPU
 *     (different streams without an ordering between them) race.  Calls on one stream, or ordered by events, are safe. */
int sz_moe_static_scratch_max(int64_t* bytes);
int sz_moe_static_status(int* error, uint64_t stream);
int sz_moe_static_reset(void);
int sz_moe_verify_static(const sz_moe_layer* layer, uint64_t x, int m, uint64_t y, uint64_t route_idx, uint64_t route_w,
                         uint64_t stream);

/* ---- lm_head over an EXL3 output.weight, dense or screened by the 2-bit proxy ("Q2_P") -------------------------------------------
 * Replaces HeadProxy (crates/shadowzero-cuda/src/session.rs:428-452, built at 2631-2674 by exl3_build_q2_proxy_*,
 * kernels/exl3.cu:915-996), mv_head_proxy_sparse (session.rs:5950-5995: exl3_rotate_rows_f32 kernels/exl3.cu:609-625,
 * proxy_q2_quant_x / proxy_q2_dp4a_bmax_* / proxy_pick_rows / proxy_compact_seen kernels/forward.cu:4367-4632,
 * matvec_cols_exl3_pre_sparse_* kernels/exl3.cu:349-480) and head_top_at (session.rs:5997-6022: topk_slices_blks, topk_merge_blks,
 * kernels/forward.cu:4635-4680).
 * rows = vocabulary, cols = hidden, both multiples of 128 (cols <= 4096, rows <= 262144); bits = 2..6 or 8; the blob sits at an
 * address = 12 mod 16.  k_blk = 0: every 128-output block is evaluated (the exact head) and w_q2 / w_sc may be 0.  k_blk > 0
 * (clamped to 16 .. rows / 128; the reference's default is 128): each row of the pass keeps its k_use best blocks by proxy score,
 * k_use = k_blk, or max(64, 3 k_blk / 4) when need_k <= 16 (session.rs:5964); only the union of those blocks is evaluated, so a
 * token outside them cannot appear in the top-64 (the reference uses this form for serving, never for its exact path). */
typedef struct sz_head {
    int32_t rows, cols, bits, k_blk;
    uint64_t weight;             /* the EXL3 blob of output.weight */
    uint64_t w_q2, w_sc;         /* the proxy: sz_head_proxy_bytes sizes them, sz_head_proxy_build fills them */
    uint64_t work;               /* sz_head_work_bytes bytes, 256-byte aligned, cleared once by sz_head_work_init */
    int64_t work_bytes;
} sz_head;
int sz_head_proxy_bytes(int rows, int cols, int64_t* q2_bytes, int64_t* sc_bytes);
int sz_head_work_bytes(int rows, int cols, int k_blk, int64_t* bytes);
int sz_head_work_init(const sz_head* h, uint64_t stream);
int sz_head_proxy_build(const sz_head* h, uint64_t stream);
/* What a pass of m rows will do: blocks kept a row, the length of the block list, and the row stride of its logits (elements):
 * max_sel * 128 packed logits with the proxy, `rows` without. */
int sz_head_plan(const sz_head* h, int m, int need_k, int32_t* k_use, int32_t* max_sel, int64_t* logits_stride);
/* x: f32 [m][xstride] device rows.  logits: f32 [m][logits_stride] (with the proxy: block list entry s at elements 128 s ..).
 * top: u32 [m][128], the layout of sz_session_result.  Asynchronous on `stream`, capturable, no allocation. */
int sz_head_top(const sz_head* h, uint64_t x, int xstride, int m, int need_k, uint64_t logits, uint64_t top, uint64_t stream);
/* Where the intermediate buffers of the last sz_head_top live inside `work` (tests, traces): rotated rows f32 [8][cols]; their
 * int8 codes [8][cols]; block scales and bias terms f32 [8][cols / 128]; block maxima f32 [8][rows / 128]; the block list u32
 * {count, blocks ascending}; the error word (nonzero: a bounded wait ran out). */
#define SZ_HEAD_XR 0
#define SZ_HEAD_XQ 1
#define SZ_HEAD_XSC 2
#define SZ_HEAD_XCORR 3
#define SZ_HEAD_BMAX 4
#define SZ_HEAD_SEL 5
#define SZ_HEAD_ERR 6
int sz_head_stage(const sz_head* h, int what, uint64_t* addr, int64_t* bytes);

#ifdef __cplusplus
}
#endif
#endif
