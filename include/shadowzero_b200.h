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
/* Number of kernel launches one sz_moe_verify call makes for this layer (for launch accounting). */
int sz_moe_launches(const sz_moe_layer* layer);

/* sz_moe_verify without a scratch argument.  (No counterpart in the reference: its session always owns a scratch buffer.)
 * For hosts that cannot allocate device memory once they are running - an engine that gave all of it to its own arena at start-up,
 * a plugin in a process that forbids the CUDA allocator after initialisation (a cudaMalloc would stall every stream of the GPU) -
 * and so have no buffer to pass.  The scratch is a fixed array of sz_moe_static_scratch_max() bytes (4 MiB) that the library keeps
 * in the memory of every GPU that loads it, until the process exits.  The call allocates nothing.
 *   - A layer shape and row count whose sz_moe_scratch_bytes exceeds the array is refused with SZ_E_SCRATCH.
 *   - The first call on a device looks the array up and clears its counters; make that call before any stream capture begins.
 *   - All calls on a device share the one array, and it keeps what the last call left: two calls that can overlap on the GPU
 *     (different streams without an ordering between them) race.  Calls on one stream, or ordered by events, are safe. */
int sz_moe_static_scratch_max(int64_t* bytes);
int sz_moe_verify_static(const sz_moe_layer* layer, uint64_t x, int m, uint64_t y, uint64_t route_idx, uint64_t route_w,
                         uint64_t stream);

#ifdef __cplusplus
}
#endif
#endif
