// The MoE sublayer of a verify pass: shared definitions (plan tables, scratch layout).
#pragma once

#include "sz_formats.cuh"

#define SZ_MAXG (SZ_MAX_VERIFY * SZ_MAX_TOPK)  // most groups (distinct experts) a pass of SZ_MAX_VERIFY rows can touch
#define SZ_MAX_EXPERTS 1024

// The routed work of one pass, grouped by expert so a matrix is streamed once for every row that chose it.  Groups are in
// ascending expert order; inside a group the rows are in ascending row order.  (The reference's group record is
// [count, in rows.., out rows..], crates/shadowzero-cuda/src/session.rs:2129-2146; pair = row * top_k + rank.)
// Expert-parallel exchange over peer memory (no collective library on the data path).  Every rank owns one exchange buffer that
// its peers map (CUDA IPC): a header, one arrival counter a source rank, and two slots of [ranks][8 * hidden] 64-bit fixed-point
// partial outputs.  The combine kernel of rank `me` stores its partial output into slot (epoch & 1), row `me`, of EVERY rank's
// buffer (plain stores over NVLink), fences, and bumps the arrival counter `me` of every rank; the finish kernel of a rank waits
// (bounded) until every source's counter reached the round's target, adds the rows - integers, so any order gives the same bits -
// and converts.  Two slots are enough: a rank can only start round e + 2 after every peer has sent round e + 1, which a peer does
// only after it has finished reading round e.
#define SZ_EP_MAX_RANKS 8
#define SZ_EP_HDR_BYTES 2048           // header (128) + 8 counters on lines of their own, padded
#define SZ_EP_SPIN_LIMIT 1000000       // polls of a counter (about a microsecond each) before a waiting block gives up and raises the error word

struct SzEpHeader {
    unsigned long long epoch;    // exchanges completed by this rank
    unsigned long long target;   // arrivals a source has made once the current exchange is complete, minus this exchange's
    unsigned int ticket;         // finish blocks done in the current exchange
    unsigned int error;          // a wait ran out
};

struct SzEpPush {
    u8* buf[SZ_EP_MAX_RANKS];    // every rank's exchange buffer as this process sees it (own or mapped)
    int world, me;
    long long row_elems;         // 8 * hidden: elements between two ranks' rows of a slot
};

__device__ __forceinline__ long long* sz_ep_slot(u8* buf, int world, long long row_elems, int slot, int src) {
    return (long long*)(buf + SZ_EP_HDR_BYTES) + ((long long)slot * world + src) * row_elems;
}
__device__ __forceinline__ unsigned long long* sz_ep_arrive(u8* buf, int src) { return (unsigned long long*)(buf + 128 + 128 * src); }

struct SzPlan {
    int32_t n_groups;
    int32_t pad[3];
    // compact types (experts < 32768, at most 8 rows, at most 128 pairs): the whole plan is 2.4 KB, small enough for a consumer
    // kernel to copy into shared memory in one sweep
    int16_t expert[SZ_MAXG];
    uint8_t count[SZ_MAXG];
    uint8_t rows[SZ_MAXG][SZ_MAX_VERIFY];   // row j of x
    uint8_t pairs[SZ_MAXG][SZ_MAX_VERIFY];  // j * top_k + rank: row of the per-pair buffers
};
static_assert(SZ_MAX_VERIFY * SZ_MAX_TOPK <= 256, "pair indices are bytes");

// Offsets (bytes) into the caller's scratch buffer.
struct SzMoeScratch {
    int64_t ctrl;      // u32[16]: [0] router ticket, [1] error flag
    int64_t logits;    // f32 [m][n_expert + 1] (column n_expert: the shared expert's gate logit)
    int64_t ridx;      // i32 [m][top_k]
    int64_t rw;        // f64 [m][top_k]
    int64_t plan;      // SzPlan: routed experts
    int64_t plan_sh;   // SzPlan: the shared expert (one group of all m rows)
    int64_t g, u;      // f32 [m * top_k][FF]: gate (or the SwiGLU product) and up outputs of the routed experts
    int64_t sg, su;    // f32 [m][SF]: the same for the shared expert
    int64_t eo;        // f32 [m * top_k][H]: down outputs per pair
    int64_t so;        // f32 [m][H]: the shared expert's output
    int64_t acc_gu;    // i64 [m * top_k + m][2][FF]: fixed-point gate / up sums of the streaming kernels (pairs, then shared rows)
    int64_t acc_d;     // i64 [m * top_k + m][H]: fixed-point down sums
    int64_t acc_bytes; // acc_gu and acc_d are contiguous: this many bytes are zeroed at the start of a call
    int64_t y_fix;     // i64 [m][H]: this rank's share of the output in fixed point (expert parallelism)
    int64_t total;
};

static inline int64_t sz_up256(int64_t v) { return (v + 255) & ~(int64_t)255; }

static inline SzMoeScratch sz_moe_layout(const sz_moe_layer* L, int m) {
    SzMoeScratch s;
    int64_t o = 0;
    const int64_t pairs = (int64_t)m * L->top_k;
    s.ctrl = o; o += 256;
    s.logits = o; o = sz_up256(o + 4 * (int64_t)m * (L->n_expert + 1));
    s.ridx = o; o = sz_up256(o + 4 * pairs);
    s.rw = o; o = sz_up256(o + 8 * pairs);
    s.plan = o; o = sz_up256(o + (int64_t)sizeof(SzPlan));
    s.plan_sh = o; o = sz_up256(o + (int64_t)sizeof(SzPlan));
    s.g = o; o = sz_up256(o + 4 * pairs * L->expert_ff);
    s.u = o; o = sz_up256(o + 4 * pairs * L->expert_ff);
    s.sg = o; o = sz_up256(o + 4 * (int64_t)m * L->shared_ff);
    s.su = o; o = sz_up256(o + 4 * (int64_t)m * L->shared_ff);
    s.eo = o; o = sz_up256(o + 4 * pairs * L->hidden);
    s.so = o; o = sz_up256(o + 4 * (int64_t)m * L->hidden);
    const int64_t ffm = L->expert_ff > L->shared_ff ? L->expert_ff : L->shared_ff;
    s.acc_gu = o; o = sz_up256(o + 8 * (pairs + m) * 2 * ffm);
    s.acc_d = o; o = sz_up256(o + 8 * (pairs + m) * L->hidden);
    s.acc_bytes = o - s.acc_gu;
    s.y_fix = o; o = sz_up256(o + 8 * (int64_t)m * L->hidden);
    s.total = o;
    return s;
}
