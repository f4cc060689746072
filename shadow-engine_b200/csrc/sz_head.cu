// C-ABI of the output projection over an EXL3 output.weight: the dense form and the screened form (2-bit proxy, block pick,
// sparse rescore, top-64 over the packed logits).  Stands where HeadProxy, mv_head_proxy_sparse and head_top_at stand in the
// reference (crates/shadowzero-cuda/src/session.rs:428-452, 2631-2674, 5950-6022).
#include "sz_head.cuh"

#include <stdlib.h>

namespace {

struct HeadWork {
    float* xr; u32* xq; float* x_sc; float* x_corr; float* bmax; u32* seen; u32* ctrl; u32* sel; u64* tk;
    int n_b, n_ob, max_sel, nb_tk;
    int64_t bytes;
};

int head_shape(int rows, int cols, int k_blk, const char* who) {
    if (rows < 128 || cols < 128 || rows % 128 || cols % 128 || cols > 4096 || rows > 256 * SZ_HEAD_PICK_KEYS * 128)
        return sz_fail(SZ_E_ARG, "%s: %d outputs x %d inputs: whole 128-blocks, at most 4096 inputs and %d outputs", who, rows, cols,
                       256 * SZ_HEAD_PICK_KEYS * 128);
    if (k_blk < 0) return sz_fail(SZ_E_ARG, "%s: k_blk = %d", who, k_blk);
    return SZ_OK;
}

int clamp_kblk(int k_blk, int n_ob) { return k_blk < 16 ? (16 < n_ob ? 16 : n_ob) : (k_blk < n_ob ? k_blk : n_ob); }

// session.rs:5964
int k_use_of(int k_blk, int need_k) {
    if (need_k > 16) return k_blk;
    int k = k_blk * 3 / 4;
    if (k < 64) k = 64;
    return k < k_blk ? k : k_blk;
}

HeadWork head_work(int rows, int cols, int k_blk, u8* base) {
    HeadWork w = {};
    w.n_b = cols / 128;
    w.n_ob = rows / 128;
    const int kb = k_blk > 0 ? clamp_kblk(k_blk, w.n_ob) : 0;
    w.max_sel = kb > 0 ? (SZ_MAX_VERIFY * kb < w.n_ob ? SZ_MAX_VERIFY * kb : w.n_ob) : 0;
    const int64_t ls = kb > 0 ? (int64_t)w.max_sel * 128 : rows;
    w.nb_tk = (int)((ls + SZ_TK_N - 1) / SZ_TK_N);
    int64_t off = 0;
    auto take = [&](int64_t n) { const int64_t o = off; off += (n + 255) & ~(int64_t)255; return base + o; };
    w.xr = (float*)take(4LL * SZ_MAX_VERIFY * cols);
    w.xq = (u32*)take(4LL * SZ_MAX_VERIFY * w.n_b * 32);
    w.x_sc = (float*)take(4LL * SZ_MAX_VERIFY * w.n_b);
    w.x_corr = (float*)take(4LL * SZ_MAX_VERIFY * w.n_b);
    w.bmax = (float*)take(4LL * SZ_MAX_VERIFY * w.n_ob);
    w.seen = (u32*)take(4LL * ((w.n_ob + 31) / 32));
    w.ctrl = (u32*)take(16);
    w.sel = (u32*)take(4LL * (1 + w.max_sel));
    w.tk = (u64*)take(8LL * SZ_MAX_VERIFY * w.nb_tk * 64);
    w.bytes = off;
    return w;
}

int head_check(const sz_head* h, const char* who, bool need_proxy) {
    if (!h) return sz_fail(SZ_E_ARG, "%s: null head", who);
    int rc = head_shape(h->rows, h->cols, h->k_blk, who);
    if (rc) return rc;
    if (h->bits < 2 || h->bits > 8 || h->bits == 7) return sz_fail(SZ_E_TYPE, "%s: EXL3 at %d bits has no head kernel (2..6 and 8 do)", who, h->bits);
    if (!h->weight || ((h->weight + 4) & 15)) return sz_fail(SZ_E_ARG, "%s: the blob must sit at an address = 12 mod 16 (its trellis 16-byte aligned)", who);
    if ((need_proxy || h->k_blk > 0) && (!h->w_q2 || !h->w_sc || (h->w_q2 & 15) || (h->w_sc & 1)))
        return sz_fail(SZ_E_ARG, "%s: null or misaligned proxy buffers", who);
    return SZ_OK;
}

template <int K>
int launch_build(const sz_head* h, cudaStream_t st) {
    SZ_CUDA(sz_launch("head_proxy_build", sz_head_build_kernel<K>, dim3(h->rows / 128, h->cols / 128), dim3(256), 0, st, false, (const u8*)h->weight,
                      (int)h->rows, (int)h->cols, (u8*)h->w_q2, (u16*)h->w_sc));
    return SZ_OK;
}

template <int K, int MC>
int launch_exl3_mc(const sz_head* h, const HeadWork& w, int m, int grid, const u32* sel, float* logits, int ls, cudaStream_t st) {
    const size_t smem = SzHeadX<K, MC>::smem_bytes(w.n_b);
    static bool set = false;  // one attribute a kernel instance
    if (!set) {
        SZ_CUDA(cudaFuncSetAttribute(sz_head_exl3_kernel<K, MC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        set = true;
    }
    if (smem > 200 * 1024) return sz_fail(SZ_E_ARG, "sz_head_top: %d inputs at %d bits need %zu bytes of shared memory", (int)h->cols, K, smem);
    SZ_CUDA(sz_launch("head_exl3", sz_head_exl3_kernel<K, MC>, dim3(grid), dim3(SZ_X3_THREADS), smem, st, true, (const u8*)h->weight, (int)h->rows,
                      (int)h->cols, (const float*)w.xr, m, sel, logits, ls, w.ctrl + 1));
    return SZ_OK;
}
template <int K>
int launch_exl3(const sz_head* h, const HeadWork& w, int m, int grid, const u32* sel, float* logits, int ls, cudaStream_t st) {
    return m <= 4 ? launch_exl3_mc<K, 4>(h, w, m, grid, sel, logits, ls, st) : launch_exl3_mc<K, 8>(h, w, m, grid, sel, logits, ls, st);
}

#define SZ_HEAD_BITS(CALL)                  \
    switch (h->bits) {                      \
        case 2: return CALL(2);             \
        case 3: return CALL(3);             \
        case 4: return CALL(4);             \
        case 5: return CALL(5);             \
        case 6: return CALL(6);             \
        default: return CALL(8);            \
    }

}  // namespace

extern "C" int sz_head_proxy_bytes(int rows, int cols, int64_t* q2_bytes, int64_t* sc_bytes) {
    int rc = head_shape(rows, cols, 0, "sz_head_proxy_bytes");
    if (rc) return rc;
    if (q2_bytes) *q2_bytes = (int64_t)rows * cols / 4;
    if (sc_bytes) *sc_bytes = (int64_t)rows * (cols / 128) * 2;
    return SZ_OK;
}

extern "C" int sz_head_work_bytes(int rows, int cols, int k_blk, int64_t* bytes) {
    int rc = head_shape(rows, cols, k_blk, "sz_head_work_bytes");
    if (rc) return rc;
    if (!bytes) return sz_fail(SZ_E_ARG, "sz_head_work_bytes: null result");
    *bytes = head_work(rows, cols, k_blk, nullptr).bytes;
    return SZ_OK;
}

extern "C" int sz_head_work_init(const sz_head* h, uint64_t stream) {
    int rc = head_check(h, "sz_head_work_init", false);
    if (rc) return rc;
    const HeadWork w = head_work(h->rows, h->cols, h->k_blk, (u8*)h->work);
    if (!h->work || (h->work & 255) || h->work_bytes < w.bytes) return sz_fail(SZ_E_SCRATCH, "sz_head_work_init: the work buffer needs %lld bytes, 256-byte aligned", (long long)w.bytes);
    SZ_CUDA(cudaMemsetAsync((void*)h->work, 0, (size_t)w.bytes, (cudaStream_t)stream));
    return SZ_OK;
}

extern "C" int sz_head_proxy_build(const sz_head* h, uint64_t stream) {
    int rc = head_check(h, "sz_head_proxy_build", true);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
#define SZ_CALL(KK) launch_build<KK>(h, st)
    SZ_HEAD_BITS(SZ_CALL)
#undef SZ_CALL
}

extern "C" int sz_head_plan(const sz_head* h, int m, int need_k, int32_t* k_use, int32_t* max_sel, int64_t* logits_stride) {
    int rc = head_check(h, "sz_head_plan", false);
    if (rc) return rc;
    if (m < 1 || m > SZ_MAX_VERIFY) return sz_fail(SZ_E_ARG, "sz_head_plan: %d rows", m);
    const int n_ob = h->rows / 128;
    int ku = 0, ms = 0;
    if (h->k_blk > 0) {
        ku = k_use_of(clamp_kblk(h->k_blk, n_ob), need_k);
        ms = m * ku < n_ob ? m * ku : n_ob;
    }
    if (k_use) *k_use = ku;
    if (max_sel) *max_sel = ms;
    if (logits_stride) *logits_stride = h->k_blk > 0 ? (int64_t)ms * 128 : h->rows;
    return SZ_OK;
}

extern "C" int sz_head_top(const sz_head* h, uint64_t x, int xstride, int m, int need_k, uint64_t logits, uint64_t top, uint64_t stream) {
    int rc = head_check(h, "sz_head_top", false);
    if (rc) return rc;
    if (m < 1 || m > SZ_MAX_VERIFY) return sz_fail(SZ_E_ARG, "sz_head_top: %d rows (1..%d)", m, SZ_MAX_VERIFY);
    if (!x || (x & 3) || xstride < h->cols || !logits || (logits & 3) || !top || (top & 3)) return sz_fail(SZ_E_ARG, "sz_head_top: null or misaligned buffer");
    const HeadWork w = head_work(h->rows, h->cols, h->k_blk, (u8*)h->work);
    if (!h->work || (h->work & 255) || h->work_bytes < w.bytes) return sz_fail(SZ_E_SCRATCH, "sz_head_top: the work buffer needs %lld bytes, 256-byte aligned", (long long)w.bytes);
    cudaStream_t st = (cudaStream_t)stream;
    const bool proxy = h->k_blk > 0;
    SZ_CUDA(sz_launch("head_rotate", sz_head_rotate_kernel, dim3((m * w.n_b + 7) / 8), dim3(256), 0, st, true, (const u8*)h->weight, (const float*)x,
                      xstride, (int)h->cols, m, w.xr, w.xq, w.x_sc, w.x_corr, proxy ? 1 : 0));
    int grid = w.n_ob, ls = h->rows;
    const u32* sel = nullptr;
    if (proxy) {
        const int ku = k_use_of(clamp_kblk(h->k_blk, w.n_ob), need_k);
        const int ms = m * ku < w.n_ob ? m * ku : w.n_ob;
        const size_t smem = (size_t)m * w.n_b * (128 + 8);
        if (m == 1)
            SZ_CUDA(sz_launch("head_proxy", sz_head_proxy_kernel<1>, dim3(w.n_ob), dim3(128), smem, st, true, (const u8*)h->w_q2, (const u16*)h->w_sc,
                              (const u32*)w.xq, (const float*)w.x_sc, (const float*)w.x_corr, w.bmax, w.n_ob, (int)h->cols, m));
        else if (m <= 4)
            SZ_CUDA(sz_launch("head_proxy", sz_head_proxy_kernel<4>, dim3(w.n_ob), dim3(128), smem, st, true, (const u8*)h->w_q2, (const u16*)h->w_sc,
                              (const u32*)w.xq, (const float*)w.x_sc, (const float*)w.x_corr, w.bmax, w.n_ob, (int)h->cols, m));
        else
            SZ_CUDA(sz_launch("head_proxy", sz_head_proxy_kernel<8>, dim3(w.n_ob), dim3(128), smem, st, true, (const u8*)h->w_q2, (const u16*)h->w_sc,
                              (const u32*)w.xq, (const float*)w.x_sc, (const float*)w.x_corr, w.bmax, w.n_ob, (int)h->cols, m));
        SZ_CUDA(sz_launch("head_pick", sz_head_pick_kernel, dim3(m), dim3(256), 0, st, true, (const float*)w.bmax, w.n_ob, ku, ms, w.seen, w.ctrl, w.sel));
        grid = ms;
        ls = ms * 128;
        sel = w.sel;
    }
    float* lg = (float*)logits;
#define SZ_CALL(KK) launch_exl3<KK>(h, w, m, grid, sel, lg, ls, st)
    auto run = [&]() -> int { SZ_HEAD_BITS(SZ_CALL) };
#undef SZ_CALL
    if ((rc = run())) return rc;
    const int nb = (ls + SZ_TK_N - 1) / SZ_TK_N;
    SZ_CUDA(sz_launch("topk_slices", sz_topk_slices_kernel, dim3(nb, m), dim3(256), 0, st, true, (const float*)lg, (int)h->rows, ls, nb, w.tk, sel));
    SZ_CUDA(sz_launch("topk_merge", sz_topk_merge_kernel, dim3(m), dim3(256), 0, st, true, (const u64*)w.tk, nb, (u32*)top));
    return SZ_OK;
}

// Addresses of the stage's intermediate buffers inside the work buffer, for tests and traces.
extern "C" int sz_head_stage(const sz_head* h, int what, uint64_t* addr, int64_t* bytes) {
    int rc = head_check(h, "sz_head_stage", false);
    if (rc) return rc;
    if (!addr || !bytes) return sz_fail(SZ_E_ARG, "sz_head_stage: null result");
    const HeadWork w = head_work(h->rows, h->cols, h->k_blk, (u8*)h->work);
    switch (what) {
        case SZ_HEAD_XR: *addr = (uint64_t)w.xr; *bytes = 4LL * SZ_MAX_VERIFY * h->cols; break;
        case SZ_HEAD_XQ: *addr = (uint64_t)w.xq; *bytes = 4LL * SZ_MAX_VERIFY * w.n_b * 32; break;
        case SZ_HEAD_XSC: *addr = (uint64_t)w.x_sc; *bytes = 4LL * SZ_MAX_VERIFY * w.n_b; break;
        case SZ_HEAD_XCORR: *addr = (uint64_t)w.x_corr; *bytes = 4LL * SZ_MAX_VERIFY * w.n_b; break;
        case SZ_HEAD_BMAX: *addr = (uint64_t)w.bmax; *bytes = 4LL * SZ_MAX_VERIFY * w.n_ob; break;
        case SZ_HEAD_SEL: *addr = (uint64_t)w.sel; *bytes = 4LL * (1 + w.max_sel); break;
        case SZ_HEAD_ERR: *addr = (uint64_t)(w.ctrl + 1); *bytes = 4; break;
        default: return sz_fail(SZ_E_ARG, "sz_head_stage: unknown buffer %d", what);
    }
    return SZ_OK;
}
