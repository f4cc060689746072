// GGUF model files into struct sz_model: the loader side of the verify session.
//
// Follows the reference's reader (crates/shadowzero-model/src/gguf.rs:330-420: header, key-values, tensor table, data section at
// the next multiple of general.alignment, type table :99-150 with the EXL3 ids 1021..1028 as blob types whose size is the span to
// the next tensor), its Config::from_gguf (crates/shadowzero-model/src/forward.rs:72-142: which keys make which field) and its
// tensor names and dimension order (crates/shadowzero-model/src/exl3_model.rs:223-243; ggml order: dims[0] is the row length).
// Expert tensors are three-dimensional, expert e at byte e * (bytes / n_expert) (forward.rs:477-485).
//
// Two placements.  HOST: the file is mapped and every tensor address points into the mapping (what a CPU consumer of struct
// sz_model reads).  DEVICE: one device allocation, every tensor copied to a 256-byte aligned place of its own; EXL3 blobs are placed
// so that their trellis starts on a 16-byte boundary, and EXL3 expert slices are re-strided to a multiple of 16 bytes, as the
// kernels need (the file cannot give that: its alignment applies to the blob's first byte).  The per-layer embedding is read when
// ple.layers names a layer of the model (one at most, as in the reference), the sparse indexer when
// attention.indexer.head_count is not 0.
#include "sz_common.cuh"

#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

namespace {

struct GVal {
    int type = -1;            // GGUF value type id
    uint64_t u = 0;           // integers, bool
    double f = 0.0;           // floats
    std::string s;            // strings
    std::vector<int64_t> ints;  // integer arrays (other arrays are skipped)
    uint64_t count = 0;       // array length
};

struct GTensor {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t type = 0;
    uint64_t offset = 0;      // absolute in the file
    uint64_t layout = 0;      // bytes by the type's block layout (0: unknown)
    uint64_t span = 0;        // bytes to the next tensor or the end of the file
    uint64_t bytes() const { return layout ? layout : span; }
};

struct Reader {
    const u8* p;
    uint64_t n, at = 0;
    bool ok = true;
    bool need(uint64_t k) { if (!ok || k > n - at) { ok = false; return false; } return true; }
    uint32_t u32v() { if (!need(4)) return 0; uint32_t v; memcpy(&v, p + at, 4); at += 4; return v; }
    uint64_t u64v() { if (!need(8)) return 0; uint64_t v; memcpy(&v, p + at, 8); at += 8; return v; }
    std::string str() {
        const uint64_t k = u64v();
        if (k > (64u << 20) || !need(k)) { ok = false; return std::string(); }   // gguf.rs:296 MAX_STR
        std::string s((const char*)p + at, (size_t)k);
        at += k;
        return s;
    }
};

// bytes of a scalar value type, 0 for strings and arrays
int scalar_bytes(uint32_t t) {
    switch (t) { case 0: case 1: case 7: return 1; case 2: case 3: return 2; case 4: case 5: case 6: return 4; case 10: case 11: case 12: return 8; default: return 0; }
}

bool read_value(Reader& r, uint32_t ty, int depth, GVal* out) {
    out->type = (int)ty;
    const int sb = scalar_bytes(ty);
    if (sb) {
        if (!r.need(sb)) return false;
        uint64_t raw = 0;
        memcpy(&raw, r.p + r.at, sb);
        r.at += sb;
        switch (ty) {
            case 1: out->u = (uint64_t)(int64_t)(int8_t)raw; break;
            case 3: out->u = (uint64_t)(int64_t)(int16_t)raw; break;
            case 5: out->u = (uint64_t)(int64_t)(int32_t)raw; break;
            case 6: { float f; memcpy(&f, &raw, 4); out->f = f; } break;
            case 12: memcpy(&out->f, &raw, 8); break;
            default: out->u = raw;
        }
        return true;
    }
    if (ty == 8) { out->s = r.str(); return r.ok; }
    if (ty == 9) {
        if (depth > 2) return r.ok = false;                      // gguf.rs:338: arrays nested more than two deep
        const uint32_t et = r.u32v();
        const uint64_t cnt = r.u64v();
        if (cnt > (1ull << 26)) return r.ok = false;             // MAX_ARRAY
        out->count = cnt;
        const bool is_int = et == 0 || et == 1 || et == 2 || et == 3 || et == 4 || et == 5 || et == 10 || et == 11;
        for (uint64_t i = 0; i < cnt && r.ok; i++) {
            GVal e;
            if (!read_value(r, et, depth + 1, &e)) return false;
            if (is_int) out->ints.push_back((int64_t)e.u);
        }
        return r.ok;
    }
    return r.ok = false;                                         // unknown value type
}

// (elements, bytes) of a block of a ggml type this reader sizes by layout (gguf.rs:99-136); 0: unknown or a blob type
bool block_of(uint32_t t, uint64_t* be, uint64_t* bb) {
    static const struct { uint32_t id; uint64_t be, bb; } T[] = {
        {0, 1, 4}, {1, 1, 2}, {2, 32, 18}, {3, 32, 20}, {6, 32, 22}, {7, 32, 24}, {8, 32, 34}, {9, 32, 36}, {10, 256, 84}, {11, 256, 110},
        {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292}, {16, 256, 66}, {17, 256, 74}, {18, 256, 98}, {19, 256, 50},
        {20, 32, 18}, {21, 256, 110}, {22, 256, 82}, {23, 256, 136}, {24, 1, 1}, {25, 1, 2}, {26, 1, 4}, {27, 1, 8}, {28, 1, 8}, {29, 256, 56},
        {30, 1, 2}, {34, 256, 54}, {35, 256, 66}, {39, 32, 17}, {40, 64, 36}, {41, 128, 18}, {42, 64, 18}};
    for (const auto& e : T)
        if (e.id == t) { *be = e.be; *bb = e.bb; return true; }
    return false;
}

bool is_exl3(uint32_t t) { return t > 1020 && t <= 1028; }

}  // namespace

struct sz_weights {
    int fd = -1;
    const u8* map = nullptr;
    uint64_t map_len = 0;
    std::map<std::string, GVal> kv;
    std::vector<GTensor> tensors;
    std::map<std::string, size_t> index;
    uint64_t data_start = 0, alignment = 32;
    std::string arch;
    int placement = 0;
    u8* dev = nullptr;          // device placement: the one allocation
    int64_t placed_bytes = 0;
    sz_model model = {};
    std::vector<sz_layer> layers;
    std::vector<int64_t> ratios;   // attention.compress_ratios, when the file has a sparse indexer
    ~sz_weights() {
        if (dev) cudaFree(dev);
        if (map) munmap((void*)map, map_len);
        if (fd >= 0) close(fd);
    }
    const GTensor* find(const std::string& name) const {
        auto it = index.find(name);
        return it == index.end() ? nullptr : &tensors[it->second];
    }
    const GVal* key(const std::string& k) const {
        auto it = kv.find(arch + "." + k);
        return it == kv.end() ? nullptr : &it->second;
    }
};

static int gguf_parse(sz_weights* w, const char* path) {
    w->fd = open(path, O_RDONLY);
    if (w->fd < 0) return sz_fail(SZ_E_ARG, "%s: cannot open", path);
    struct stat st;
    if (fstat(w->fd, &st) != 0 || st.st_size < 24) return sz_fail(SZ_E_ARG, "%s: not a GGUF this reader understands: too short", path);
    w->map_len = (uint64_t)st.st_size;
    void* m = mmap(nullptr, w->map_len, PROT_READ, MAP_PRIVATE, w->fd, 0);
    if (m == MAP_FAILED) return sz_fail(SZ_E_ARG, "%s: cannot map", path);
    w->map = (const u8*)m;
    Reader r{w->map, w->map_len};
    if (memcmp(r.p, "GGUF", 4) != 0) return sz_fail(SZ_E_ARG, "%s: not a GGUF this reader understands: no GGUF magic", path);
    r.at = 4;
    const uint32_t version = r.u32v();
    if (version < 2 || version > 3) return sz_fail(SZ_E_ARG, "%s: not a GGUF this reader understands: version %u (2 and 3 are read)", path, version);
    const uint64_t n_tensors = r.u64v(), n_kv = r.u64v();
    if (n_tensors > (1u << 20) || n_kv > (1u << 20)) return sz_fail(SZ_E_ARG, "%s: %llu tensors, %llu key-values", path, (unsigned long long)n_tensors, (unsigned long long)n_kv);
    for (uint64_t i = 0; i < n_kv && r.ok; i++) {
        const std::string k = r.str();
        const uint32_t ty = r.u32v();
        GVal v;
        if (!read_value(r, ty, 0, &v)) break;
        w->kv[k] = v;
    }
    for (uint64_t i = 0; i < n_tensors && r.ok; i++) {
        GTensor t;
        t.name = r.str();
        const uint32_t nd = r.u32v();
        if (nd == 0 || nd > 8) return sz_fail(SZ_E_ARG, "%s: tensor %s has %u dimensions", path, t.name.c_str(), nd);
        for (uint32_t d = 0; d < nd; d++) t.dims.push_back(r.u64v());
        t.type = r.u32v();
        t.offset = r.u64v();
        w->tensors.push_back(t);
    }
    if (!r.ok) return sz_fail(SZ_E_ARG, "%s: not a GGUF this reader understands: the header runs past the end of the file or holds an unknown value type", path);
    auto al = w->kv.find("general.alignment");
    w->alignment = al != w->kv.end() ? al->second.u : 32;
    if (w->alignment == 0 || (w->alignment & (w->alignment - 1))) return sz_fail(SZ_E_ARG, "%s: general.alignment %llu", path, (unsigned long long)w->alignment);
    w->data_start = (r.at + w->alignment - 1) / w->alignment * w->alignment;
    // spans: each tensor runs to the next one's start, the last to the end of the file (gguf.rs:392-404)
    std::vector<size_t> order(w->tensors.size());
    for (size_t i = 0; i < order.size(); i++) order[i] = i;
    for (size_t i = 1; i < order.size(); i++)          // insertion sort by offset: files are written in order, so this is linear
        for (size_t j = i; j > 0 && w->tensors[order[j]].offset < w->tensors[order[j - 1]].offset; j--) { size_t t = order[j]; order[j] = order[j - 1]; order[j - 1] = t; }
    for (size_t k = 0; k < order.size(); k++) {
        GTensor& t = w->tensors[order[k]];
        const uint64_t start = w->data_start + t.offset;
        const uint64_t end = k + 1 < order.size() ? w->data_start + w->tensors[order[k + 1]].offset : w->map_len;
        if (start > w->map_len || end < start) return sz_fail(SZ_E_ARG, "%s: tensor %s at %llu is outside the file (%llu bytes)", path, t.name.c_str(), (unsigned long long)start, (unsigned long long)w->map_len);
        t.span = end - start;
    }
    for (size_t i = 0; i < w->tensors.size(); i++) {
        GTensor& t = w->tensors[i];
        t.offset += w->data_start;
        uint64_t be = 0, bb = 0, elems = 1;
        for (uint64_t d : t.dims) elems *= d;
        if (block_of(t.type, &be, &bb) && t.dims[0] % be == 0) t.layout = elems / be * bb;
        if (t.layout > t.span) return sz_fail(SZ_E_ARG, "%s: tensor %s needs %llu bytes but has %llu", path, t.name.c_str(), (unsigned long long)t.layout, (unsigned long long)t.span);
        w->index[t.name] = i;
    }
    auto ar = w->kv.find("general.architecture");
    w->arch = ar != w->kv.end() && ar->second.type == 8 ? ar->second.s : "qwen35next";   // forward.rs:73
    return SZ_OK;
}

// ---- struct sz_model from the table ---------------------------------------------------------------------------------------------
namespace {

struct Placer {
    sz_weights* w;
    int64_t at = 0;       // device placement: next free byte
    bool measure = true;  // first pass sizes the allocation, the second copies
    cudaStream_t st;
    int rc = SZ_OK;

    // bytes [src, src + n) of the file as a tensor address; lead: the address must be = lead (mod 16)
    uint64_t put(uint64_t src_off, uint64_t n, int lead) {
        if (w->placement == 0) return (uint64_t)(w->map + src_off);
        int64_t o = (at + 255) & ~(int64_t)255;
        o += lead;
        at = o + (int64_t)n;
        if (measure) return 0;
        if (cudaMemcpyAsync(w->dev + o, w->map + src_off, n, cudaMemcpyHostToDevice, st) != cudaSuccess && rc == SZ_OK) rc = sz_fail(SZ_E_CUDA, "upload of %llu bytes failed", (unsigned long long)n);
        return (uint64_t)(w->dev + o);
    }
    // n_slices slices of `slice` bytes each, laid out `stride` bytes apart
    uint64_t put_strided(uint64_t src_off, uint64_t slice, uint64_t stride, uint64_t n_slices, int lead) {
        if (w->placement == 0) return (uint64_t)(w->map + src_off);
        int64_t o = (at + 255) & ~(int64_t)255;
        o += lead;
        at = o + (int64_t)(stride * n_slices);
        if (measure) return 0;
        if (cudaMemcpy2DAsync(w->dev + o, stride, w->map + src_off, slice, slice, n_slices, cudaMemcpyHostToDevice, st) != cudaSuccess && rc == SZ_OK)
            rc = sz_fail(SZ_E_CUDA, "upload of %llu expert slices failed", (unsigned long long)n_slices);
        return (uint64_t)(w->dev + o);
    }
};

int get_u(const sz_weights* w, const char* k, int32_t* out) {
    const GVal* v = w->key(k);
    if (!v || scalar_bytes((uint32_t)v->type) == 0 || v->type == 6 || v->type == 12) return sz_fail(SZ_E_ARG, "missing %s", k);   // forward.rs:78
    *out = (int32_t)v->u;
    return SZ_OK;
}

int tens(Placer& P, const std::string& name, int64_t cols, int64_t rows, sz_tensor* out) {
    const GTensor* t = P.w->find(name);
    if (!t) return sz_fail(SZ_E_ARG, "no tensor %s", name.c_str());
    uint64_t elems = 1;
    for (uint64_t d : t->dims) elems *= d;
    if (t->dims[0] != (uint64_t)cols || elems != (uint64_t)(cols * rows))
        return sz_fail(SZ_E_ARG, "%s: expected [%lld, %lld], the file has %llu elements in rows of %llu", name.c_str(), (long long)cols, (long long)rows,
                       (unsigned long long)elems, (unsigned long long)t->dims[0]);
    out->type = (int32_t)t->type; out->reserved = 0; out->rows = rows; out->cols = cols;
    uint64_t n = t->bytes();
    if (is_exl3(t->type)) {
        const uint64_t K = t->type - 1020;
        n = 2 * (uint64_t)cols + 2 * (uint64_t)rows + 4 + (uint64_t)cols * rows * K / 8;     // exl3.rs:388-398 blob_len
        if (n > t->span) return sz_fail(SZ_E_ARG, "%s: an EXL3 blob of %llu bytes in a span of %llu", name.c_str(), (unsigned long long)n, (unsigned long long)t->span);
    }
    // an EXL3 blob sits so that its trellis (after suh, svh and the 4-byte marker) starts on a 16-byte boundary
    const int lead = is_exl3(t->type) ? (int)((16 - (2 * cols + 2 * rows + 4) % 16) % 16) : 0;
    out->data = P.put(t->offset, n, lead);
    return SZ_OK;
}

int vec(Placer& P, const std::string& name, int64_t n, sz_tensor* out) {
    const GTensor* t = P.w->find(name);
    if (!t) return sz_fail(SZ_E_ARG, "no tensor %s", name.c_str());
    uint64_t elems = 1;
    for (uint64_t d : t->dims) elems *= d;
    if (t->type != SZ_TYPE_F32 || elems != (uint64_t)n) return sz_fail(SZ_E_ARG, "%s: expected %lld F32 values", name.c_str(), (long long)n);
    out->type = SZ_TYPE_F32; out->reserved = 0; out->rows = 1; out->cols = n;
    out->data = P.put(t->offset, (uint64_t)n * 4, 0);
    return SZ_OK;
}

// an expert tensor [in, out, n_expert]: base and stride
int experts(Placer& P, const std::string& name, int64_t n_in, int64_t n_out, int64_t ne, int32_t* type, uint64_t* base, uint64_t* stride) {
    const GTensor* t = P.w->find(name);
    if (!t) return sz_fail(SZ_E_ARG, "no tensor %s", name.c_str());
    if (t->dims.size() != 3 || t->dims[0] != (uint64_t)n_in || t->dims[1] != (uint64_t)n_out || t->dims[2] != (uint64_t)ne)
        return sz_fail(SZ_E_ARG, "%s: expected [%lld, %lld, %lld]", name.c_str(), (long long)n_in, (long long)n_out, (long long)ne);
    *type = (int32_t)t->type;
    if (is_exl3(t->type)) {
        const uint64_t K = t->type - 1020;
        const uint64_t slice = 2 * (uint64_t)n_in + 2 * (uint64_t)n_out + 4 + (uint64_t)n_in * n_out * K / 8;
        if (slice * ne > t->span) return sz_fail(SZ_E_ARG, "%s: %lld EXL3 blobs of %llu bytes in a span of %llu", name.c_str(), (long long)ne, (unsigned long long)slice, (unsigned long long)t->span);
        const int lead = (int)((16 - (2 * n_in + 2 * n_out + 4) % 16) % 16);
        *stride = P.w->placement == 0 ? slice : (slice + 15) & ~15ull;
        *base = P.put_strided(t->offset, slice, *stride, (uint64_t)ne, lead);
        return SZ_OK;
    }
    if (!t->layout || t->layout % (uint64_t)ne) return sz_fail(SZ_E_ARG, "%s: the size of an expert's slice is not known", name.c_str());
    *stride = t->layout / (uint64_t)ne;                                                            // forward.rs:477-485
    if (*stride % 16) return sz_fail(SZ_E_ARG, "%s: expert slices of %llu bytes are not multiples of 16", name.c_str(), (unsigned long long)*stride);
    *base = P.put(t->offset, t->layout, 0);
    return SZ_OK;
}

int hc(Placer& P, const sz_model_config& c, const std::string& prefix, bool inject, sz_hc* out) {
    const int64_t CH = (int64_t)c.streams * c.hidden;
    int rc;
    *out = sz_hc();
    if ((rc = vec(P, prefix + "_norm.weight", CH, &out->norm))) return rc;
    if ((rc = tens(P, prefix + "_down.weight", CH, c.hc_rank, &out->down))) return rc;
    if ((rc = tens(P, prefix + "_up.weight", c.hc_rank, CH, &out->up))) return rc;
    if (inject && (rc = tens(P, prefix + "_inject.weight", CH, c.streams, &out->inject))) return rc;
    return SZ_OK;
}

int build(Placer& P) {
    sz_weights* w = P.w;
    sz_model_config& c = w->model.cfg;
    int rc;
    const int64_t H = c.hidden;
    const int64_t kd = (int64_t)c.ssm_k_heads * c.ssm_head_dim, vd = (int64_t)c.ssm_v_heads * c.ssm_head_dim, ch = 2 * kd + vd;
    const int64_t qd = (int64_t)c.n_head * c.head_dim, kvd = (int64_t)c.n_kv_head * c.head_dim;
    if ((rc = tens(P, "token_embd.weight", H, c.vocab, &w->model.token_embd))) return rc;
    if ((rc = tens(P, "output.weight", H, c.vocab, &w->model.output))) return rc;
    if ((rc = hc(P, c, "output_hc", false, &w->model.output_hc))) return rc;
    if (w->model.ple.ngram >= 2) {   // the per-layer embedding of one layer (forward.rs:93-136; tensor names docs/ARCH.md:171-172)
        sz_ple& p = w->model.ple;
        const std::string pp = "blk." + std::to_string(p.layer) + ".";
        const int64_t CH = (int64_t)c.streams * H;
        const GTensor* tt = w->find("per_layer_token_embd.weight");
        if (!tt || tt->dims.size() < 2 || (int64_t)tt->dims[0] != p.head_dim) return sz_fail(SZ_E_ARG, "per_layer_token_embd.weight: a table of rows of %d weights is expected", p.head_dim);
        if ((rc = tens(P, "per_layer_token_embd.weight", p.head_dim, (int64_t)tt->dims[1], &p.table))) return rc;
        if ((rc = tens(P, pp + "ple_key.weight", H, CH, &p.key)) || (rc = tens(P, pp + "ple_value.weight", H, H, &p.value))) return rc;
        if ((rc = vec(P, pp + "ple_norm_key.weight", CH, &p.norm_key)) || (rc = vec(P, pp + "ple_norm_query.weight", CH, &p.norm_query)) ||
            (rc = vec(P, pp + "ple_norm_conv.weight", CH, &p.norm_conv)) || (rc = vec(P, pp + "ple_conv1d.weight", CH * p.conv_k, &p.conv1d)))
            return rc;
    }
    for (int l = 0; l < c.n_layer; l++) {
        sz_layer& L = w->layers[l];
        const std::string p = "blk." + std::to_string(l) + ".";
        if ((rc = hc(P, c, p + "hc_attn", true, &L.hc_attn))) return rc;
        if ((rc = hc(P, c, p + "hc_ffn", true, &L.hc_ffn))) return rc;
        if (l % c.attn_interval == c.attn_interval - 1) {
            if ((rc = tens(P, p + "attn_q.weight", H, 2 * qd, &L.attn_q))) return rc;
            if ((rc = tens(P, p + "attn_k.weight", H, kvd, &L.attn_k))) return rc;
            if ((rc = tens(P, p + "attn_v.weight", H, kvd, &L.attn_v))) return rc;
            if ((rc = tens(P, p + "attn_output.weight", qd, H, &L.attn_output))) return rc;
            if ((rc = vec(P, p + "attn_q_norm.weight", c.head_dim, &L.attn_q_norm))) return rc;
            if ((rc = vec(P, p + "attn_k_norm.weight", c.head_dim, &L.attn_k_norm))) return rc;
            if (c.idx_heads > 0) {   // the sparse indexer (names: exl3_model.rs:227)
                if ((rc = tens(P, p + "indexer.q_proj.weight", H, (int64_t)c.idx_heads * c.idx_dim, &L.idx_q))) return rc;
                if ((rc = tens(P, p + "indexer.k_proj.weight", H, c.idx_dim, &L.idx_k))) return rc;
                if ((rc = vec(P, p + "indexer.q_norm.weight", c.idx_dim, &L.idx_q_norm))) return rc;
                if ((rc = vec(P, p + "indexer.k_norm.weight", c.idx_dim, &L.idx_k_norm))) return rc;
                L.idx_ratio = l < (int)w->ratios.size() && w->ratios[l] > 0 ? (int32_t)w->ratios[l] : 1;
            }
        } else {
            if ((rc = tens(P, p + "attn_qkv.weight", H, ch, &L.attn_qkv))) return rc;
            if ((rc = tens(P, p + "attn_gate.weight", H, vd, &L.attn_gate))) return rc;
            if ((rc = tens(P, p + "ssm_beta.weight", H, c.ssm_v_heads, &L.ssm_beta))) return rc;
            if ((rc = tens(P, p + "ssm_alpha.weight", H, c.ssm_v_heads, &L.ssm_alpha))) return rc;
            if ((rc = tens(P, p + "ssm_out.weight", vd, H, &L.ssm_out))) return rc;
            if ((rc = vec(P, p + "ssm_conv1d.weight", ch * c.conv_k, &L.ssm_conv1d))) return rc;
            if ((rc = vec(P, p + "ssm_a", c.ssm_v_heads, &L.ssm_a))) return rc;
            if ((rc = vec(P, p + "ssm_dt.bias", c.ssm_v_heads, &L.ssm_dt_bias))) return rc;
            if ((rc = vec(P, p + "ssm_norm.weight", c.ssm_head_dim, &L.ssm_norm))) return rc;
        }
        sz_moe_layer& M = L.moe;
        M = sz_moe_layer();
        M.hidden = c.hidden; M.n_expert = c.n_expert; M.top_k = c.n_expert_used; M.expert_ff = c.expert_ff;
        sz_tensor router, shrouter;
        if ((rc = tens(P, p + "ffn_gate_inp.weight", H, c.n_expert, &router))) return rc;
        if (router.type != SZ_TYPE_F32) return sz_fail(SZ_E_TYPE, "%sffn_gate_inp.weight: the router is F32 in every model this reads (type %d)", p.c_str(), router.type);
        M.router = router.data;
        int32_t ty = 0, ty2 = 0;
        if ((rc = experts(P, p + "ffn_gate_exps.weight", H, c.expert_ff, c.n_expert, &ty, &M.gate, &M.gate_stride))) return rc;
        M.expert_type = ty;
        if ((rc = experts(P, p + "ffn_up_exps.weight", H, c.expert_ff, c.n_expert, &ty2, &M.up, &M.up_stride))) return rc;
        if (ty2 != ty) return sz_fail(SZ_E_TYPE, "%s: gate and up experts of different types (%d, %d)", p.c_str(), ty, ty2);
        if ((rc = experts(P, p + "ffn_down_exps.weight", c.expert_ff, H, c.n_expert, &ty2, &M.down, &M.down_stride))) return rc;
        if (ty2 != ty) return sz_fail(SZ_E_TYPE, "%s: gate and down experts of different types (%d, %d)", p.c_str(), ty, ty2);
        // the shared expert: its width comes from its tensors (forward.rs:118 sets shared_ff = expert_ff, the matvecs size themselves)
        const GTensor* sg = w->find(p + "ffn_gate_shexp.weight");
        if (sg) {
            if (sg->dims.size() < 2 || sg->dims[0] != (uint64_t)H) return sz_fail(SZ_E_ARG, "%sffn_gate_shexp.weight: rows of %llu, hidden is %lld", p.c_str(), (unsigned long long)sg->dims[0], (long long)H);
            M.shared_ff = (int32_t)sg->dims[1];
            sz_tensor a, b, d;
            if ((rc = vec(P, p + "ffn_gate_inp_shexp.weight", H, &shrouter))) return rc;
            M.shared_router = shrouter.data;
            if ((rc = tens(P, p + "ffn_gate_shexp.weight", H, M.shared_ff, &a))) return rc;
            if ((rc = tens(P, p + "ffn_up_shexp.weight", H, M.shared_ff, &b))) return rc;
            if ((rc = tens(P, p + "ffn_down_shexp.weight", M.shared_ff, H, &d))) return rc;
            if (a.type != b.type || a.type != d.type) return sz_fail(SZ_E_TYPE, "%s: the shared expert's matrices have different types", p.c_str());
            M.shared_type = a.type; M.sh_gate = a.data; M.sh_up = b.data; M.sh_down = d.data;
        }
        if (l == 0) c.shared_ff = M.shared_ff;
    }
    return P.rc;
}

}  // namespace

extern "C" int sz_model_load_gguf(const char* path, int placement, uint64_t stream, sz_weights** out) {
    if (!path || !out || placement < 0 || placement > 1) return sz_fail(SZ_E_ARG, "sz_model_load_gguf: bad argument");
    sz_weights* w = new (std::nothrow) sz_weights();
    if (!w) return sz_fail(SZ_E_ARG, "out of host memory");
    int rc = gguf_parse(w, path);
    if (rc) { delete w; return rc; }
    if (w->arch == "flint") { delete w; return sz_fail(SZ_E_TYPE, "%s: general.architecture = \"flint\" is not read (forward.rs:74-77)", path); }
    w->placement = placement;
    sz_model_config& c = w->model.cfg;
    c = sz_model_config();
    int32_t inner = 0;
    if ((rc = get_u(w, "block_count", &c.n_layer)) || (rc = get_u(w, "embedding_length", &c.hidden)) || (rc = get_u(w, "attention.key_length", &c.head_dim)) ||
        (rc = get_u(w, "hyper_connection.count", &c.streams)) || (rc = get_u(w, "hyper_connection.low_rank", &c.hc_rank)) ||
        (rc = get_u(w, "attention.head_count", &c.n_head)) || (rc = get_u(w, "attention.head_count_kv", &c.n_kv_head)) ||
        (rc = get_u(w, "rope.dimension_count", &c.rope_dims)) || (rc = get_u(w, "expert_count", &c.n_expert)) ||
        (rc = get_u(w, "expert_used_count", &c.n_expert_used)) || (rc = get_u(w, "expert_feed_forward_length", &c.expert_ff)) ||
        (rc = get_u(w, "ssm.group_count", &c.ssm_k_heads)) || (rc = get_u(w, "ssm.time_step_rank", &c.ssm_v_heads)) ||
        (rc = get_u(w, "ssm.inner_size", &inner)) || (rc = get_u(w, "ssm.conv_kernel", &c.conv_k)) ||
        (rc = get_u(w, "full_attention_interval", &c.attn_interval))) {
        delete w;
        return rc;
    }
    if (c.n_layer < 1 || c.n_layer > 4096 || c.ssm_v_heads < 1 || c.attn_interval < 1) { delete w; return sz_fail(SZ_E_ARG, "%s: bad shape keys", path); }
    c.ssm_head_dim = inner / c.ssm_v_heads;
    const GVal* eps = w->key("attention.layer_norm_rms_epsilon");
    c.eps = eps && (eps->type == 6 || eps->type == 12) ? (float)eps->f : 1e-6f;
    const GVal* th = w->key("rope.freq_base");
    c.rope_theta = th && (th->type == 6 || th->type == 12) ? th->f : 1e7;
    const GTensor* ow = w->find("output.weight");
    if (!ow || ow->dims.size() < 2) { delete w; return sz_fail(SZ_E_ARG, "%s: no output.weight", path); }
    c.vocab = (int32_t)ow->dims[1];                                                               // forward.rs:106
    // the per-layer embedding (forward.rs:93-136): one layer at most, as in the reference; a layer index past the last = none
    {
        const GVal* pl = w->key("ple.layers");
        int n_ple = 0;
        int64_t which = -1;
        if (pl)
            for (int64_t l : pl->ints)
                if (l >= 0 && l < c.n_layer) { n_ple++; which = l; }
        if (n_ple > 1) { delete w; return sz_fail(SZ_E_TYPE, "%s: ple.layers names %d layers; one per-layer embedding is implemented (as in the reference)", path, n_ple); }
        if (n_ple == 1) {
            sz_ple& p = w->model.ple;
            p = sz_ple();
            p.layer = (int32_t)which;
            if ((rc = get_u(w, "ple.ngram_size", &p.ngram)) || (rc = get_u(w, "ple.heads_per_ngram", &p.heads_per_ngram)) ||
                (rc = get_u(w, "embedding_length_per_layer_input", &p.head_dim)) || (rc = get_u(w, "ple.conv_kernel", &p.conv_k)) ||
                (rc = get_u(w, "ple.eos_token_id", &p.eos))) { delete w; return rc; }
            const GVal *km = w->key("ple.layer_multipliers"), *kv = w->key("ple.head_vocab_sizes"), *ko = w->key("ple.head_offsets");
            const int heads = (p.ngram - 1) * p.heads_per_ngram;
            if (p.ngram < 2 || p.ngram > SZ_PLE_MAX_NGRAM || heads < 1 || heads > SZ_PLE_MAX_HEADS || !km || !kv || !ko || (int)km->ints.size() < p.ngram ||
                (int)kv->ints.size() < heads || (int)ko->ints.size() < heads) {
                delete w;
                return sz_fail(SZ_E_ARG, "%s: the per-layer embedding's keys (ple.ngram_size, ple.heads_per_ngram, ple.layer_multipliers, ple.head_vocab_sizes, ple.head_offsets) do not fit together", path);
            }
            for (int i = 0; i < p.ngram; i++) p.multipliers[i] = km->ints[i];
            for (int i = 0; i < heads; i++) { p.vocab[i] = kv->ints[i]; p.offsets[i] = ko->ints[i]; }
        }
    }
    // the sparse indexer (forward.rs:137-140): heads 0 = the file has none (its budget is then never reached)
    {
        int32_t ih = 0, id = 0, ib = 0;
        const GVal* kh = w->key("attention.indexer.head_count");
        if (kh && !get_u(w, "attention.indexer.head_count", &ih) && ih > 0) {
            if ((rc = get_u(w, "attention.indexer.key_length", &id)) || (rc = get_u(w, "attention.indexer.top_k", &ib))) { delete w; return rc; }
            c.idx_heads = ih; c.idx_dim = id; c.idx_budget = ib;
            const GVal* cr = w->key("attention.compress_ratios");
            if (cr) w->ratios = cr->ints;
        }
    }
    w->layers.assign((size_t)c.n_layer, sz_layer());
    w->model.layers = w->layers.data();
    Placer P{w};
    P.st = (cudaStream_t)stream;
    if (placement == 1) {
        P.measure = true;
        if ((rc = build(P))) { delete w; return rc; }
        w->placed_bytes = P.at + 256;
        if (cudaMalloc((void**)&w->dev, (size_t)w->placed_bytes) != cudaSuccess) {
            const long long need = w->placed_bytes;
            delete w;
            return sz_fail(SZ_E_CUDA, "%s: cannot allocate %lld bytes of device memory for the tensors", path, need);
        }
        P.at = 0;
        P.measure = false;
    }
    if ((rc = build(P))) { delete w; return rc; }
    if (placement == 1 && cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) { delete w; return sz_fail(SZ_E_CUDA, "%s: the upload failed", path); }
    if (placement == 0) w->placed_bytes = (int64_t)(w->map_len - w->data_start);
    *out = w;
    return SZ_OK;
}

// The header alone: key-values and the tensor table, no model description (sz_weights_model gives null).  For tools and tests.
extern "C" int sz_gguf_open(const char* path, sz_weights** out) {
    if (!path || !out) return sz_fail(SZ_E_ARG, "sz_gguf_open: null argument");
    sz_weights* w = new (std::nothrow) sz_weights();
    if (!w) return sz_fail(SZ_E_ARG, "out of host memory");
    const int rc = gguf_parse(w, path);
    if (rc) { delete w; return rc; }
    w->placement = -1;
    *out = w;
    return SZ_OK;
}

// An unsigned-integer key-value by its full name (`general.alignment`, `<architecture>.block_count`, ..); for an array, its length.
extern "C" int sz_weights_key_u64(const sz_weights* w, const char* key, uint64_t* out) {
    if (!w || !key || !out) return sz_fail(SZ_E_ARG, "sz_weights_key_u64: null argument");
    auto it = w->kv.find(key);
    if (it == w->kv.end()) return sz_fail(SZ_E_ARG, "no key %s", key);
    if (it->second.type == 9) { *out = it->second.count; return SZ_OK; }
    if (scalar_bytes((uint32_t)it->second.type) == 0 || it->second.type == 6 || it->second.type == 12) return sz_fail(SZ_E_TYPE, "%s is not an integer", key);
    *out = it->second.u;
    return SZ_OK;
}

extern "C" const sz_model* sz_weights_model(const sz_weights* w) { return w && w->placement >= 0 ? &w->model : nullptr; }
extern "C" int64_t sz_weights_bytes(const sz_weights* w) { return w ? w->placed_bytes : -1; }
extern "C" void sz_weights_free(sz_weights* w) { delete w; }

// Header-level queries, for tools and tests (the reference's `Gguf::get` / `tensor`, gguf.rs:503-520): the number of tensors, and one
// tensor's type, dimensions and byte size by name.  Returns SZ_E_ARG for an unknown name.
extern "C" int sz_weights_tensor_count(const sz_weights* w) { return w ? (int)w->tensors.size() : -1; }
extern "C" int sz_weights_tensor_info(const sz_weights* w, const char* name, int32_t* type, int64_t dims[4], int64_t* bytes) {
    if (!w || !name) return sz_fail(SZ_E_ARG, "sz_weights_tensor_info: null argument");
    const GTensor* t = w->find(name);
    if (!t) return sz_fail(SZ_E_ARG, "no tensor %s", name);
    if (type) *type = (int32_t)t->type;
    if (dims)
        for (int i = 0; i < 4; i++) dims[i] = i < (int)t->dims.size() ? (int64_t)t->dims[i] : 1;
    if (bytes) *bytes = (int64_t)t->bytes();
    return SZ_OK;
}
