"""ctypes binding of the CPU oracle (libsz_oracle.so).  TEST INFRASTRUCTURE ONLY: the checker, never the product."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

F32, F16, Q8_0, IQ3_S, BF16, EXL3_BASE = 0, 1, 8, 21, 30, 1020


def build():
    """Compiles the oracle with the committed Makefile (gcc, -ffp-contract=off)."""
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libsz_oracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.szo_f16_to_f32.restype = C.c_float
        L.szo_f16_to_f32.argtypes = [C.c_uint16]
        L.szo_f32_to_f16.restype = C.c_uint16
        L.szo_f32_to_f16.argtypes = [C.c_float]
        L.szo_bf16_to_f32.restype = C.c_float
        L.szo_bf16_to_f32.argtypes = [C.c_uint16]
        L.szo_f32_to_bf16.restype = C.c_uint16
        L.szo_f32_to_bf16.argtypes = [C.c_float]
        L.szo_f64_to_f16_bits.restype = C.c_uint16
        L.szo_f64_to_f16_bits.argtypes = [C.c_double]
        L.szo_dequant.restype = C.c_int
        L.szo_dequant.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]
        L.szo_exl3_cb.restype = C.c_float
        L.szo_exl3_cb.argtypes = [C.c_int, C.c_uint32]
        L.szo_exl3_state.restype = C.c_uint32
        L.szo_exl3_blob_len.restype = C.c_size_t
        L.szo_exl3_blob_len.argtypes = [C.c_size_t, C.c_size_t, C.c_int, C.c_int]
        L.szo_exl3_reconstruct.argtypes = [C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.szo_exl3_matvec_blob.argtypes = [C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.c_int]
        L.szo_matvec.restype = C.c_int
        L.szo_matvec.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int]
        L.szo_route.restype = C.c_int
        L.szo_route.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.szo_sigmoid.restype = C.c_float
        L.szo_sigmoid.argtypes = [C.c_float]
        L.szo_silu.restype = C.c_float
        L.szo_silu.argtypes = [C.c_float]
        L.szo_softplus.restype = C.c_float
        L.szo_softplus.argtypes = [C.c_float]
        L.szo_moe.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.szo_kv_q8_head_bytes.restype = C.c_size_t
        L.szo_kv_q8_head_bytes.argtypes = [C.c_int]
        L.szo_kv_quant_q8.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.szo_kv_dequant_q8.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.szo_top64.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.szo_session_new.restype = C.c_void_p
        L.szo_session_new.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.szo_session_free.argtypes = [C.c_void_p]
        L.szo_session_len.argtypes = [C.c_void_p]
        L.szo_session_routes.restype = C.POINTER(C.c_int32)
        L.szo_session_routes.argtypes = [C.c_void_p]
        L.szo_session_route_weights.restype = C.POINTER(C.c_double)
        L.szo_session_route_weights.argtypes = [C.c_void_p]
        L.szo_session_assign.argtypes = [C.c_void_p, C.c_void_p]
        L.szo_session_clone.restype = C.c_void_p
        L.szo_session_clone.argtypes = [C.c_void_p]
        L.szo_session_step.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.szo_session_fill_synthetic.argtypes = [C.c_void_p, C.c_int, C.c_uint32]
        L.szo_session_tree.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.szo_tree_accept_sampled.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_uint64, C.c_int,
                                              C.c_void_p, C.POINTER(C.c_uint32)]
        L.szo_tree_accept_greedy.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_uint32)]
        L.szo_session_selected.restype = C.c_int
        L.szo_session_selected.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        L.szo_session_idx_scores.restype = C.c_int
        L.szo_session_idx_scores.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        L.szo_session_state.restype = C.c_void_p
        L.szo_session_state.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_size_t)]
        L.szo_lookup.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        L.szo_drafter_new.restype = C.c_void_p
        L.szo_drafter_new.argtypes = [C.c_int, C.c_int, C.c_int]
        L.szo_drafter_free.argtypes = [C.c_void_p]
        L.szo_drafter_push.argtypes = [C.c_void_p, C.c_uint32]
        L.szo_drafter_len.argtypes = [C.c_void_p]
        L.szo_drafter_propose.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_int)]
        L.szo_drafter_propose_with_min.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_int)]
        L.szo_drafter_propose_after.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_int)]
        L.szo_splitmix64.restype = C.c_uint64
        L.szo_splitmix64.argtypes = [C.c_uint64]
        L.szo_uniform.restype = C.c_double
        L.szo_uniform.argtypes = [C.c_uint64, C.c_uint64]
        L.szo_sample.restype = C.c_uint32
        L.szo_sample.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_uint64]
        L.szo_sample_top.restype = C.c_uint32
        L.szo_sample_top.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_uint64]
        L.szo_generate.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.szo_head_rotate.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.szo_head_proxy_build.argtypes = [C.c_size_t, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.szo_proxy_quant_x.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
        L.szo_proxy_bmax.argtypes = [C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.szo_head_k_use.argtypes = [C.c_int, C.c_int]
        L.szo_proxy_pick.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        _LIB = L
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def dequant(ty, data):
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    be, bb = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q8_0: (32, 34), IQ3_S: (256, 110)}[ty]
    out = np.empty(data.size // bb * be, dtype=np.float32)
    rc = lib().szo_dequant(ty, _p(data), data.size, _p(out), out.size)
    if rc != 0:
        raise ValueError("szo_dequant: %d" % rc)
    return out


def exl3_blob_len(n_in, n_out, bits, half=0):
    return lib().szo_exl3_blob_len(n_in, n_out, bits, half)


def exl3_reconstruct(n_in, n_out, bits, blob, cb=2, half=0):
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    assert blob.size == exl3_blob_len(n_in, n_out, bits, half)
    w = np.empty((n_in, n_out), dtype=np.float32)
    lib().szo_exl3_reconstruct(n_in, n_out, bits, half, cb, _p(blob), _p(w))
    return w


def exl3_decode_tile(tile, bits, cb=2, half=0, fast=False):
    tile = np.ascontiguousarray(tile, dtype=np.uint16)
    out = np.empty(256, dtype=np.float32)
    fn = lib().szo_exl3_decode_tile_fast if fast else lib().szo_exl3_decode_tile
    fn(_p(tile), C.c_int(bits), C.c_int(half), C.c_int(cb), _p(out))
    return out


def wht128(v):
    v = np.array(v, dtype=np.float32).copy()
    lib().szo_wht128(_p(v))
    return v


def matvec(ty, data, rows, cols, x, threads=1):
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.size == cols
    y = np.empty(rows, dtype=np.float32)
    rc = lib().szo_matvec(ty, _p(data), rows, cols, _p(x), _p(y), threads)
    if rc != 0:
        raise ValueError("szo_matvec: %d" % rc)
    return y


def route(logits, k):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    idx = np.empty(k, dtype=np.int32)
    w = np.empty(k, dtype=np.float64)
    n = lib().szo_route(_p(logits), logits.size, k, _p(idx), _p(w))
    return idx[:n], w[:n]


class MoeLayerC(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("n_expert", C.c_int32), ("top_k", C.c_int32), ("expert_ff", C.c_int32),
                ("shared_ff", C.c_int32), ("expert_type", C.c_int32), ("shared_type", C.c_int32),
                ("router", C.c_void_p), ("shared_router", C.c_void_p),
                ("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p),
                ("gate_stride", C.c_uint64), ("up_stride", C.c_uint64), ("down_stride", C.c_uint64),
                ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p)]


def moe(layer, u, threads=1):
    """`layer`: dict of numpy arrays and shapes (see shadow-engine_b200 `synth.make_moe_layer`).  One token.

    Returns (y[hidden] f32, route_idx[k] i32, route_w[k] f64, logits[n_expert] f32)."""
    Ls = MoeLayerC(layer["hidden"], layer["n_expert"], layer["top_k"], layer["expert_ff"], layer["shared_ff"],
                   layer["expert_type"], layer["shared_type"],
                   _p(layer["router"]), _p(layer["shared_router"]),
                   _p(layer["gate"]), _p(layer["up"]), _p(layer["down"]),
                   layer["gate"].strides[0], layer["up"].strides[0], layer["down"].strides[0],
                   _p(layer["sh_gate"]), _p(layer["sh_up"]), _p(layer["sh_down"]))
    u = np.ascontiguousarray(u, dtype=np.float32)
    y = np.empty(layer["hidden"], dtype=np.float32)
    idx = np.empty(layer["top_k"], dtype=np.int32)
    w = np.empty(layer["top_k"], dtype=np.float64)
    logits = np.empty(layer["n_expert"], dtype=np.float32)
    lib().szo_moe(C.byref(Ls), _p(u), _p(y), _p(idx), _p(w), _p(logits), threads)
    return y, idx, w, logits


# ---- part 2: sessions, cache formats, drafting, sampling, the speculation loop ------------------------------------------------

class SamplerC(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("min_p", C.c_float), ("seed", C.c_uint64)]


class GenParamsC(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("spec_k", "max_new", "lookup_min", "greedy", "eog_token", "reserved")] + [("sampler", SamplerC)]


class GenStatsC(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_tokens", "passes", "drafted", "accepted", "lookup_passes")] + \
               [("pos_tried", C.c_int32 * 8), ("pos_right", C.c_int32 * 8)]


def kv_quant_q8(v):
    v = np.ascontiguousarray(v, dtype=np.float32)
    out = np.empty(lib().szo_kv_q8_head_bytes(v.size), dtype=np.uint8)
    lib().szo_kv_quant_q8(_p(v), v.size, _p(out))
    return out


def kv_dequant_q8(b, hd):
    out = np.empty(hd, dtype=np.float32)
    lib().szo_kv_dequant_q8(_p(np.ascontiguousarray(b, dtype=np.uint8)), hd, _p(out))
    return out


def top64(logits):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    v = np.empty(64, dtype=np.float32)
    i = np.empty(64, dtype=np.uint32)
    lib().szo_top64(_p(logits), logits.size, _p(v), _p(i))
    return v, i


class Session:
    """The CPU reference session over a host-resident struct sz_model (`model_struct`: a ctypes struct kept alive by the caller)."""

    def __init__(self, host_model, kv_q8=False, threads=1):
        self.hm = host_model
        self.vocab = host_model.cfg["vocab"]
        self.h = lib().szo_session_new(C.byref(host_model.model), 1 if kv_q8 else 0, threads)

    def __del__(self):
        if getattr(self, "h", None) and _LIB is not None:
            _LIB.szo_session_free(self.h)
            self.h = None

    def __len__(self):
        return lib().szo_session_len(self.h)

    def clone(self):
        """A copy of the whole state: the snapshot the CPU side of the speculation loop takes before a pass."""
        c = Session.__new__(Session)
        c.hm, c.vocab = self.hm, self.vocab
        c.h = lib().szo_session_clone(self.h)
        return c

    def assign(self, other):
        """Become a copy of `other` (restore a snapshot)."""
        lib().szo_session_assign(self.h, other.h)

    def step(self, token, want_logits=True, want_u=False):
        lg = np.empty(self.vocab, dtype=np.float32) if want_logits else None
        u = np.empty(self.hm.cfg["hidden"], dtype=np.float32) if want_u else None
        lib().szo_session_step(self.h, int(token), _p(lg) if want_logits else None, _p(u) if want_u else None)
        return (lg, u) if want_u else lg

    def tree(self, ids, parents, keep_path=None):
        """Logits [m, vocab] of a pass over a draft tree (row j = the sequence root .. j); with keep_path the session then becomes
        the one that read those rows."""
        m = len(ids)
        a, p = np.array(ids, dtype=np.uint32), np.array(parents, dtype=np.int32)
        lg = np.empty((m, self.vocab), dtype=np.float32)
        kp = np.array(keep_path if keep_path is not None else [], dtype=np.int32)
        lib().szo_session_tree(self.h, _p(a), _p(p), m, _p(lg), _p(kp) if kp.size else None, int(kp.size))
        return lg

    def fill_synthetic(self, length, seed=1):
        lib().szo_session_fill_synthetic(self.h, length, seed)

    def state(self, what, layer):
        """A copy of one piece of the state: 0 recurrent state, 1 carried conv rows (float32), 2 / 3 the K / V cache (bytes)."""
        n = C.c_size_t()
        p = lib().szo_session_state(self.h, what, layer, C.byref(n))
        raw = np.frombuffer(C.string_at(p, n.value), dtype=np.uint8).copy()
        return raw.view(np.float32) if what < 2 else raw

    def selected(self, layer):
        """Positions attention layer `layer` attended to in the last step, ascending (the trace stream `layerL.selected`)."""
        out = np.empty(len(self) + 8, dtype=np.int32)
        n = lib().szo_session_selected(self.h, layer, _p(out), out.size)
        return out[:n].copy()

    def idx_scores(self, layer):
        out = np.empty(len(self) + 8, dtype=np.float32)
        n = lib().szo_session_idx_scores(self.h, layer, _p(out), out.size)
        return out[:n].copy()

    def routes(self):
        n, k = self.hm.cfg["n_layer"], self.hm.cfg["n_expert_used"]
        idx = np.ctypeslib.as_array(lib().szo_session_routes(self.h), shape=(n, k)).copy()
        w = np.ctypeslib.as_array(lib().szo_session_route_weights(self.h), shape=(n, k)).copy()
        return idx, w

    def generate(self, prompt, max_new, spec_k=3, greedy=True, sampler=None, lookup_min=4, eog=-1):
        p = GenParamsC(spec_k, max_new, lookup_min, 1 if greedy else 0, eog, 0, sampler or SamplerC(1.0, 20, 0.95, 0.0, 1))
        pr = np.array(prompt, dtype=np.uint32)
        out = np.zeros(max_new, dtype=np.uint32)
        log = np.zeros(2 * max_new, dtype=np.int32)
        st = GenStatsC()
        n = lib().szo_generate(self.h, _p(pr), len(prompt), C.byref(p), _p(out), _p(log), max_new, C.byref(st))
        return [int(t) for t in out[:n]], [(int(log[2 * i]), int(log[2 * i + 1])) for i in range(st.passes)], st


class Drafter:
    def __init__(self, min_match=4, max_match=32, capacity=4096):
        self.h = lib().szo_drafter_new(min_match, max_match, capacity)

    def __del__(self):
        if getattr(self, "h", None) and _LIB is not None:
            _LIB.szo_drafter_free(self.h)
            self.h = None

    def extend(self, toks):
        for t in toks:
            lib().szo_drafter_push(self.h, int(t))

    def __len__(self):
        return lib().szo_drafter_len(self.h)

    def propose(self, k, min_match=None):
        out = np.zeros(max(k, 1), dtype=np.uint32)
        ml = C.c_int()
        n = lib().szo_drafter_propose(self.h, k, _p(out), C.byref(ml)) if min_match is None else \
            lib().szo_drafter_propose_with_min(self.h, k, min_match, _p(out), C.byref(ml))
        return [int(t) for t in out[:n]], ml.value

    def propose_after(self, extra, k):
        out = np.zeros(max(k, 1), dtype=np.uint32)
        ex = np.array(extra, dtype=np.uint32)
        ml = C.c_int()
        n = lib().szo_drafter_propose_after(self.h, _p(ex), len(extra), k, _p(out), C.byref(ml))
        return [int(t) for t in out[:n]], ml.value


def tree_accept_greedy(logits, ids, parents, eog=-1):
    """(kept path, next token) of greedy acceptance down a draft tree."""
    m, vocab = logits.shape
    a, p = np.array(ids, dtype=np.uint32), np.array(parents, dtype=np.int32)
    path = np.zeros(m, dtype=np.int32)
    nxt = C.c_uint32()
    n = lib().szo_tree_accept_greedy(_p(np.ascontiguousarray(logits, dtype=np.float32)), vocab, _p(a), _p(p), m, eog, _p(path), C.byref(nxt))
    return [int(t) for t in path[:n]], int(nxt.value)


def tree_accept_sampled(sampler, tv, ti, ids, parents, draft_prob, pos, eog=-1):
    """(kept path, next token) of rejection-sampling acceptance down a draft tree; tv / ti: [m, 64] values and ids of the rows' top-64."""
    m = len(ids)
    tv = np.ascontiguousarray(tv, dtype=np.float32)
    ti = np.ascontiguousarray(ti, dtype=np.uint32)
    a, p, q = np.array(ids, dtype=np.uint32), np.array(parents, dtype=np.int32), np.array(draft_prob, dtype=np.float32)
    path = np.zeros(m, dtype=np.int32)
    nxt = C.c_uint32()
    n = lib().szo_tree_accept_sampled(C.byref(sampler), _p(tv), _p(ti), _p(a), _p(p), m, _p(q), pos, eog, _p(path), C.byref(nxt))
    return [int(t) for t in path[:n]], int(nxt.value)


def lookup(hist, k, lens=(3, 2)):
    h = np.array(hist, dtype=np.uint32)
    ls = np.array(lens, dtype=np.int32)
    out = np.zeros(max(k, 1), dtype=np.uint32)
    n = lib().szo_lookup(_p(h), len(hist), k, _p(ls), len(lens), _p(out))
    return [int(t) for t in out[:n]]


# ---- part 3: the lm_head's 2-bit screening proxy --------------------------------------------------------------------------------

def head_proxy_build(rows, cols, bits, blob):
    """(w_q2 uint8 [rows * cols / 4], w_sc uint16 [rows * cols / 128]) of an EXL3 output.weight blob."""
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    assert blob.size == exl3_blob_len(cols, rows, bits)
    q2 = np.empty(rows * cols // 4, dtype=np.uint8)
    sc = np.empty(rows * cols // 128, dtype=np.uint16)
    lib().szo_head_proxy_build(rows, cols, bits, _p(blob), _p(q2), _p(sc))
    return q2, sc


def head_rotate(blob, x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    xr = np.empty_like(x)
    for j in range(x.shape[0]):
        lib().szo_head_rotate(_p(blob), _p(x[j]), x.shape[1], _p(xr[j]))
    return xr


def proxy_quant_x(xr):
    """xr: [m, cols] -> (xq int8 [m, cols], x_sc f32 [m, cols / 128], x_corr f32 [m, cols / 128])."""
    xr = np.ascontiguousarray(xr, dtype=np.float32)
    m, cols = xr.shape
    xq = np.empty((m, cols), dtype=np.int8)
    sc = np.empty((m, cols // 128), dtype=np.float32)
    corr = np.empty((m, cols // 128), dtype=np.float32)
    for j in range(m):
        lib().szo_proxy_quant_x(_p(xr[j]), cols, _p(xq[j]), _p(sc[j]), _p(corr[j]))
    return xq, sc, corr


def proxy_bmax(rows, cols, q2, sc, xq, x_sc, x_corr):
    m = xq.shape[0]
    out = np.empty((m, rows // 128), dtype=np.float32)
    for j in range(m):
        lib().szo_proxy_bmax(rows, cols, _p(q2), _p(sc), _p(np.ascontiguousarray(xq[j])), _p(np.ascontiguousarray(x_sc[j])),
                             _p(np.ascontiguousarray(x_corr[j])), _p(out[j]))
    return out


def head_k_use(k_blk, need_k):
    return lib().szo_head_k_use(k_blk, need_k)


def proxy_pick(bmax, k_use, max_sel):
    bmax = np.ascontiguousarray(bmax, dtype=np.float32)
    m, n_ob = bmax.shape
    sel = np.empty(max(max_sel, 1), dtype=np.uint32)
    n = lib().szo_proxy_pick(_p(bmax), m, n_ob, k_use, max_sel, _p(sel))
    return sel[:n].copy()


def mma_cols_q8(w_bytes, rows, cols, x):
    """The arithmetic of the reference's tensor-core projections for a long prompt (kernels/matvec.cu:758-775 and `mma_core`, :1100-1180):
    a weight is decoded as the scalar path decodes it (the f32 product d * q), rounded to f16; the input is rounded to f16; products are
    summed in f32 by the tensor core in an order of its own.  Returned in f64 from the rounded operands, so a test can bound the
    distance by what f32 accumulation of `cols` terms may add.  x: [m][cols] f32 -> ([m][rows] f64, [m][rows] f64 sum of |products|)."""
    w = dequant(Q8_0, w_bytes).reshape(rows, cols)                 # d * q in f32, exactly (quant.rs:174-179)
    w16 = w.astype(np.float16).astype(np.float64)
    x16 = np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float64)
    return x16 @ w16.T, np.abs(x16) @ np.abs(w16).T
