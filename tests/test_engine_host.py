"""Host-side speculation logic (CPU only): the library's C++ drafter, lookup, sampler and draft policy against the reference's own
unit-test vectors (crates/shadowzero-serve/src/engine.rs:2899-2941, sampler.rs:226-347) and against the oracle's C restatement."""
import ctypes as C

import numpy as np

from oracle import binding as ob
from tests.util import pkg

szlib, md = pkg.lib, pkg.model
L = szlib.load()


def u32(a):
    return (C.c_uint32 * len(a))(*[int(t) for t in a])


class LibDrafter:
    def __init__(self, min_match=4, max_match=32, capacity=4096):
        self.h = L.sz_drafter_new(min_match, max_match, capacity)

    def extend(self, toks):
        L.sz_drafter_extend(self.h, u32(toks), len(toks))

    def propose(self, k, min_match=None):
        out = (C.c_uint32 * max(k, 1))()
        ml = C.c_int()
        n = L.sz_drafter_propose(self.h, k, out, C.byref(ml)) if min_match is None else L.sz_drafter_propose_with_min(self.h, k, min_match, out, C.byref(ml))
        return list(out[:n]), ml.value

    def propose_after(self, extra, k):
        out = (C.c_uint32 * max(k, 1))()
        ml = C.c_int()
        n = L.sz_drafter_propose_after(self.h, u32(extra), len(extra), k, out, C.byref(ml))
        return list(out[:n]), ml.value

    def __len__(self):
        return L.sz_drafter_len(self.h)

    def __del__(self):
        L.sz_drafter_free(self.h)


def test_suffix_drafter_reference_vector():
    # engine.rs:2899-2918: longest then most recent match; propose_after chains without touching the history
    for D in (LibDrafter, ob.Drafter):
        sd = D(4, 32, 4096)
        sd.extend([1, 2, 10, 11, 12, 13, 20, 21, 22, 99])
        sd.extend([5, 9, 10, 11, 12, 13, 30, 31, 32, 33, 88])
        sd.extend([9, 10, 11, 12, 13])
        assert sd.propose(4) == ([30, 31, 32, 33], 5)
        n0 = len(sd)
        assert sd.propose_after([30, 31], 3) == ([32, 33, 88], 7)
        assert len(sd) == n0
        assert sd.propose(0) == ([], 0)
        assert sd.propose_after([], 2) == ([30, 31], 5)


def test_drafter_and_lookup_match_the_oracle_on_random_histories():
    rng = np.random.default_rng(5)
    for trial in range(40):
        vocab = int(rng.integers(3, 12))  # tiny vocabularies: many repeats, many hash-table collisions of intent
        hist = [int(t) for t in rng.integers(0, vocab, int(rng.integers(1, 300)))]
        mm = int(rng.integers(3, 6))
        a, b = LibDrafter(mm, 32, 64), ob.Drafter(mm, 32, 64)
        for i, t in enumerate(hist):
            a.extend([t]); b.extend([t])
            if i % 7 == 0:
                k = int(rng.integers(0, 8))
                assert a.propose(k) == b.propose(k)
                assert a.propose(k, 3) == b.propose(k, 3)
                ex = [int(t) for t in rng.integers(0, vocab, int(rng.integers(0, 4)))]
                assert a.propose_after(ex, k) == b.propose_after(ex, k)
        for k in (1, 3, 5):
            out = (C.c_uint32 * 8)()
            lens = (C.c_int * 2)(3, 2)
            n = L.sz_lookup(u32(hist), len(hist), k, lens, 2, out)
            assert list(out[:n]) == ob.lookup(hist, k, (3, 2))


def test_lookup_by_hand():
    # engine.rs:823-839: the latest earlier occurrence of the last 3 tokens, else of the last 2
    out = (C.c_uint32 * 8)()
    lens = (C.c_int * 2)(3, 2)
    h = [1, 2, 3, 4, 9, 1, 2, 3, 7, 8, 1, 2, 3]
    assert list(out[:L.sz_lookup(u32(h), len(h), 3, lens, 2, out)]) == [7, 8, 1]
    h = [5, 6, 1, 2, 9, 9, 1, 2]
    assert list(out[:L.sz_lookup(u32(h), len(h), 4, lens, 2, out)]) == [9, 9, 1, 2]
    h = [1, 2, 3]
    assert L.sz_lookup(u32(h), len(h), 4, lens, 2, out) == 0


def test_draft_policy_reference_vector():
    # engine.rs:2920-2941
    p = L.sz_policy_new(8, 3, 0.03)
    assert L.sz_policy_neural_k(p, 100) == 3
    for _ in range(4):
        L.sz_policy_observe(p, 0, 4, 3, 0, 12.0)
    assert L.sz_policy_neural_k(p, 100) == 4
    lk = C.c_int()
    t = L.sz_policy_choose(p, 4, 6, 16, C.byref(lk))
    assert lk.value == 1 and t >= 5
    for _ in range(8):
        L.sz_policy_observe(p, 0, 4, 0, 0, 12.0)
    assert L.sz_policy_neural_k(p, 100) == 2
    assert L.sz_policy_neural_k(p, 1) == 1 and L.sz_policy_neural_k(p, 0) == 0
    # chaining: a sure neural draft followed by a long match is worth extending, a hopeless one is not
    assert 1 <= L.sz_policy_chain(p, 3, 0.9, 4, 30) <= 4
    assert L.sz_policy_chain(p, 3, 0.0, 4, 2) == 0 and L.sz_policy_chain(p, 8, 0.9, 4, 30) == 0
    L.sz_policy_observe_chain(p, 3, 4, 6, 30, 14.0)
    assert 0.0 < L.sz_policy_accept_ema(p) < 1.0
    L.sz_policy_free(p)


def _top_of(l):
    v, i = ob.top64(l)
    return np.concatenate([v.view(np.uint32), i]).astype(np.uint32)


def test_top64_order():
    # kernels/forward.cu:3565-3573 and crates/shadowzero-cuda/tests/topk.rs:28-44: ties to the lower id, NaN as -inf, short rows padded
    l = np.zeros(5000, dtype=np.float32)
    v, i = ob.top64(l)
    assert list(i) == list(range(64)) and np.all(v == 0)
    l = np.full(100, -np.inf, dtype=np.float32); l[7] = np.nan; l[50] = 1.0
    v, i = ob.top64(l)
    assert i[0] == 50 and list(i[1:5]) == [0, 1, 2, 3]
    v, i = ob.top64(np.array([3.0, 1.0, 2.0], dtype=np.float32))
    assert list(i[:3]) == [0, 2, 1] and np.all(i[3:] == 0xffffffff) and np.all(np.isneginf(v[3:]))
    rng = np.random.default_rng(1)
    l = np.floor(rng.random(40000) * 50).astype(np.float32)  # heavy ties
    v, i = ob.top64(l)
    order = sorted(range(l.size), key=lambda t: (-l[t], t))[:64]
    assert list(i) == order


def test_a_draw_from_the_top_64_is_the_draw_from_the_whole_row():
    # sampler.rs:236-268: five configurations, rows with ties and smooth rows; library (top-64) == oracle (whole row) == oracle (top-64)
    configs = [(0.7, 20, 0.95, 0.0, 3), (1.0, 64, 1.0, 0.0, 4), (1.5, 1, 0.95, 0.0, 5), (0.3, 40, 0.95, 0.05, 6), (2.0, 30, 0.9, 0.0, 7)]
    for c, (temp, tk, tp, mp, seed) in enumerate(configs):
        so = ob.SamplerC(temp, tk, tp, mp, seed)
        sl = md.Sampler(temp, tk, tp, mp, seed)
        for pos in range(120):
            u = np.array([(ob.lib().szo_splitmix64((pos * 5000 + i) ^ 0x77) >> 40) / 16777216.0 for i in range(5000)], dtype=np.float32)
            l = (np.floor(u * np.float32(24.0)) * np.float32(0.25)).astype(np.float32) if pos % 2 == 0 else (u * np.float32(8.0)).astype(np.float32)
            whole = ob.lib().szo_sample(C.byref(so), l.ctypes.data_as(C.c_void_p), l.size, pos)
            top = _top_of(l)
            assert L.sz_sample_top(C.byref(sl), top.ctypes.data_as(C.POINTER(C.c_uint32)), pos) == whole, (c, pos)


def test_uniform_is_a_pure_function_of_seed_and_position():
    for seed in (0, 1, 42, 2 ** 63):
        for pos in (0, 1, 5, 10 ** 6):
            a, b = L.sz_uniform(seed, pos), ob.lib().szo_uniform(seed, pos)
            assert a == b and 0.0 <= a < 1.0
    assert L.sz_uniform(1, 2) != L.sz_uniform(2, 1)
    # two tokens with logits ln 3 and 0: drawn 0.75 / 0.25 (sampler.rs:332-341)
    l = np.full(100, -30.0, dtype=np.float32); l[10] = np.log(np.float32(3.0)); l[20] = 0.0
    top = _top_of(l)
    s = md.Sampler(1.0, 64, 1.0, 0.0, 5)
    hits = sum(L.sz_sample_top(C.byref(s), top.ctypes.data_as(C.POINTER(C.c_uint32)), p) == 10 for p in range(8000))
    assert abs(hits / 8000 - 0.75) < 0.02


def test_q8_kv_quantiser_round_trip():
    # crates/shadowzero-cuda/tests/kv_q8.rs:108-170: relative L2 error below 0.015, padding zeroed, 272 bytes at head_dim 256
    rng = np.random.default_rng(2)
    for hd, nbytes in ((64, 80), (128, 144), (256, 272)):
        v = rng.standard_normal(hd).astype(np.float32)
        q = ob.kv_quant_q8(v)
        assert q.size == nbytes
        assert np.all(q[hd + 2 * (hd // 32):] == 0)
        back = ob.kv_dequant_q8(q, hd)
        assert np.linalg.norm(back - v) / np.linalg.norm(v) < 0.015
    z = ob.kv_quant_q8(np.zeros(64, dtype=np.float32))
    assert np.all(z == 0)
